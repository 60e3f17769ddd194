from .engine import GenerationEngine, SamplingParams, KVSlotManager, sample_next, GENERATION_MODES
from .scheduler import ContinuousBatcher, Request
from .pipeline_generate import PipelineGenerator
