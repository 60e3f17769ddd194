from .trainer import EnhancedConversationTrainer, TrainingMetrics, MoEOptimizationManager, is_oom_error, SyntheticOOM
from .checkpoint import CheckpointManager, CheckpointError
from .schedulers import LRSchedule, build_scheduler
from .precision import PrecisionManager, QuantizationManager, DynamicLossScaler
