from .transformer import (DeepSeekTransformer, TransformerBlock, GroupedQueryAttention, DenseSwiGLU, SwiGLUExpert,
                          MoEFFNLayer, MoDRouter, MoDFFN, RMSNorm, LayerNorm, RotaryEmbedding, KVCache,
                          estimate_parameters)
from ..config import ModelConfig, DeepSeekConfig
