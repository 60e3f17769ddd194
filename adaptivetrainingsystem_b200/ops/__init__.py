"""Operators: hand-written sm_100a kernels with PyTorch definitions as CPU path and oracle."""
from . import _lib
from ._lib import build, check_status, KernelError
from .functional import (rms_norm, rms_norm_skip, rms_norm_reference, layer_norm, layer_norm_reference, masked_softmax, masked_softmax_reference, linear, swiglu, swiglu_reference, swiglu_mlp,
                         rope_tables, rope_reference, rope_packed, embedding, cross_entropy,
                         cross_entropy_reference, linear_cross_entropy, attention, attention_reference, attention_packed, attention_packed_available, rope_attention_packed,
                         sumsq, clip_coef, adamw_step)
from .gemm import (gemm_nt, gemm_nn, gemm_tn, gemm_nt_swiglu, gemm_nn_swiglu_bwd, grouped_nt, grouped_nn, grouped_nn_swiglu_bwd,
                   grouped_tn)
from .moe import (expert_capacity, gate_logits, route, load_balancing_loss, plan_slots, dispatch, combine,
                  slot_dot, moe_ffn, moe_ffn_reference)
from .serving import (decode_attention, decode_attention_available, decode_attention_reference, sample_tokens,  # noqa: E402,F401
                      sample_reference)
from . import fp8  # noqa: E402,F401
from . import int8  # noqa: E402,F401
from . import int4  # noqa: E402,F401
