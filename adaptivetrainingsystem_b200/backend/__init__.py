"""Backend wrappers with the uniform API of the reference backends (``backend/backend_fsdp.py:311-616``,
``backend_deepspeed.py:211-467``, ``backend_colossalai.py:79-141``): ``__call__ / backward / step / zero_grad / train /
eval / state_dict / load_state_dict / get_lr / get_global_grad_norm / save_checkpoint / load_checkpoint / module /
world_size / local_rank / is_main_process / get_memory_stats``.

All three names map onto the one native engine: FSDP sharding strategies and DeepSpeed / ColossalAI ZeRO stages select
the ZeRO stage of :class:`~adaptivetrainingsystem_b200.parallel.zero.ShardedEngine`."""
from .native import NativeBackend, create_fsdp_backend, create_deepspeed_backend, create_colossalai_backend, create_backend
