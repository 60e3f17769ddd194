"""Expert parallelism (placeholder until the peer-memory path lands in this file)."""


def attach_expert_parallel(model, mesh, cfg, use_fused=True):
    raise NotImplementedError
