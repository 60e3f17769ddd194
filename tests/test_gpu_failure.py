"""Failure detection on the device without faulting it: a wait on a peer flag that nothing sets runs out of its (short,
run-time) budget, the kernel returns with the status word set, the host raises ``KernelError`` and the context stays usable.
Kernels that follow a timed-out barrier must leave their buffers alone."""
import ctypes

import pytest
import torch

from adaptivetrainingsystem_b200 import ops
from adaptivetrainingsystem_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _lib_peer():
    from adaptivetrainingsystem_b200.parallel import peer
    return peer, peer._L()


def test_peer_flag_wait_gives_up_and_context_survives():
    peer, lib = _lib_peer()
    dev = torch.device("cuda", 0)
    # A two-"rank" barrier whose two flag arrays are the same local buffer: thread 1 waits for flag [1], which no peer sets.
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 2)(ctypes.c_void_p(flags.data_ptr()), ctypes.c_void_p(flags.data_ptr()))
    st = _lib.status_tensor(dev)
    st.zero_()
    assert abs(peer.get_wait_budget() - 1.0) < 1e-6
    peer.set_wait_budget(0.005)
    try:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(lib.ats_peer_barrier(table, None, None, 0, 2, _lib.ptr(counter), _lib.ptr(st), None, _lib.stream_ptr(dev)), "peer_barrier")
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        assert 4.0 < ms < 500.0, ms  # gave up after the 5 ms budget, not after the default second
        assert int(counter.item()) == 1 and int(flags[0].item()) == 1 and int(flags[1].item()) == 0
        with pytest.raises(ops.KernelError, match="peer flag never arrived"):
            ops.check_status()
    finally:
        peer.set_wait_budget(None)
    # the status word was cleared by the raise; the context is intact and the next kernels run
    x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
    w = torch.ones(256, device=dev, dtype=torch.bfloat16)
    y = ops.rms_norm(x, w, 1e-6)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert (y.float() - ref).abs().max().item() < 3e-2
    ops.check_status()


def test_barrier_epoch_lives_on_the_device_and_survives_graph_replay():
    """A captured barrier must use a fresh epoch on every replay: the kernel advances a counter in device memory."""
    peer, lib = _lib_peer()
    dev = torch.device("cuda", 0)
    bar = peer.PeerBarrier(None, dev)  # world of one: no wait, but the counter and the flag advance
    bar()
    torch.cuda.synchronize()
    assert bar.epoch == 1
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        bar()
        bar()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert bar.epoch == 1 + 3 * 2
    assert int(bar.flags[0].item()) == bar.epoch
    ops.check_status()


def test_update_kernels_do_nothing_after_a_timed_out_wait():
    peer, lib = _lib_peer()
    dev = torch.device("cuda", 0)
    n = 4096
    grads = (torch.randn(n, device=dev) * 0.1).bfloat16()
    params = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    g32 = torch.full((n,), 7.0, device=dev)
    partial = torch.zeros(2048, device=dev)
    sumsq = torch.zeros(1, device=dev)
    master = torch.ones(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    hyper = torch.tensor([1e-2, 0.9, 0.95, 1e-8, 0.0, 1.0], device=dev)
    bad = torch.tensor([5, 0, 0, 0], dtype=torch.int32, device=dev)  # a private status word that says "a peer wait timed out"
    gt = (ctypes.c_void_p * 1)(ctypes.c_void_p(grads.data_ptr()))
    pt = (ctypes.c_void_p * 1)(ctypes.c_void_p(params.data_ptr()))
    stream = _lib.stream_ptr(dev)
    _lib.check(lib.ats_peer_reduce_shard(gt, 1, 0, 0, n, _lib.ptr(g32), _lib.ptr(partial), _lib.ptr(sumsq), 0, _lib.ptr(bad), stream), "reduce")
    _lib.check(lib.ats_adamw_push(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g32), pt, 1, 0, 0, n, _lib.ptr(hyper), None, 0.0,
                                  _lib.ptr(bad), stream), "adamw_push")
    torch.cuda.synchronize()
    assert torch.all(g32 == 7.0) and torch.all(master == 1.0) and torch.all(params == 0) and float(sumsq) == 0.0
    ok = torch.zeros(4, dtype=torch.int32, device=dev)
    _lib.check(lib.ats_peer_reduce_shard(gt, 1, 0, 0, n, _lib.ptr(g32), _lib.ptr(partial), _lib.ptr(sumsq), 0, _lib.ptr(ok), stream), "reduce")
    _lib.check(lib.ats_adamw_push(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g32), pt, 1, 0, 0, n, _lib.ptr(hyper), None, 0.0,
                                  _lib.ptr(ok), stream), "adamw_push")
    torch.cuda.synchronize()
    assert torch.allclose(g32, grads.float()) and abs(float(sumsq) - float(grads.float().pow(2).sum())) < 1e-2 * float(sumsq)
    assert not torch.all(master == 1.0) and torch.equal(params, master.bfloat16())
