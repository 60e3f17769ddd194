"""Symmetric peer memory and the device-side flag barrier.

Every rank allocates the same buffer with ``cudaMalloc`` inside the native library, publishes its CUDA IPC handle
through ``torch.distributed`` (the plumbing), and opens the handles of its peers; kernels then receive the table of
peer pointers and move data over NVLink / NVSwitch with plain loads and stores.  No collective library call is
involved after set-up, and no cluster-multicast load is ever issued on peer memory.

Failure handling: the barrier kernel spins on flags for at most a second; when a peer never arrives it sets the
library status word, and :func:`adaptivetrainingsystem_b200.ops.check_status` turns that into a ``KernelError``
on the host -- the GPU context stays usable.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib

_vp, _c_int, _c_ll, _c_f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_sig = False


def _L():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        def sig(name, *args):
            f = getattr(lib, name)
            f.restype = _c_int
            f.argtypes = list(args)
        sig("ats_ipc_alloc", ctypes.c_ulonglong, ctypes.POINTER(_vp), ctypes.c_char_p)
        sig("ats_ipc_open", ctypes.c_char_p, ctypes.POINTER(_vp))
        sig("ats_ipc_close", _vp)
        sig("ats_ipc_free", _vp)
        sig("ats_peer_barrier", ctypes.POINTER(_vp), ctypes.POINTER(_vp), _vp, _c_int, _c_int, _vp, _vp, _vp, _vp)
        sig("ats_peer_reduce_shard", ctypes.POINTER(_vp), _c_int, _c_int, _c_ll, _c_ll, _vp, _vp, _vp, _c_int, _vp, _vp)
        sig("ats_clip_coef_slots", _vp, _c_int, _c_f, _c_f, _vp, _vp)
        sig("ats_adamw_push", _vp, _vp, _vp, _vp, ctypes.POINTER(_vp), _c_int, _c_int, _c_ll, _c_ll, _vp, _vp, _c_f, _vp, _vp)
        lib.ats_set_wait_budget_ns.restype = None
        lib.ats_set_wait_budget_ns.argtypes = [ctypes.c_ulonglong]
        lib.ats_get_wait_budget_ns.restype = ctypes.c_ulonglong
        lib.ats_get_wait_budget_ns.argtypes = []
        sig("ats_peer_copy", _vp, _vp, _c_ll, _c_int, _vp)
        sig("ats_splitk_reduce_signal", _vp, _c_int, _c_ll, _c_ll, _vp, _vp, _vp, ctypes.POINTER(_vp), _c_int, _c_int, _vp)
        sig("ats_peer_gather", ctypes.POINTER(_vp), _c_int, _vp, _c_ll, _c_int, _vp, _vp)
        sig("ats_peer_reduce_rows", ctypes.POINTER(_vp), _c_int, _c_int, _c_ll, _c_ll, _vp, _c_int, _vp, _c_int, _vp)
        _sig = True
    return lib


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap a raw device pointer without copying."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


def wrap_pointer(ptr: int, nbytes: int, device: torch.device, owner=None) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes, owner), device=device)


class SymmetricBuffer:
    """Same-sized buffer on every rank of ``group``.  ``ptrs[i]`` is the address of rank i's copy in THIS process."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        lib = _L()
        local = _vp()
        handle = ctypes.create_string_buffer(64)
        err = lib.ats_ipc_alloc(self.nbytes, ctypes.byref(local), handle)
        if err == 2:  # out of memory: give PyTorch's cached blocks back to the driver and try once more
            torch.cuda.empty_cache()
            err = lib.ats_ipc_alloc(self.nbytes, ctypes.byref(local), handle)
        if err:
            free, total = torch.cuda.mem_get_info(self.device)
            raise _lib.KernelError(f"ipc_alloc of {self.nbytes / 2**30:.2f} GiB failed with CUDA error {err}: {free / 2**30:.1f} of "
                                   f"{total / 2**30:.1f} GiB free on the device, {torch.cuda.memory_reserved(self.device) / 2**30:.1f} GiB "
                                   f"reserved by PyTorch")
        self.local_ptr = int(local.value)
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self.local_ptr
        self._opened: List[int] = []
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for i, h in enumerate(handles):
                if i == self.rank:
                    continue
                p = _vp()
                _lib.check(lib.ats_ipc_open(h, ctypes.byref(p)), f"ipc_open(rank {i})")
                self.ptrs[i] = int(p.value)
                self._opened.append(int(p.value))
        self._table = (_vp * self.world)(*[_vp(p) for p in self.ptrs])
        self.bytes_view = wrap_pointer(self.local_ptr, self.nbytes, self.device, owner=self)

    def table(self, offset_bytes: int = 0):
        """ctypes array of the peers' base addresses (+ offset), for kernel launches."""
        if offset_bytes == 0:
            return self._table
        return (_vp * self.world)(*[_vp(p + offset_bytes) for p in self.ptrs])

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // es if numel is None else numel
        return self.bytes_view[offset_bytes:offset_bytes + n * es].view(dtype)

    def peer_tensor(self, rank: int, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        """View of a peer's copy (debug / tests only; hot paths hand raw pointers to kernels)."""
        es = torch.empty((), dtype=dtype).element_size()
        return wrap_pointer(self.ptrs[rank] + offset_bytes, numel * es, self.device, owner=self).view(dtype)

    def close(self) -> None:
        lib = _L()
        for p in self._opened:
            lib.ats_ipc_close(_vp(p))
        self._opened = []
        if self.local_ptr:
            lib.ats_ipc_free(_vp(self.local_ptr))
            self.local_ptr = 0


def set_wait_budget(seconds: Optional[float]) -> None:
    """Budget of every wait on a peer (flag barriers, gathered-weight chunks) in launches issued after this call;
    ``None`` restores the default of one second.  ``Config.peer_wait_budget_s`` is applied through this."""
    _L().ats_set_wait_budget_ns(0 if seconds is None else max(1, int(seconds * 1e9)))


def get_wait_budget() -> float:
    return _L().ats_get_wait_budget_ns() / 1e9


class PeerBarrier:
    """Flag barrier across the ranks of a group, executed by a one-warp kernel on the caller's stream.  Optionally
    carries one float from every rank to every rank (``slots`` then holds the ``world`` values).

    The epoch that the ranks exchange is a counter in device memory which the kernel itself advances, so a barrier
    that was captured into a CUDA graph synchronises on every replay (a host-side epoch would be frozen into the
    captured launch and every replay after the first would fall through on the stale flags)."""

    def __init__(self, group=None, device: Optional[torch.device] = None):
        self.group = group
        # [0:256) flags (int32[<=64]), [256:512) payload slots (float[<=64]), [512:516) this rank's epoch counter
        self.buf = SymmetricBuffer(1024, group, device)
        self.world, self.rank = self.buf.world, self.buf.rank
        self.flags = self.buf.tensor(torch.int32, 64, 0)
        self.slots = self.buf.tensor(torch.float32, 64, 256)
        self.epoch_counter = self.buf.tensor(torch.int32, 1, 512)
        # per-peer wait time (ns) and call count, accumulated by the kernel: entry t = time spent waiting for rank t, entry 16 = calls
        self.wait_ns = torch.zeros(17, dtype=torch.int64, device=self.buf.device)
        self._flag_table = self.buf.table(0)
        self._slot_table = self.buf.table(256)
        if self.world > 1:
            dist.barrier(group)  # every rank's flags are zeroed and mapped before the first device barrier

    @property
    def epoch(self) -> int:
        """Number of barriers executed so far (reads device memory: diagnostics and tests only)."""
        return int(self.epoch_counter.item())

    def __call__(self, payload: Optional[torch.Tensor] = None) -> None:
        st = _lib.status_tensor(self.buf.device)
        _lib.check(_L().ats_peer_barrier(self._flag_table, self._slot_table if payload is not None else None,
                                         _lib.ptr(payload), self.rank, self.world, _lib.ptr(self.epoch_counter), _lib.ptr(st),
                                         _lib.ptr(self.wait_ns), _lib.stream_ptr(self.buf.device)), "peer_barrier")

    def wait_statistics(self, reset: bool = True) -> dict:
        """Time this rank's barrier kernels spent waiting since the last reset: total of the slowest peer per call is not kept,
        the per-peer sums are -- ``max_peer_ms`` is the largest of them (the peer this rank waits for most)."""
        v = self.wait_ns.tolist()
        if reset:
            self.wait_ns.zero_()
        per_peer = [x / 1e6 for x in v[:self.world]]
        return {"calls": int(v[16]), "max_peer_ms": max(per_peer) if per_peer else 0.0, "per_peer_ms": per_peer}


def peers_available(group=None) -> bool:
    """True when every pair of GPUs in the group can map each other's memory."""
    if not torch.cuda.is_available() or not dist.is_initialized():
        return False
    n = torch.cuda.device_count()
    me = torch.cuda.current_device()
    ok = all(torch.cuda.can_device_access_peer(me, j) for j in range(n) if j != me)
    t = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(t.item())
