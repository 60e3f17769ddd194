"""Update rules for the flat-bucket optimiser: AdamW (default), LAMB, SGD with momentum, and a host (CPU) AdamW for
optimiser-state offload.  Every rule works on one bucket shard: fp32 ``master`` + state, bf16 gradient in, bf16
parameter shard out, the shared clip state honoured (scale, skip on non-finite).

On CUDA each rule is one native launch (``csrc/loss_optim.cu``, ``csrc/optim_extra.cu``); the PyTorch bodies are the
CPU path and the test oracle.  The host rule calls the AVX library (``csrc/host/cpu_adam.cpp``).

Reference counterparts: ``torch.optim.AdamW(fused=True)`` in the trainer (reference ``training/trainer.py:2227-2233``) and
the vendored multi-tensor Adam / LAMB / SGD and CPU Adam kernels (colossalai ``extensions/csrc/cuda/multi_tensor_*.cu``,
``cpu_adam.cpp``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import functional as F_

_vp, _ci, _cll, _cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_sig = False


def _fns():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        lib.ats_sgd.restype = _ci
        lib.ats_sgd.argtypes = [_vp, _vp, _vp, _vp, _cll, _vp, _vp, _cf, _vp]
        lib.ats_lamb_chunk.restype = _ci
        lib.ats_lamb.restype = _ci
        lib.ats_lamb.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _vp, _ci, _vp, _vp, _cf, _ci, _vp]
        lib.ats_scale_check.restype = _ci
        lib.ats_scale_check.argtypes = [_vp, _ci, _vp, _cll, _vp, _cf, _vp, _vp]
        lib.ats_absmax.restype = _ci
        lib.ats_absmax.argtypes = [_vp, _ci, _cll, _vp, _vp]
        _sig = True
    return lib


# ------------------------------------------------------------------------------------------------------------ helpers
def scale_check(src: torch.Tensor, scale: float = 1.0, scale_tensor: Optional[torch.Tensor] = None,
                flag: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 copy of ``src`` times ``scale`` (x ``scale_tensor[0]``); ``flag[0]`` becomes 1 if ``src`` holds inf / nan."""
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=src.device)
    out = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    if src.is_cuda and src.dtype in (torch.float32, torch.bfloat16) and src.is_contiguous():
        err = _fns().ats_scale_check(_lib.ptr(src), int(src.dtype == torch.float32), _lib.ptr(out), src.numel(), _lib.ptr(scale_tensor),
                                     float(scale), _lib.ptr(flag), _lib.stream_ptr(src.device))
        _lib.check(err, "ats_scale_check")
        return out, flag
    s = scale * (float(scale_tensor[0]) if scale_tensor is not None else 1.0)
    out.copy_(src.float() * s)
    if not torch.isfinite(src.float()).all():
        flag.fill_(1)
    return out, flag


def absmax(src: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Running max of |src| into ``out[0]`` (fp32, zeroed when created here): the max-norm of a list of tensors."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=src.device)
    if src.is_cuda and src.dtype in (torch.float32, torch.bfloat16) and src.is_contiguous():
        err = _fns().ats_absmax(_lib.ptr(src), int(src.dtype == torch.float32), src.numel(), _lib.ptr(out), _lib.stream_ptr(src.device))
        _lib.check(err, "ats_absmax")
    elif src.numel():
        out[0] = torch.maximum(out[0], src.float().abs().max())
    return out


# ------------------------------------------------------------------------------------------------------------ rules
class UpdateRule:
    """State and update of one bucket shard.  ``hyper`` is the engine's device vector [lr, b1, b2, eps, wd, step]."""
    name = "base"

    def init_state(self, master: torch.Tensor) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def update(self, state: Dict[str, torch.Tensor], master: torch.Tensor, grad: torch.Tensor, param_out: torch.Tensor,
               hyper: torch.Tensor, clip_state: Optional[torch.Tensor], decay: bool, segments=None, group=None) -> None:
        raise NotImplementedError


class AdamWRule(UpdateRule):
    name = "adamw"

    def init_state(self, master):
        return {"exp_avg": torch.zeros_like(master), "exp_avg_sq": torch.zeros_like(master)}

    def update(self, state, master, grad, param_out, hyper, clip_state, decay, segments=None, group=None):
        F_.adamw_step(master, state["exp_avg"], state["exp_avg_sq"], grad, param_out, hyper, clip_state, 1.0 if decay else 0.0)


class SGDRule(UpdateRule):
    """SGD with momentum (PyTorch semantics: weight decay added to the gradient, first step seeds the buffer)."""
    name = "sgd"

    def __init__(self, momentum: float = 0.9, dampening: float = 0.0, nesterov: bool = False):
        self.momentum, self.dampening, self.nesterov = momentum, dampening, nesterov
        self._hyper: Dict[Tuple, torch.Tensor] = {}

    def init_state(self, master):
        return {"momentum_buffer": torch.zeros_like(master)}

    def update(self, state, master, grad, param_out, hyper, clip_state, decay, segments=None, group=None):
        # own hyper vector {lr, momentum, dampening, wd, nesterov, first}: lr / wd / step are copied on the device
        key = (master.device, id(state["momentum_buffer"]))
        h = self._hyper.get(key)
        if h is None:
            h = torch.tensor([0.0, self.momentum, self.dampening, 0.0, float(self.nesterov), 0.0], dtype=torch.float32, device=master.device)
            self._hyper[key] = h
        h[0:1].copy_(hyper[0:1])
        h[3:4].copy_(hyper[4:5])
        h[5:6].copy_((hyper[5:6] <= 1.0).float())
        if master.is_cuda and grad.dtype == torch.bfloat16:
            err = _fns().ats_sgd(_lib.ptr(master), _lib.ptr(state["momentum_buffer"]), _lib.ptr(grad), _lib.ptr(param_out), master.numel(),
                                 _lib.ptr(h), _lib.ptr(clip_state), 1.0 if decay else 0.0, _lib.stream_ptr(master.device))
            _lib.check(err, "ats_sgd")
            return
        if clip_state is not None and float(clip_state[2]) != 0.0:
            return
        gs = float(clip_state[0]) if clip_state is not None else 1.0
        lr, wd, first = float(h[0]), float(h[3]) * (1.0 if decay else 0.0), float(h[5]) != 0.0
        g = grad.float() * gs + wd * master
        if self.momentum != 0.0:
            buf = state["momentum_buffer"]
            if first:
                buf.copy_(g)
            else:
                buf.mul_(self.momentum).add_(g, alpha=1.0 - self.dampening)
            g = g + self.momentum * buf if self.nesterov else buf
        master.sub_(lr * g)
        param_out.copy_(master.to(param_out.dtype))


class LAMBRule(UpdateRule):
    """LAMB: Adam direction with a per-tensor trust ratio |w| / |u|.  ``segments`` = [(start, length, tensor id)] of the
    tensors inside the shard; ids index one table shared by every rank of ``group``, so a tensor cut by a shard boundary
    contributes partial sums on two ranks and the all-reduce completes them."""
    name = "lamb"

    def __init__(self):
        self._tables: Dict[int, Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]] = {}

    def init_state(self, master):
        return {"exp_avg": torch.zeros_like(master), "exp_avg_sq": torch.zeros_like(master), "update": torch.zeros_like(master)}

    @staticmethod
    def chunk_tables(segments: Sequence[Tuple[int, int]], chunk: int):
        starts, lens, segs = [], [], []
        for seg in segments:
            s, n, si = seg
            o = 0
            while o < n:
                c = min(chunk, n - o)
                starts.append(s + o)
                lens.append(c)
                segs.append(si)
                o += c
        return starts, lens, segs

    def update(self, state, master, grad, param_out, hyper, clip_state, decay, segments=None, group=None, n_segments=None):
        import torch.distributed as dist
        segments = [tuple(x) if len(x) == 3 else (x[0], x[1], i) for i, x in enumerate(segments)] if segments else [(0, master.numel(), 0)]
        n_seg = int(n_segments) if n_segments else max(x[2] for x in segments) + 1  # the table must have the same size on every rank
        multi = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
        if master.is_cuda and grad.dtype == torch.bfloat16:
            lib = _fns()
            key = id(state["update"])
            tab = self._tables.get(key)
            if tab is None or tab[3] != hash(tuple(segments)):
                st, ln, sg = self.chunk_tables(segments, lib.ats_lamb_chunk())
                dev = master.device
                tab = (torch.tensor(st, dtype=torch.int64, device=dev), torch.tensor(ln, dtype=torch.int32, device=dev),
                       torch.tensor(sg, dtype=torch.int32, device=dev), hash(tuple(segments)))
                self._tables[key] = tab
            sums = state.setdefault("seg_sums", torch.zeros(n_seg, 2, dtype=torch.float32, device=master.device))
            if sums.shape[0] != n_seg:
                sums = state["seg_sums"] = torch.zeros(n_seg, 2, dtype=torch.float32, device=master.device)

            def call(stage):
                err = lib.ats_lamb(_lib.ptr(master), _lib.ptr(state["exp_avg"]), _lib.ptr(state["exp_avg_sq"]), _lib.ptr(grad),
                                   _lib.ptr(param_out), _lib.ptr(state["update"]), _lib.ptr(tab[0]), _lib.ptr(tab[1]), _lib.ptr(tab[2]),
                                   tab[0].numel(), _lib.ptr(sums), n_seg, _lib.ptr(hyper), _lib.ptr(clip_state), 1.0 if decay else 0.0, stage,
                                   _lib.stream_ptr(master.device))
                _lib.check(err, "ats_lamb")
            if multi:
                call(1)
                dist.all_reduce(sums, group=group)
                call(2)
            else:
                call(0)
            return
        if clip_state is not None and float(clip_state[2]) != 0.0:
            return
        gs = float(clip_state[0]) if clip_state is not None else 1.0
        lr, b1, b2, eps, wd, step = [float(x) for x in hyper.tolist()]
        wd = wd if decay else 0.0
        g = grad.float() * gs
        m, v = state["exp_avg"], state["exp_avg_sq"]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        u = (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps) + wd * master
        sums = torch.zeros(n_seg, 2, dtype=torch.float32, device=master.device)
        for (s, n, i) in segments:
            sums[i, 0] = master[s:s + n].pow(2).sum()
            sums[i, 1] = u[s:s + n].pow(2).sum()
        if multi:
            dist.all_reduce(sums, group=group)
        for (s, n, i) in segments:
            wn, un = float(sums[i, 0]) ** 0.5, float(sums[i, 1]) ** 0.5
            trust = wn / un if wn > 0 and un > 0 else 1.0
            master[s:s + n].sub_(lr * trust * u[s:s + n])
        param_out.copy_(master.to(param_out.dtype))


class LARSRule(UpdateRule):
    """LARS (You et al. 2017; the vendored ``colossalai/nn/optimizer/lars.py``): SGD with momentum whose step is scaled per
    tensor by ``trust * |w| / (|g| + wd |w| + eps)``.  ``segments`` / ``group`` as in :class:`LAMBRule`: a tensor cut by a shard
    boundary gets its norms completed by an all-reduce.  Tensor operations of the framework, not a kernel of its own: the
    rule exists for parity of the optimiser list; vector-shaped tensors (norm gains) are better left to a group without decay."""
    name = "lars"

    def __init__(self, momentum: float = 0.9, trust_coefficient: float = 1e-3, eps: float = 1e-8):
        self.momentum, self.trust, self.eps = momentum, trust_coefficient, eps

    def init_state(self, master):
        return {"momentum_buffer": torch.zeros_like(master)}

    def update(self, state, master, grad, param_out, hyper, clip_state, decay, segments=None, group=None, n_segments=None):
        import torch.distributed as dist
        segments = [tuple(x) if len(x) == 3 else (x[0], x[1], i) for i, x in enumerate(segments)] if segments else [(0, master.numel(), 0)]
        n_seg = int(n_segments) if n_segments else max(x[2] for x in segments) + 1
        multi = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
        skip = clip_state[2] != 0.0 if clip_state is not None else None          # non-finite gradients: leave everything as it is
        gs = clip_state[0] if clip_state is not None else 1.0
        lr, wd = hyper[0], hyper[4] * (1.0 if decay else 0.0)
        g = grad.float() * gs
        sums = torch.zeros(n_seg, 2, dtype=torch.float32, device=master.device)
        for (s, n, i) in segments:
            sums[i, 0] += master[s:s + n].pow(2).sum()
            sums[i, 1] += g[s:s + n].pow(2).sum()
        if multi:
            dist.all_reduce(sums, group=group)
        wn, gn = sums[:, 0].sqrt(), sums[:, 1].sqrt()
        ratio = torch.where((wn > 0) & (gn > 0), self.trust * wn / (gn + wd * wn + self.eps), torch.ones_like(wn))
        buf = state["momentum_buffer"]
        new_buf = buf * self.momentum
        for (s, n, i) in segments:
            new_buf[s:s + n] += (lr * ratio[i]) * (g[s:s + n] + wd * master[s:s + n])
        if skip is not None:
            new_buf = torch.where(skip, buf, new_buf)
            master.copy_(torch.where(skip, master, master - new_buf))
        else:
            master.sub_(new_buf)
        buf.copy_(new_buf)
        param_out.copy_(master.to(param_out.dtype))


class HostAdamWRule(UpdateRule):
    """AdamW with master / m / v in pinned host memory (optimiser-state offload).  Each step copies the reduced gradient
    shard device -> host, runs the AVX kernel, and copies the bf16 parameter shard back; the GPU keeps only parameters and
    gradients.  ``master`` handed to ``update`` is ignored after the first call (the host copy is authoritative)."""
    name = "adamw_host"

    def __init__(self, pin: bool = True, spill_dir: Optional[str] = None):
        """``spill_dir``: keep master / m / v in memory-mapped files of that directory (a local NVMe mount) instead of pinned
        host memory: the page cache holds what fits and the rest lives on the drive (the reference's ``nvme_offload_optimizer``
        / ``nvme_path`` flags, which it only forwards to DeepSpeed, ``config/config_manager.py:79-85``)."""
        self.pin = pin
        self.spill_dir = spill_dir
        self._files = 0
        self._host: Dict[int, Dict[str, torch.Tensor]] = {}

    @staticmethod
    def isa() -> int:
        lib = _lib.host_lib()
        return int(lib.ats_cpu_isa()) if lib is not None else -1

    def init_state(self, master):
        n = master.numel()
        pin = self.pin and torch.cuda.is_available()
        mk = lambda dt: torch.zeros(n, dtype=dt).pin_memory() if pin else torch.zeros(n, dtype=dt)  # noqa: E731

        def mapped(tag):
            # file-backed fp32 state: written through the mapping by the host kernel, paged by the OS
            os.makedirs(self.spill_dir, exist_ok=True)
            path = os.path.join(self.spill_dir, f"ats_optim_{os.getpid()}_{self._files}_{tag}.bin")
            self._files += 1
            t = torch.from_file(path, shared=True, size=max(n, 1), dtype=torch.float32)[:n]
            t.zero_()
            return t

        big = mapped if self.spill_dir else (lambda tag: mk(torch.float32))
        st = {"master_host": big("master"), "exp_avg": big("m"), "exp_avg_sq": big("v"),
              "grad_host": mk(torch.bfloat16), "param_host": mk(torch.bfloat16)}
        st["master_host"].copy_(master.detach().float().cpu())
        return st

    def update(self, state, master, grad, param_out, hyper, clip_state, decay, segments=None, group=None, force_isa: int = -1):
        hy = hyper.tolist()  # one small D2H read per step: the host kernel needs the scalars
        if clip_state is not None:
            cs = clip_state.tolist()
            if cs[2] != 0.0:
                return
            gscale = cs[0]
        else:
            gscale = 1.0
        gh = state["grad_host"]
        if grad.dtype == torch.bfloat16:
            gh.copy_(grad.detach().reshape(-1), non_blocking=False)
            g_ptr, g_bf16 = gh.data_ptr(), 1
        else:
            g32 = grad.detach().float().cpu().contiguous()
            g_ptr, g_bf16 = g32.data_ptr(), 0
        lib = _lib.host_lib()
        n = gh.numel()
        if lib is not None:
            lib.ats_cpu_adamw.restype = _ci
            lib.ats_cpu_adamw.argtypes = [_vp, _vp, _vp, _vp, _ci, _vp, _cll, _cf, _cf, _cf, _cf, _cf, _cll, _cf, _ci]
            err = lib.ats_cpu_adamw(state["master_host"].data_ptr(), state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr(), g_ptr, g_bf16,
                                    state["param_host"].data_ptr(), n, hy[0], hy[1], hy[2], hy[3], hy[4] if decay else 0.0, int(hy[5]),
                                    gscale, force_isa)
            if err:
                raise RuntimeError(f"ats_cpu_adamw failed: {err}")
        else:  # no compiler on this machine: same arithmetic in PyTorch
            g = (gh.float() if g_bf16 else g32) * gscale
            m, v, w = state["exp_avg"], state["exp_avg_sq"], state["master_host"]
            m.mul_(hy[1]).add_(g, alpha=1 - hy[1])
            v.mul_(hy[2]).addcmul_(g, g, value=1 - hy[2])
            denom = v.sqrt() / (1 - hy[2] ** hy[5]) ** 0.5 + hy[3]
            w.mul_(1 - hy[0] * (hy[4] if decay else 0.0)).addcdiv_(m, denom, value=-hy[0] / (1 - hy[1] ** hy[5]))
            state["param_host"].copy_(w.to(torch.bfloat16))
        param_out.copy_(state["param_host"].to(param_out.dtype) if param_out.dtype != torch.bfloat16 else state["param_host"], non_blocking=False)
        master.copy_(state["master_host"], non_blocking=False) if master.device.type == "cpu" else None


RULES = {"adamw": AdamWRule, "sgd": SGDRule, "lamb": LAMBRule, "lars": LARSRule, "adamw_host": HostAdamWRule}


def make_rule(name: str, **kw) -> UpdateRule:
    try:
        return RULES[name.lower()](**kw)
    except KeyError:
        raise ValueError(f"unknown optimizer {name!r}; choose from {sorted(RULES)}") from None


__all__ = ["UpdateRule", "AdamWRule", "SGDRule", "LAMBRule", "LARSRule", "HostAdamWRule", "make_rule", "scale_check", "absmax", "RULES"]
