"""Loader and builder for the native libraries.

``libats_b200.so`` holds every sm_100a kernel (plain C ABI, called through ctypes so that no
torch C++ headers are needed to build it and a launch costs a few microseconds of host time).
``libats_host.so`` holds the host-side C++ pieces (AVX CPU AdamW, data packing).  Both are built
in-tree under ``adaptivetrainingsystem_b200/_C`` with ``nvcc`` / ``g++``.

On a machine with a GPU a missing or stale CUDA library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import glob
import os
import shutil
import subprocess
import threading
from typing import List, Optional

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_ROOT, "csrc")
OUT_DIR = os.path.join(_PKG, "_C")
CUDA_LIB = os.path.join(OUT_DIR, "libats_b200.so")
# the same kernels with every data-dependent index range-checked (-DATS_DEBUG); loaded instead of the release library when the
# environment says ATS_DEBUG_BUILD=1
DEBUG_LIB = os.path.join(OUT_DIR, "libats_b200_debug.so")
DEBUG_BUILD = os.environ.get("ATS_DEBUG_BUILD", "0") == "1"
HOST_LIB = os.path.join(OUT_DIR, "libats_host.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared"]
# Kernels that may only run in single-GPU jobs (none at present) would be listed here and built into a
# separate library so the main one never names a multicast load.
SINGLE_GPU_ONLY: List[str] = []

_lock = threading.Lock()
_cuda = None
_host = None


def _nvcc() -> Optional[str]:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _stale(target: str, sources: List[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def cuda_sources() -> List[str]:
    return sorted(s for s in glob.glob(os.path.join(CSRC, "*.cu")) if os.path.basename(s) not in SINGLE_GPU_ONLY)


def build_debug(force: bool = False) -> None:
    """The bounds-checking build: -DATS_DEBUG, relocatable device code (one report word shared by all translation units)."""
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = cuda_sources()
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    if not (force or _stale(DEBUG_LIB, srcs + headers)):
        return
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    cmd = [nvcc] + NVCC_FLAGS + ["-DATS_DEBUG", "-rdc=true", "-I", CSRC, "-o", DEBUG_LIB + ".tmp"] + srcs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc (debug build) failed:\n" + r.stdout + r.stderr)
    os.replace(DEBUG_LIB + ".tmp", DEBUG_LIB)


def build(force: bool = False, verbose: bool = False) -> None:
    """Compile every native source for sm_100a (cross-compiles without a GPU)."""
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = cuda_sources()
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    if srcs and (force or _stale(CUDA_LIB, srcs + headers)):
        nvcc = _nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
        extra = os.environ.get("ATS_NVCC_EXTRA", "").split()  # e.g. -DATS_AB_SPLIT=4 for kernel tuning experiments
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", CSRC, "-o", CUDA_LIB + ".tmp"] + srcs
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        if verbose:
            print(r.stderr)
        os.replace(CUDA_LIB + ".tmp", CUDA_LIB)
    host_srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    if host_srcs and (force or _stale(HOST_LIB, host_srcs)):
        cxx = shutil.which("g++") or "g++"
        cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-mavx2", "-mfma", "-o", HOST_LIB + ".tmp"] + host_srcs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
        os.replace(HOST_LIB + ".tmp", HOST_LIB)


def cuda_lib() -> ctypes.CDLL:
    """The CUDA kernel library; raises if it is not there."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = DEBUG_LIB if DEBUG_BUILD else CUDA_LIB
                if not os.path.exists(path):
                    if _nvcc() is not None:
                        build_debug() if DEBUG_BUILD else build()
                    else:
                        raise RuntimeError(f"{path} is missing and nvcc is unavailable; run __graft_entry__.build()")
                _cuda = ctypes.CDLL(path)
    return _cuda


def host_lib() -> Optional[ctypes.CDLL]:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                if not os.path.exists(HOST_LIB):
                    try:
                        build()
                    except Exception:
                        return None
                if os.path.exists(HOST_LIB):
                    _host = ctypes.CDLL(HOST_LIB)
    return _host


def use_cuda_kernels(t: torch.Tensor) -> bool:
    """Kernels take bf16 CUDA tensors; everything else (CPU, fp32 oracles) runs the PyTorch definition."""
    return t.is_cuda and t.dtype == torch.bfloat16 and os.environ.get("ATS_FORCE_TORCH", "0") != "1"


class KernelError(RuntimeError):
    pass


_STATUS_NAMES = {1: "TMA stage never arrived", 2: "TMA stage never released", 3: "accumulator never produced",
                 4: "accumulator never released", 5: "peer flag never arrived", 6: "bad argument"}
_DEBUG_KERNELS = {1: "plan_slots", 2: "dispatch_rows", 3: "combine_rows", 4: "slot_dot", 5: "grouped GEMM row counts", 6: "decode attention",
                  7: "serve_plan_dispatch", 8: "serve_combine", 9: "embedding_bwd", 10: "peer_reduce", 11: "mod_rows"}


def debug_report() -> Optional[dict]:
    """Debug build only: the first failed bounds check since the last call ({kernel, block, detail}), or ``None``; clears it."""
    if not DEBUG_BUILD or _cuda is None:
        return None
    out = (ctypes.c_int * 4)()
    _cuda.ats_debug_report.restype = ctypes.c_int
    _cuda.ats_debug_report.argtypes = [ctypes.POINTER(ctypes.c_int)]
    if _cuda.ats_debug_report(out) != 1 or out[0] == 0:
        return None
    return {"code": out[0], "kernel": _DEBUG_KERNELS.get(out[1], out[1]), "block": out[2], "detail": out[3]}
_status = {}


def status_tensor(device: torch.device) -> torch.Tensor:
    """One int32 word per device that kernels set when a bounded wait runs out."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None) -> None:
    """Raise if any kernel reported a timed-out wait (synchronises the device)."""
    for key, t in list(_status.items()):
        v = int(t[0].item())
        if v != 0:
            t.zero_()
            raise KernelError(f"device {key}: kernel wait timed out: {_STATUS_NAMES.get(v, v)}")
    rep = debug_report()
    if rep is not None:
        raise KernelError(f"bounds check failed in {rep['kernel']} (block {rep['block']}, value {rep['detail']}); the access was skipped")


_launches = 0


def launch_count() -> int:
    """Number of native entry points called so far (each launches at least one kernel)."""
    return _launches


def check(err: int, what: str) -> None:
    global _launches
    _launches += 1
    if err != 0:
        if err >= 1000:
            raise KernelError(f"{what}: argument/tensor-map error {err}")
        raise KernelError(f"{what}: CUDA error {err}")


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(device=None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
