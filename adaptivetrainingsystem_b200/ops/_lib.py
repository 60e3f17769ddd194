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
                if not os.path.exists(CUDA_LIB):
                    if _nvcc() is not None:
                        build()
                    else:
                        raise RuntimeError(f"{CUDA_LIB} is missing and nvcc is unavailable; run __graft_entry__.build()")
                _cuda = ctypes.CDLL(CUDA_LIB)
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
