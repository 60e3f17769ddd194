"""System information, environment validation and a training-time estimate from measured throughput
(reference ``utils/environment.py:11-292``; its estimator uses a hard-coded tokens/s table, this one uses the measured
roofline of the machine and the model's FLOPs per token)."""
from __future__ import annotations

import os
import platform
import shutil
import sys
from typing import Any, Dict, List

import torch

from .profiler import measured_peaks


def get_system_info() -> Dict[str, Any]:
    info: Dict[str, Any] = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
                            "cuda_available": torch.cuda.is_available(), "cuda_version": torch.version.cuda,
                            "cpu_count": os.cpu_count(), "gpus": []}
    try:
        import psutil
        vm = psutil.virtual_memory()
        info["host_memory_gb"] = vm.total / 2 ** 30
        info["host_memory_available_gb"] = vm.available / 2 ** 30
    except Exception:
        pass
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["gpus"].append({"index": i, "name": p.name, "memory_gb": p.total_memory / 2 ** 30, "sm_count": p.multi_processor_count,
                                 "capability": f"{p.major}.{p.minor}"})
        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if hasattr(torch.cuda, "nccl") else None
    return info


def validate_environment(config=None) -> List[str]:
    """Returns a list of problems (empty = fine)."""
    issues: List[str] = []
    if sys.version_info < (3, 9):
        issues.append("Python 3.9+ required")
    if not torch.cuda.is_available():
        issues.append("no CUDA device: kernels are unavailable, the PyTorch definitions will run on CPU")
    else:
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            issues.append(f"compute capability {major}.{minor}: the native kernels are built for sm_100a (B200) only")
        from ..ops import _lib
        if not os.path.exists(_lib.CUDA_LIB) and shutil.which("nvcc") is None:
            issues.append("kernel library not built and nvcc not found")
    if config is not None:
        if getattr(config, "train_data_path", None) and config.training_mode != "base_only" and not os.path.exists(config.train_data_path):
            issues.append(f"train_data_path {config.train_data_path} does not exist")
        ws = config.world_size or 1
        if config.use_moe and config.expert_parallel_size and config.num_experts % config.expert_parallel_size:
            issues.append("num_experts is not divisible by expert_parallel_size")
        if ws > 1 and ws % max(config.expert_parallel_size or 1, 1):
            issues.append("world_size is not divisible by expert_parallel_size")
    return issues


def estimate_training_time(config, dataset_tokens: int, world_size: int = 1, mfu: float = 0.45) -> Dict[str, float]:
    """tokens/s = world * mfu * sustained bf16 peak / (6 * active parameters)."""
    pk = measured_peaks()
    flops_per_token = 6.0 * config.num_parameters(active_only=True)
    tps = world_size * mfu * pk["bf16_tflops_sustained"] * 1e12 / flops_per_token
    total = dataset_tokens * config.num_epochs
    return {"tokens_per_second": tps, "total_tokens": float(total), "hours": total / tps / 3600.0, "assumed_mfu": mfu,
            "peaks": pk["source"]}


def print_system_diagnostics() -> None:
    info = get_system_info()
    print(f"python {info['python']} | torch {info['torch']} | cuda {info['cuda_version']} | {info['cpu_count']} cpus")
    for g in info["gpus"]:
        print(f"  gpu{g['index']}: {g['name']} {g['memory_gb']:.0f} GB, {g['sm_count']} SMs, sm_{g['capability'].replace('.', '')}")
    for issue in validate_environment():
        print("  ! " + issue)
