"""Machine and network report for planning a run: what the node has (CPU, memory, disks, GPUs and their NVLink state, software
versions), which configuration fits it, and whether the node is ready for a multi-process job (interfaces, free rendezvous
ports, a loop-back rendezvous that really opens a TCP store, the environment variables NCCL will read).

``python -m adaptivetrainingsystem_b200.utils.system_report [--network] [--json] [--nodes host1,host2]``

Everything here only READS state (``/proc``, ``/sys``, NVML queries); nothing changes a clock, a power limit or a mode.
The reference ships the same two helpers as shell scripts (``scripts/get_native_properties.sh:50-405``: OS / CPU / memory / GPU /
Python / PyTorch / disk sections and a recommended parameter block; ``scripts/net.sh:50-407``: interfaces, connectivity, port
availability, firewall, distributed readiness, per-node reachability, recommendations).
"""
from __future__ import annotations

import argparse
import json
import os
import platform
import shutil
import socket
import sys
import time
from typing import Any, Dict, List, Optional, Sequence


# ---- machine ---------------------------------------------------------------------------------------------------------------
def _cpu() -> Dict[str, Any]:
    out: Dict[str, Any] = {"logical_cores": os.cpu_count(), "arch": platform.machine()}
    try:
        flags: List[str] = []
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name") and "model" not in out:
                    out["model"] = line.split(":", 1)[1].strip()
                elif line.startswith("flags") and not flags:
                    flags = line.split(":", 1)[1].split()
        out["simd"] = [x for x in ("avx", "avx2", "avx512f", "amx_bf16", "fma") if x in flags]
    except OSError:
        pass
    try:
        out["affinity"] = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    return out


def _memory() -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    try:
        with open("/proc/meminfo") as f:
            kv = {l.split(":")[0]: int(l.split()[1]) for l in f if ":" in l and l.split()[1].isdigit()}
        out = {"total_gb": kv.get("MemTotal", 0) / 2 ** 20, "available_gb": kv.get("MemAvailable", 0) / 2 ** 20,
               "swap_gb": kv.get("SwapTotal", 0) / 2 ** 20, "hugepages": kv.get("HugePages_Total", 0)}
    except OSError:
        pass
    try:  # the pinned-memory budget of data loaders and optimiser offload
        import resource
        soft, _ = resource.getrlimit(resource.RLIMIT_MEMLOCK)
        out["memlock_limit_gb"] = None if soft == resource.RLIM_INFINITY else soft / 2 ** 30
    except Exception:
        pass
    return out


def _gpus(nvml=None) -> List[Dict[str, Any]]:
    """Read-only NVML queries.  ``nvml`` can be a stand-in module with the same functions (tests)."""
    if nvml is None:
        try:
            import pynvml as nvml  # type: ignore
        except Exception:
            return []
    try:
        nvml.nvmlInit()
    except Exception:
        return []
    out = []
    try:
        for i in range(nvml.nvmlDeviceGetCount()):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            g: Dict[str, Any] = {"index": i}

            def q(key, fn):
                try:
                    g[key] = fn()
                except Exception:
                    g[key] = None

            q("name", lambda: (lambda n: n.decode() if isinstance(n, bytes) else n)(nvml.nvmlDeviceGetName(h)))
            q("memory_gb", lambda: nvml.nvmlDeviceGetMemoryInfo(h).total / 2 ** 30)
            q("memory_used_gb", lambda: nvml.nvmlDeviceGetMemoryInfo(h).used / 2 ** 30)
            q("capability", lambda: "%d.%d" % tuple(nvml.nvmlDeviceGetCudaComputeCapability(h)))
            q("sm_clock_mhz", lambda: nvml.nvmlDeviceGetClockInfo(h, nvml.NVML_CLOCK_SM))
            q("sm_clock_max_mhz", lambda: nvml.nvmlDeviceGetMaxClockInfo(h, nvml.NVML_CLOCK_SM))
            q("power_limit_w", lambda: nvml.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0)
            q("temperature_c", lambda: nvml.nvmlDeviceGetTemperature(h, nvml.NVML_TEMPERATURE_GPU))
            links = 0
            for l in range(int(getattr(nvml, "NVML_NVLINK_MAX_LINKS", 18))):
                try:
                    if nvml.nvmlDeviceGetNvLinkState(h, l):
                        links += 1
                except Exception:
                    break
            g["nvlink_active_links"] = links
            out.append(g)
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass
    return out


def _software() -> Dict[str, Any]:
    out: Dict[str, Any] = {"python": sys.version.split()[0], "executable": sys.executable}
    try:
        import torch
        out.update(torch=torch.__version__, cuda_runtime=torch.version.cuda, cuda_available=torch.cuda.is_available(),
                   distributed_backends=[b for b in ("nccl", "gloo") if getattr(torch.distributed, f"is_{b}_available")()])
        if hasattr(torch.cuda, "nccl"):
            try:
                out["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
            except Exception:
                pass
    except Exception as e:  # pragma: no cover
        out["torch"] = f"not importable: {e}"
    out["nvcc"] = shutil.which("nvcc")
    from ..ops import _lib
    out["kernel_library_built"] = os.path.exists(_lib.CUDA_LIB)
    return out


def _disks(paths: Sequence[str] = (".", "/tmp", "/dev/shm")) -> List[Dict[str, Any]]:
    out = []
    for p in paths:
        try:
            u = shutil.disk_usage(p)
            out.append({"path": os.path.abspath(p), "total_gb": u.total / 2 ** 30, "free_gb": u.free / 2 ** 30})
        except OSError:
            pass
    return out


def recommend(gpus: List[Dict[str, Any]], memory: Dict[str, Any]) -> Dict[str, Any]:
    """A starting configuration for the detected hardware (the fields are those of ``config.Config``)."""
    n = len(gpus)
    if n == 0:
        return {"preset": "debug", "precision": "fp32", "batch_size": 1, "gradient_accumulation_steps": 32, "use_flash_attention": False,
                "note": "no GPU: only the PyTorch definitions of the operators run"}
    mem = min((g.get("memory_gb") or 0) for g in gpus)
    cap = gpus[0].get("capability") or "0.0"
    native = cap.startswith("10.")
    rec: Dict[str, Any] = {"precision": "mixed_bf16" if float(cap) >= 8.0 else "mixed_fp16", "use_flash_attention": True, "world_size": n,
                           "native_kernels": native}
    if mem >= 150:      # B200-class: the whole 6 B MoE state fits one GPU
        rec.update(preset="b1_moe" if n < 8 else "mixtral_8x7b", batch_size=8, gradient_accumulation_steps=4, zero_stage=1,
                   gradient_checkpointing=True, expert_parallel_size=min(8, n))
    elif mem >= 70:
        rec.update(preset="b1", batch_size=8, gradient_accumulation_steps=4, zero_stage=2 if n > 1 else 0, gradient_checkpointing=True)
    elif mem >= 30:
        rec.update(preset="b1", batch_size=4, gradient_accumulation_steps=8, zero_stage=3 if n > 1 else 0, gradient_checkpointing=True)
    else:
        rec.update(preset="debug", batch_size=2, gradient_accumulation_steps=16, zero_stage=3 if n > 1 else 0, gradient_checkpointing=True)
    if not native:
        rec["note"] = "the kernels of this framework are built for sm_100a only"
    if memory.get("memlock_limit_gb") is not None and memory["memlock_limit_gb"] < 1:
        rec["warning"] = "locked-memory limit below 1 GB: pinned host buffers (data loader, optimiser offload) will fail to allocate"
    return rec


def native_properties(nvml=None) -> Dict[str, Any]:
    mem, gpus = _memory(), _gpus(nvml)
    return {"os": {"system": platform.system(), "release": platform.release(), "platform": platform.platform(), "hostname": socket.gethostname()},
            "cpu": _cpu(), "memory": mem, "gpus": gpus, "software": _software(), "disks": _disks(), "recommended": recommend(gpus, mem)}


# ---- network ---------------------------------------------------------------------------------------------------------------
def _interfaces() -> List[Dict[str, Any]]:
    out = []
    base = "/sys/class/net"
    if not os.path.isdir(base):
        return out
    for name in sorted(os.listdir(base)):
        d: Dict[str, Any] = {"name": name}
        for key, fn in (("state", "operstate"), ("mtu", "mtu"), ("speed_mbps", "speed"), ("mac", "address")):
            try:
                with open(os.path.join(base, name, fn)) as f:
                    v = f.read().strip()
                d[key] = int(v) if key in ("mtu", "speed_mbps") and v.lstrip("-").isdigit() else v
            except OSError:
                d[key] = None
        d["infiniband"] = os.path.isdir(os.path.join(base, name, "device", "infiniband"))
        out.append(d)
    return out


def port_free(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def reachable(host: str, port: int, timeout_s: float = 1.0) -> Optional[float]:
    """TCP connect time in ms, or ``None``."""
    t0 = time.perf_counter()
    try:
        with socket.create_connection((host, port), timeout=timeout_s):
            return (time.perf_counter() - t0) * 1e3
    except OSError:
        return None


def rendezvous_self_test(port: Optional[int] = None, timeout_s: float = 5.0) -> Dict[str, Any]:
    """Opens the store a job's rank 0 would open, on the loop-back address, writes and reads one key."""
    import datetime
    import torch.distributed as dist
    if port is None:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
    t0 = time.perf_counter()
    try:
        store = dist.TCPStore("127.0.0.1", port, 1, True, timeout=datetime.timedelta(seconds=timeout_s))
        store.set("probe", "1")
        ok = store.get("probe") == b"1"
        del store
        return {"ok": ok, "port": port, "ms": (time.perf_counter() - t0) * 1e3}
    except Exception as e:
        return {"ok": False, "port": port, "error": str(e)}


NCCL_ENV = ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK", "LOCAL_RANK", "NCCL_SOCKET_IFNAME", "NCCL_IB_DISABLE", "NCCL_IB_HCA",
            "NCCL_P2P_DISABLE", "NCCL_NVLS_ENABLE", "NCCL_DEBUG", "GLOO_SOCKET_IFNAME", "CUDA_VISIBLE_DEVICES")


def network_report(master_port: int = 29500, nodes: Sequence[str] = (), extra_ports: Sequence[int] = ()) -> Dict[str, Any]:
    host = socket.gethostname()
    try:
        addrs = sorted({a[4][0] for a in socket.getaddrinfo(host, None)})
        resolves = True
    except OSError:
        addrs, resolves = [], False
    ifs = _interfaces()
    ports = {p: port_free(p) for p in [master_port, master_port + 1, *extra_ports]}
    rep: Dict[str, Any] = {"hostname": host, "hostname_resolves": resolves, "addresses": addrs, "interfaces": ifs, "ports_free": ports,
                           "rendezvous": rendezvous_self_test(), "environment": {k: os.environ.get(k) for k in NCCL_ENV if k in os.environ},
                           "nodes": {n: reachable(n, master_port) for n in nodes}}
    advice: List[str] = []
    if not resolves:
        advice.append("the host name does not resolve: use --master-addr 127.0.0.1 for single-node jobs")
    if not ports[master_port]:
        advice.append(f"port {master_port} is taken: pick another --master-port")
    up = [i for i in ifs if i["state"] == "up" and i["name"] != "lo"]
    if any(i["infiniband"] for i in ifs):
        advice.append("InfiniBand present: leave NCCL_IB_DISABLE unset; set NCCL_IB_HCA to the ports on the GPU's PCIe switch")
    elif len(up) > 1 and "NCCL_SOCKET_IFNAME" not in os.environ:
        advice.append("several interfaces are up: pin the one to use with NCCL_SOCKET_IFNAME / GLOO_SOCKET_IFNAME")
    slow = [i["name"] for i in up if isinstance(i.get("speed_mbps"), int) and 0 < i["speed_mbps"] < 10000]
    if slow and nodes:
        advice.append(f"interfaces below 10 Gb/s ({', '.join(slow)}): multi-node gradient traffic will dominate the step")
    for n, ms in rep["nodes"].items():
        if ms is None:
            advice.append(f"{n}:{master_port} is not reachable (rank 0 not started yet, or a firewall)")
    rep["advice"] = advice
    rep["ready_single_node"] = bool(rep["rendezvous"]["ok"])
    return rep


def _print(d: Dict[str, Any], indent: int = 0) -> None:
    pad = "  " * indent
    for k, v in d.items():
        if isinstance(v, dict):
            print(f"{pad}{k}:")
            _print(v, indent + 1)
        elif isinstance(v, list) and v and isinstance(v[0], dict):
            print(f"{pad}{k}:")
            for item in v:
                print(f"{pad}  - " + ", ".join(f"{a}={b:.1f}" if isinstance(b, float) else f"{a}={b}" for a, b in item.items()))
        else:
            print(f"{pad}{k}: {v:.2f}" if isinstance(v, float) else f"{pad}{k}: {v}")


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--network", action="store_true", help="network / rendezvous report instead of the machine report")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--nodes", default="", help="comma-separated hosts to reach on the master port")
    a = ap.parse_args(argv)
    rep = network_report(a.master_port, [n for n in a.nodes.split(",") if n]) if a.network else native_properties()
    if a.json:
        print(json.dumps(rep, indent=1, default=str))
    else:
        _print(rep)
    return 0


if __name__ == "__main__":
    sys.exit(main())
