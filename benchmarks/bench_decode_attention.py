"""Decode attention (one query token per sequence against the grouped-query KV cache) timed with CUDA events; small enough for a
profiler capture:

    python benchmarks/bench_decode_attention.py --batch 64 --ctx 1100 --heads 32 --kv-heads 8 --dim 128
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200 import ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1100)
    ap.add_argument("--max-len", type=int, default=1280)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4, help="distinct caches walked in turn, so that no cache stays in L2")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    B, Hq, Hk, D = a.batch, a.heads, a.kv_heads, a.dim
    caches = [(torch.randn(B, a.max_len, Hk, D, device=dev).bfloat16(), torch.randn(B, a.max_len, Hk, D, device=dev).bfloat16())
              for _ in range(a.layers)]
    qkv = torch.randn(B, 1, (Hq + 2 * Hk) * D, device=dev).bfloat16()
    lengths = torch.full((B,), a.ctx, dtype=torch.int32, device=dev)

    def run(i):
        k, v = caches[i % a.layers]
        return ops.decode_attention(qkv, k, v, lengths, Hq, Hk, D)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = e0.elapsed_time(e1) / a.iters
    nbytes = 2 * B * (a.ctx + 1) * Hk * D * 2
    print(json.dumps({"decode_attention": [B, a.ctx, Hq, Hk, D], "ms": ms, "kv_bytes": nbytes, "gb_per_s": nbytes / ms / 1e6,
                      "l2": f"{a.layers} caches of {2 * B * a.max_len * Hk * D * 2 / 2 ** 20:.0f} MiB walked in turn"}))


if __name__ == "__main__":
    main()
