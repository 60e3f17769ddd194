#!/usr/bin/env python
"""MoE inference benchmark: batch of equal-length random prompts -> prefill, then greedy decode with the GQA KV cache.

    python benchmarks/bench_inference.py [--config mixtral_8x7b] [--batch 64] [--prompt 1024] [--new 256]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_inference.py ...

With several ranks the experts are spread over the ranks (EP = gcd(E, N)) and the BATCH IS SPLIT: every rank owns
``batch / N`` sequences and their KV cache, runs them through the replicated attention / router weights, and the routed
tokens of all ranks meet at the experts through peer memory.  Prints one JSON line with prefill and decode tokens/s of the
whole batch (device-synchronised wall clock around each phase, max over ranks)."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from adaptivetrainingsystem_b200.inference.benchmark import run_decode_benchmark  # noqa: E402
from adaptivetrainingsystem_b200.parallel import init_distributed  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="mixtral_8x7b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="debug only")
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--pack-experts", type=int, default=1, help="store the expert weights tile by tile for serving (1) or keep the training layout (0)")
    ap.add_argument("--quantize", default="", choices=["", "fp8", "int8", "int4"],
                    help="post-training quantisation of the weights before serving (fp8 covers the experts on one GPU; not the headline figure)")
    a = ap.parse_args()
    rank, local, world = init_distributed()
    out = run_decode_benchmark(a.config, a.batch, a.prompt, a.new, a.layers, bool(a.pack_experts) and not a.quantize, a.repeat,
                               quantize=a.quantize or None)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
