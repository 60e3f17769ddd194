#!/usr/bin/env python
"""Tile / wave arithmetic of the persistent GEMM kernels for one training micro-batch of a preset (no GPU needed).

    python benchmarks/gemm_wave_model.py [--config b1_moe] [--sms 148]

For every product of a layer it prints the number of output tiles, the waves they take on CTA pairs (256 x 256 tiles, one
pair per two SMs) and on single CTAs (128 x 256 tiles), and the share of the last wave that is idle.  Tiles of one launch
are handed out round-robin and take equal time, so ``utilisation = tiles / (waves x workers)``.  It is a model of the
scheduling loss only (no memory or power effects); measured times are in ``profiles/``.
"""
from __future__ import annotations

import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from adaptivetrainingsystem_b200.config import ConfigPresets  # noqa: E402


def waves(tiles: int, workers: int):
    w = math.ceil(tiles / workers)
    return w, tiles / (w * workers)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="b1_moe")
    ap.add_argument("--sms", type=int, default=148)
    a = ap.parse_args()
    cfg = ConfigPresets.get(a.config, num_workers=0)
    mc = cfg.to_model_config()
    T = cfg.micro_batch_size * cfg.seq_length
    H, I = mc.hidden_size, mc.intermediate_size
    d = H // mc.num_heads
    qkv = (mc.num_heads + 2 * mc.num_kv_heads) * d
    E, k = max(mc.num_experts, 1), max(mc.moe_top_k, 1)
    slots = T * k if mc.use_moe else T          # rows of the expert products, all experts together
    per_e = slots // E if mc.use_moe else slots
    groups = E if mc.use_moe else 1
    pairs, singles = a.sms // 2, a.sms
    rows = [
        ("qkv forward", T, qkv, 1), ("o forward", T, H, 1),
        ("expert up + SwiGLU", per_e, I, groups), ("expert down", per_e, H, groups),
        ("dh + SwiGLU backward", per_e, I, groups), ("expert input gradient", per_e, H, groups),
        ("expert down weight gradient", H, I, groups), ("expert up weight gradient", 2 * I, H, groups),
        ("o input gradient", T, H, 1), ("o weight gradient", H, H, 1),
        ("qkv input gradient", T, H, 1), ("qkv weight gradient", qkv, H, 1),
    ]
    print(f"{a.config}: {T} tokens per micro-batch, hidden {H}, intermediate {I}, {E} experts top-{k}; {pairs} CTA pairs / {singles} CTAs")
    print(f"{'product':32s} {'M':>7s} {'N':>6s} {'pair tiles':>10s} {'waves':>6s} {'util':>6s}   {'single tiles':>12s} {'waves':>6s} {'util':>6s}")
    for name, M, N, g in rows:
        tn = math.ceil(N / 256) if "SwiGLU" not in name or "backward" in name else math.ceil(N / 128)
        tp = g * math.ceil(M / 256) * tn
        ts = g * math.ceil(M / 128) * tn
        wp, up = waves(tp, pairs)
        ws, us = waves(ts, singles)
        print(f"{name:32s} {M:7d} {N:6d} {tp:10d} {wp:6d} {up:6.3f}   {ts:12d} {ws:6d} {us:6.3f}")


if __name__ == "__main__":
    main()
