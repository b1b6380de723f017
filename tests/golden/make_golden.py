"""Generates the committed golden vectors in this folder. Run from the repo root:

    python tests/golden/make_golden.py

Sources of truth (none of them is the vectorised oracle under test):
  routing_planted.npz  routes planted first, logits built so they win, packed rows obtained by
                       counting in ascending token order: the construction of the reference's own
                       routing self-check (sm120a/benchmarks/benchmark.cu:135-183), redone here
                       with plain Python loops.
  ue4m3.npz            brute force over the 127 representable UE4M3 values with exact rationals:
                       smallest representable >= x, plus the reference's sub-2^-6 rule
                       (sm120a/preamble.cuh:17-36).
  ff1_kat.npz          the analytic FF1 known-answer test of the reference
                       (ff1_w4a4_swiglu_topk_reduce.cu:1043-1075, 1222-1238): constant E2M1
                       patterns, unit scales, expected = silu(H*w1*x) * (H*x).
  toy_layer.npz        regression pin of the oracle's own output on the toy config (seed 0).
"""
from __future__ import annotations

import sys
from fractions import Fraction
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
HERE = Path(__file__).resolve().parent

from xcaliber_b200 import synth  # noqa: E402


def bf16_bits_of(x: float) -> int:
    return int(torch.tensor([x], dtype=torch.float32).to(torch.bfloat16).view(torch.int16).item()) & 0xFFFF


def planted_case(n, e, k, mode, gate, seed):
    logits, idx, w = synth.planted_routes(n, e, k, mode, seed, gate)
    idx = idx.numpy()
    np_ = (n + 31) & ~31
    counts = [0] * e
    topk_off = np.zeros((n, k), dtype=np.uint16)
    etw = np.zeros((e, np_), dtype=np.uint16)
    eti = np.zeros((e, np_ + 1), dtype=np.uint16)
    for t in range(n):
        for s in range(k):
            ex = int(idx[t, s])
            p = counts[ex]
            counts[ex] += 1
            topk_off[t, s] = p
            etw[ex, p] = bf16_bits_of(float(w[t, s]))
            eti[ex, 1 + p] = t
    for ex in range(e):
        eti[ex, 0] = counts[ex]
    return dict(logits=logits.view(torch.int16).numpy().view(np.uint16), idx=idx.astype(np.int32),
                w=w.numpy().astype(np.float32), topk_off=topk_off, expert_topk_w=etw, expert_token_idx=eti)


def ue4m3_values():
    vals = {}
    for code in range(0x7F):
        ex, m = code >> 3, code & 7
        vals[code] = Fraction(m, 512) if ex == 0 else Fraction(8 + m, 8) * Fraction(2) ** (ex - 7)
    return vals


def ue4m3_ceil_exact(x: float, vals) -> int:
    if not x > 0:
        return 0
    fx = Fraction(x)
    if fx >= 448:
        return 0x7E
    if fx < Fraction(1, 64):  # below the smallest normal: ceil(512 x) clipped to 7
        c = -((-fx * 512) // 1)
        return int(min(c, 7))
    best = None
    for code, v in vals.items():
        if code >= 8 and v >= fx and (best is None or v < vals[best]):
            best = code
    return best


def main():
    cases = {}
    for name, args in {
        "toy_uniform_softmax": (64, 8, 2, "uniform", "softmax", 1),
        "qwen_zipf_softmax": (100, 128, 8, "zipf", "softmax", 2),
        "gptoss_burst_softmax": (77, 128, 4, "burst", "softmax", 3),
        "flat_sigmoid": (50, 64, 6, "zipf", "sigmoid", 4),
        "two_chunks": (300, 32, 4, "zipf", "softmax", 5),
    }.items():
        for key, val in planted_case(*args).items():
            cases[f"{name}/{key}"] = val
    np.savez_compressed(HERE / "routing_planted.npz", **cases)

    vals = ue4m3_values()
    rng = np.random.default_rng(0)
    xs = np.concatenate([
        np.array([0.0, 1e-9, 1 / 512, 1.5 / 512, 7 / 512, 7.5 / 512, 1 / 64, 1 / 64 + 1e-6, 0.1, 0.5, 1.0, 1.0001,
                  1.125, 1.9999, 2.0, 3.3, 100.0, 447.9, 448.0, 1000.0], dtype=np.float32),
        np.exp(rng.uniform(np.log(1e-4), np.log(500.0), 2000)).astype(np.float32),
        np.array([float(v) for v in vals.values()], dtype=np.float32),
    ])
    codes = np.array([ue4m3_ceil_exact(float(x), vals) for x in xs], dtype=np.uint8)
    dec = np.array([float(vals[c]) for c in range(0x7F)], dtype=np.float32)
    np.savez_compressed(HERE / "ue4m3.npz", x=xs, ceil_code=codes, decode=dec)

    # analytic FF1 known answer: H = 512, I = 256 (4 planes of 64 rows), 32 tokens
    h, i, n = 512, 256, 32
    plane = (np.arange(i) * 4) // i
    w1 = 0.5 * (plane + 1)                       # E2M1 codes 1..4
    xv = 0.25 * (1 + ((np.arange(n) + (np.arange(n) >> 3)) & 3))   # code (1..4) * XGSINV 0.5
    d1 = h * w1[:, None] * xv[None, :]
    d3 = h * 1.0 * xv[None, :]
    expected = (d1 / (1.0 + np.exp(-d1))) * d3   # [I, N]
    np.savez_compressed(HERE / "ff1_kat.npz", hidden=h, inter=i, tokens=n, w1_code=(plane + 1).astype(np.uint8),
                        w3_code=np.uint8(2), x_code=(1 + ((np.arange(n) + (np.arange(n) >> 3)) & 3)).astype(np.uint8),
                        xgs_inv=np.float32(0.5), scale_byte=np.uint8(0x38), expected=expected.astype(np.float32))

    from oracle import moe_oracle as O

    shape = synth.SHAPES["toy"]
    w = synth.make_weights(shape, seed=0)
    x, logits = synth.make_inputs(shape, w, 64, seed=0)
    ref = O.layer_forward(x, logits, w, shape)
    np.savez_compressed(HERE / "toy_layer.npz", y_bits=O.bf16_bits(ref["y"]), idx=ref["idx"],
                        counts=ref["pack"]["counts"], topk_off=ref["pack"]["topk_off"],
                        x_bits_head=O.bf16_bits(x)[:2, :16], logits_bits_head=O.bf16_bits(logits)[:2],
                        w13_packed_head=w.w13_packed[0, 0, :16].numpy(), xgs=ref["xgs"], xgs_inv=ref["xgs_inv"],
                        sx_head=ref["sx"][:2], codes_head=ref["codes"][:2, :64])
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
