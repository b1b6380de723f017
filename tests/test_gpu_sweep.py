"""Validated sweep over published MoE layer shapes x batch sizes x routing patterns, through the C ABI.

The reference's proof board runs 7 model shapes x N in (8, 256, 512) x {uniform, zipf, burst} routes and
validates every case before it reports a time (sm120a/benchmarks/colab_sweep_models.py:11-23; the checks are
benchmark.cu:618-671: routing exact against the planted routes, finite output, padded rows untouched). This
test does the same on this library: routes are planted (synth.planted_routes), every case must reproduce them
exactly, pass the stage-wise oracle check, return finite values and leave padding rows alone; the time of 20
calls is recorded and, when XMOE_SWEEP_CSV names a file, appended to it as CSV.
"""
import csv
import os

import numpy as np
import pytest
import torch

from tests import helpers as Hh
from oracle import stagewise as S
from xcaliber_b200 import synth

pytestmark = pytest.mark.gpu

# name: (experts, intermediate, hidden, top-k, activation)
MODELS = {
    "kimi_k2": (384, 2048, 7168, 8, "silu"),
    "qwen3_30b_a3b": (128, 768, 2048, 8, "silu"),
    "qwen3_235b_a22b": (128, 1536, 4096, 8, "silu"),
    "minimax_m2": (256, 1536, 3072, 8, "silu"),
    "gpt_oss_120b": (128, 2880, 2880, 4, "swiglu_clamp"),
    "gpt_oss_20b": (32, 2880, 2880, 4, "swiglu_clamp"),
    "gemma4_26b_a4b": (128, 704, 2816, 8, "silu"),
}
NS = (8, 256, 512)
ROUTES = ("uniform", "zipf", "burst")
ITERS = 20


def _time_ms(layer, x, logits, y):
    for _ in range(3):
        layer.forward(x, logits, out=y)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for _ in range(ITERS):
        layer.forward(x, logits, out=y)
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / ITERS


@pytest.mark.parametrize("model", sorted(MODELS))
def test_sweep(model):
    e, inter, hidden, topk, act = MODELS[model]
    shape = synth.MoEShape(model, hidden, inter, e, topk, activation=act)
    ckpt, rw, layer = Hh.build_layer_on_gpu(shape)
    rows = []
    case = sorted(MODELS).index(model) * len(NS) * len(ROUTES)
    for n in NS:
        for route in ROUTES:
            seed = 0x6A09 + case
            case += 1
            logits, idx, w = synth.planted_routes(n, e, topk, mode=route, seed=seed)
            gen = torch.Generator().manual_seed(seed)
            x = torch.randn(n, hidden, generator=gen).to(torch.bfloat16)
            xd, ld = x.cuda(), logits.cuda()
            # poison the row buffers: padding rows of the packed containers must come out as they went in
            layer.forward(xd, ld)
            torch.cuda.synchronize()
            v0 = layer.view(n)
            v0["out_rows"].fill_(float("nan"))
            y = layer.forward(xd, ld)
            torch.cuda.synchronize()
            assert layer.status(n) == 0
            view = layer.view(n)
            # routing by construction: the planted experts in slot order, weights to the reference's 2^-8
            np.testing.assert_array_equal(view["topk_idx"].cpu().numpy()[:n], idx.numpy())
            assert (view["topk_w"].float().cpu()[:n] - w).abs().max() <= 2.0 ** -8
            assert torch.isfinite(y.float()).all()
            res = S.check_layer_stages(shape, ckpt, rw, x, logits, y, view, seed=seed, experts_cap=5, rows_cap=24,
                                       ff1_cols=128, ff2_cols=128)
            pad = ~Hh.valid_row_mask(res["pack"])
            if pad.any():
                got = view["out_rows"][: len(pad)][torch.from_numpy(pad).cuda()]
                assert torch.isnan(got.float()).all(), "a padding row was written"
            ms = _time_ms(layer, xd, ld, torch.empty_like(xd))
            live = int((res["pack"]["counts"] > 0).sum())
            by = synth.algorithmic_bytes(shape, n, live)
            rows.append(dict(model=model, experts=e, inter=inter, hidden=hidden, topk=topk, tokens=n, routing=route,
                             live_experts=live, ms=round(ms, 5), algorithmic_mb=round(by / 1e6, 1),
                             tb_per_s=round(by / (ms * 1e-3) / 1e12, 3), ff1_max_rel=f"{res['worst']['ff1'][0]:.2e}",
                             ff2_max_rel=f"{res['worst']['ff2'][0]:.2e}", status="VALID"))
    out = os.environ.get("XMOE_SWEEP_CSV")
    if out:
        new = not os.path.exists(out)
        with open(out, "a", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0]))
            if new:
                wr.writeheader()
            wr.writerows(rows)
    del layer, ckpt
    torch.cuda.empty_cache()
