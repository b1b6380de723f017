"""GPU parity at the sizes of the published model shapes (the shapes bench.py times), through the C ABI.

The small-weight shapes run the whole oracle chain; the large ones are checked stage by stage on sampled
experts, rows and output columns (tests/helpers.py: stagewise_case), with routing, permutation, NVFP4
packets and the combine bit-exact on every token.
"""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests import helpers as Hh
from xcaliber_b200 import ops, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mixtral():
    shape = synth.SHAPES["mixtral"]
    out = (shape,) + Hh.build_layer_on_gpu(shape)
    yield out
    del out
    torch.cuda.empty_cache()


@pytest.mark.parametrize("n", [1, 16, 256, 4096])
def test_mixtral_full_size(mixtral, n):
    # H 4096, I 14336, 8 experts, top-2: 896 FF1 tiles, 112 K stages in FF2. 4096 tokens is the launch the
    # benchmark times (2-SM FF1 and FF2 kernels); 1 / 16 / 256 take the small-tile kernels.
    shape, ckpt, rw, layer = mixtral
    res = Hh.stagewise_case(shape, ckpt, rw, layer, n, experts_cap=8 if n <= 256 else 4,
                            rows_cap=40 if n <= 256 else 72)
    if n == 4096:
        assert res["view"]["token_tile"] == 128 and int(res["pack"]["counts"].min()) >= 320


@pytest.fixture(scope="module")
def gptoss():
    shape = synth.SHAPES["gptoss"]
    out = (shape,) + Hh.build_layer_on_gpu(shape)
    yield out
    del out
    torch.cuda.empty_cache()


@pytest.mark.parametrize("n", [16, 64, 4096])
def test_gptoss_full_size(gptoss, n):
    # H = I = 2880: 45 K blocks of 64 (padded to 48) in FF1, 22.5 K groups of 128 in FF2 (an odd number of K
    # stages with many tiles per SM: the phantom-stage walk), partial 128-row tiles, clamped SwiGLU
    shape, ckpt, rw, layer = gptoss
    Hh.stagewise_case(shape, ckpt, rw, layer, n, experts_cap=8, rows_cap=40)


def test_qwen3_full_size_whole_chain():
    # H 2048, I 768, 128 experts, top-8 with the Zipf-skewed bias: small weights, so the full oracle chain runs
    shape = synth.SHAPES["qwen3"]
    ckpt, rw, layer = Hh.build_layer_on_gpu(shape)
    fields = [getattr(ckpt, f.name) for f in dataclasses.fields(ckpt)]
    w_cpu = synth.LayerWeights(*[None if t is None else t.cpu() for t in fields])
    from tests.test_gpu_layer import check_stages

    for n in (1, 64, 512):
        x, logits = synth.make_inputs(shape, rw, n)
        y = layer.forward(x.cuda(), logits.cuda())
        torch.cuda.synchronize()
        assert layer.status(n) == 0
        ref = O.layer_forward(x, logits, w_cpu, shape)
        check_stages(shape, n, y, ref, layer.view(n))
    # a prefill batch, stage by stage
    Hh.stagewise_case(shape, ckpt, rw, layer, 8192, experts_cap=8, rows_cap=40)


def test_dsv3_full_size():
    # H 7168, I 2048, 256 routed experts in 8 groups (top-4 groups, bias-corrected sigmoid scores) + 1 shared
    # expert, activation top-k keeping 512 of 2048. The kept set is checked exactly against the rule applied
    # to the kernel's own dense FF1 rows (a second layer over the same weights with the top-k off).
    shape = synth.SHAPES["dsv3"]
    ckpt, rw, layer = Hh.build_layer_on_gpu(shape)
    dense = ops.FusedMoE(dataclasses.replace(shape, act_topk_keep=0), layer.weights)
    for n in (64, 256):
        res = Hh.stagewise_case(shape, ckpt, rw, layer, n, experts_cap=10, rows_cap=40, dense_layer=dense)
        assert shape.num_experts in res["experts"]  # the shared expert is among the checked ones
        ya = Hh.bits(res["view"]["yact"])
        m = Hh.valid_row_mask(res["pack"])
        assert ((ya[: len(m)][m] & 0x7FFF) != 0).sum(axis=1).max() <= shape.act_topk_keep
