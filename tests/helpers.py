"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch

from oracle import moe_oracle as O
from xcaliber_b200 import ops, synth


def small_shape(name="toy", **kw):
    return synth.scaled_shape(synth.SHAPES[name], **kw)


def build_layer(shape, seed=0, token_tile=0):
    w = synth.make_weights(shape, seed=seed, device="cpu")
    pw = ops.PreparedWeights.from_checkpoint(shape, w.w13_packed, w.w13_scale, w.w13_gs, w.w2_qweight, w.w2_scales,
                                             router_bias=w.router_bias, device="cuda")
    return w, ops.FusedMoE(shape, pw, token_tile=token_tile)


def bits(t):
    return O.bf16_bits(t)


def assert_routing_equal(view, ref, n):
    """Routing indices, packed rows and counts must be bit-exact."""
    pk = ref["pack"]
    np.testing.assert_array_equal(view["topk_idx"].cpu().numpy(), pk["idx"])
    np.testing.assert_array_equal(view["counts"].cpu().numpy(), pk["counts"])
    np.testing.assert_array_equal(view["offsets"].cpu().numpy(), pk["offsets"])
    np.testing.assert_array_equal(view["topk_off"].cpu().numpy(), pk["topk_off"])
    np.testing.assert_array_equal(view["topk_row"].cpu().numpy(), pk["topk_row"])
    rows = int(pk["offsets"][-1])
    live = pk["row_token"] >= 0
    np.testing.assert_array_equal(view["row_token"].cpu().numpy()[:rows][live], pk["row_token"][live])
    # gate weights: the reference's own check allows 2^-8 absolute (benchmark.cu:622-624)
    gw = O.bits_to_f32(bits(view["topk_w"]))
    ew = O.bits_to_f32(pk["w_bits"])
    assert np.abs(gw - ew).max() <= 2.0 ** -8


def valid_row_mask(pk):
    rows = int(pk["offsets"][-1])
    m = np.zeros(rows, dtype=bool)
    for e, c in enumerate(pk["counts"]):
        m[pk["offsets"][e]: pk["offsets"][e] + c] = True
    return m
