"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch

from oracle import moe_oracle as O
from oracle import stagewise as S
from xcaliber_b200 import ops, synth


def small_shape(name="toy", **kw):
    return synth.scaled_shape(synth.SHAPES[name], **kw)


def build_layer(shape, seed=0, token_tile=0, expert_scale=None):
    w = synth.make_weights(shape, seed=seed, device="cpu")
    pw = ops.PreparedWeights.from_checkpoint(shape, w.w13_packed, w.w13_scale, w.w13_gs, w.w2_qweight, w.w2_scales,
                                             router_bias=w.router_bias, expert_scale=expert_scale, device="cuda")
    return w, ops.FusedMoE(shape, pw, token_tile=token_tile)


def bits(t):
    return O.bf16_bits(t)


def bits_t(t):
    """bf16 tensor -> int16 tensor of its bit patterns (on the tensor's device)."""
    return t.contiguous().view(torch.int16)


def assert_routing_equal(view, ref, n=None):
    """Routing indices, packed rows and counts must be bit-exact."""
    S.assert_routing_equal(view, ref["pack"])


def valid_row_mask(pk):
    rows = int(pk["offsets"][-1])
    m = np.zeros(rows, dtype=bool)
    for e, c in enumerate(pk["counts"]):
        m[pk["offsets"][e]: pk["offsets"][e] + c] = True
    return m


# ---------------------------------------------------------------------------------------
# Stage-wise parity at checkpoint sizes (the checks themselves live in oracle/stagewise.py)
# ---------------------------------------------------------------------------------------
def router_only(w):
    return synth.LayerWeights(None, None, None, None, None, w.router_weight.cpu(),
                              None if w.router_bias is None else w.router_bias.cpu(),
                              None if w.logit_bias is None else w.logit_bias.cpu())


def oracle_routing(shape, rw, logits):
    return S.oracle_routing(shape, rw, logits)


def build_layer_on_gpu(shape, seed=0, token_tile=0):
    """Weights synthesised on the GPU (the same generator bench.py uses); returns (checkpoint tensors on the
    GPU, router parts on the CPU, layer)."""
    ckpt = synth.make_weights(shape, seed=seed, device="cuda")
    pw = ops.PreparedWeights.from_checkpoint(shape, ckpt.w13_packed, ckpt.w13_scale, ckpt.w13_gs, ckpt.w2_qweight,
                                             ckpt.w2_scales, router_bias=ckpt.router_bias, device="cuda")
    return ckpt, router_only(ckpt), ops.FusedMoE(shape, pw, token_tile=token_tile)


def stagewise_case(shape, ckpt, rw, layer, n, *, seed=0, dense_layer=None, **caps):
    """One batch of n tokens through `layer`, every stage checked by oracle.stagewise.check_layer_stages.
    dense_layer: the same weights with the activation top-k off (needed when shape.act_topk_keep > 0)."""
    x, logits = synth.make_inputs(shape, rw, n, seed=seed)
    xd, ld = x.cuda(), logits.cuda()
    y = layer.forward(xd, ld)
    torch.cuda.synchronize()
    assert layer.status(n) == 0
    dview = None
    if 0 < shape.act_topk_keep < shape.inter:
        assert dense_layer is not None
        dense_layer.forward(xd, ld)
        torch.cuda.synchronize()
        assert dense_layer.status(n) == 0
        dview = dense_layer.view(n)
    view = layer.view(n)
    res = S.check_layer_stages(shape, ckpt, rw, x, logits, y, view, dense_view=dview, seed=seed, **caps)
    res.update(y=y, view=view)
    return res
