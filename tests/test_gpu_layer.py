"""GPU parity of the whole layer and of its stages against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests import helpers as Hh
from xcaliber_b200 import synth

pytestmark = pytest.mark.gpu

# output tolerance of the path: max relative error 2e-2, mean 5e-3 (relative to max(|exp|, rms))
MAX_REL, MEAN_REL = 2e-2, 5e-3


def run_case(shape, n, token_tile=0, seed=0):
    w, layer = Hh.build_layer(shape, seed=seed, token_tile=token_tile)
    x, logits = synth.make_inputs(shape, w, n, seed=seed)
    y = layer.forward(x.cuda(), logits.cuda())
    torch.cuda.synchronize()
    status = layer.status(n)
    assert status == 0, f"device status {status:#x}"
    ref = O.layer_forward(x, logits, w, shape)
    view = layer.view(n)
    return w, layer, x, logits, y, ref, view


def check_stages(shape, n, y, ref, view, check_bits=True):
    Hh.assert_routing_equal(view, ref, n)
    pk = ref["pack"]
    # activation scale + NVFP4 packets: bit-exact integer work
    sc = view["act_scale"].cpu().numpy()
    assert sc[0] == ref["xgs"] and sc[1] == ref["xgs_inv"]
    rows_tok = pk["topk_row"].reshape(-1)
    tok = np.repeat(np.arange(n), shape.k_eff)
    xq = view["xq"].cpu().numpy()
    np.testing.assert_array_equal(xq[rows_tok], O.pack_nibbles(ref["codes"])[tok])
    sfx = view["sfx"].cpu().numpy()
    kb16 = shape.hidden // 16
    r = rows_tok[:, None]
    c = np.arange(kb16)[None, :]
    nt = view['token_tile']
    got_sf = sfx[r // nt, c // 4, (r % 32) * 16 + ((r % nt) // 32) * 4 + (c % 4)]
    np.testing.assert_array_equal(got_sf, ref["sx"][tok])
    # FF1 output rows
    m = Hh.valid_row_mask(pk)
    ya = view["yact"].float().cpu()[: len(m)][m]
    ye = torch.from_numpy(O.bits_to_f32(ref["yact_bits"][m]))
    mx, mean = O.rel_errors(ya, ye)
    assert mx <= MAX_REL and mean <= MEAN_REL, f"FF1 rel err max {mx:.4g} mean {mean:.4g}"
    oa = view["out_rows"].float().cpu()[: len(m)][m]
    oe = torch.from_numpy(O.bits_to_f32(ref["out_rows"][m]))
    mx, mean = O.rel_errors(oa, oe)
    assert mx <= MAX_REL and mean <= MEAN_REL, f"FF2 rel err max {mx:.4g} mean {mean:.4g}"
    mx, mean = O.rel_errors(y.float().cpu(), ref["y"].float())
    assert mx <= MAX_REL and mean <= MEAN_REL, f"layer rel err max {mx:.4g} mean {mean:.4g}"


@pytest.mark.parametrize("token_tile", [32, 64, 128])
def test_toy_layer(token_tile):
    shape = synth.SHAPES["toy"]
    _, _, _, _, y, ref, view = run_case(shape, 64, token_tile)
    check_stages(shape, 64, y, ref, view)


@pytest.mark.parametrize("n", [1, 7, 33, 200])
def test_toy_ragged_batches(n):
    shape = synth.SHAPES["toy"]
    _, _, _, _, y, ref, view = run_case(shape, n)
    check_stages(shape, n, y, ref, view)


def test_zero_tokens():
    shape = synth.SHAPES["toy"]
    w, layer = Hh.build_layer(shape)
    y = layer.forward(torch.empty(0, shape.hidden, dtype=torch.bfloat16, device="cuda"),
                      torch.empty(0, shape.num_experts, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, shape.hidden)


def test_partial_tiles_gptoss_like():
    # I and H not multiples of 128 / 256: partial M tiles, zero-filled K tail, clamped SwiGLU
    shape = synth.scaled_shape(synth.SHAPES["gptoss"], hidden=704, inter=352, num_experts=16)
    _, _, _, _, y, ref, view = run_case(shape, 48)
    check_stages(shape, 48, y, ref, view)


def test_qwen3_like_skewed():
    shape = synth.scaled_shape(synth.SHAPES["qwen3"], hidden=512, inter=256, num_experts=128)
    _, _, _, _, y, ref, view = run_case(shape, 300)
    check_stages(shape, 300, y, ref, view)


def test_forward_host_matches_device():
    shape = synth.SHAPES["toy"]
    w, layer = Hh.build_layer(shape)
    x, logits = synth.make_inputs(shape, w, 64)
    y_dev = layer.forward(x.cuda(), logits.cuda()).cpu()
    xh, lh = x.pin_memory(), logits.pin_memory()
    yh = torch.empty_like(x).pin_memory()
    layer.forward_host(xh, lh, yh)
    assert torch.equal(yh, y_dev)


def test_forward_routed_matches_router():
    shape = synth.SHAPES["toy"]
    w, layer = Hh.build_layer(shape)
    x, logits = synth.make_inputs(shape, w, 64)
    y = layer.forward(x.cuda(), logits.cuda())
    v = layer.view(64)
    y2 = layer.forward_routed(x.cuda(), v["topk_idx"].clone(), v["topk_w"].clone())
    assert torch.equal(y, y2)


def test_deterministic_run_to_run():
    shape = synth.SHAPES["toy"]
    w, layer = Hh.build_layer(shape)
    x, logits = synth.make_inputs(shape, w, 200)
    xa, la = x.cuda(), logits.cuda()
    y1 = layer.forward(xa, la).clone()
    y2 = layer.forward(xa, la).clone()
    assert torch.equal(y1, y2)


def test_ff1_cta_pair_variant(monkeypatch):
    # 2-SM (cta_group::2) FF1, the default for prefill-sized experts, and the single-CTA kernel
    # (XMOE_FF1_PAIR=0) must give the same rows, bit for bit
    shape = synth.scaled_shape(synth.SHAPES["mixtral"], hidden=512, inter=384, num_experts=4)
    _, layer, x, logits, y, ref, view = run_case(shape, 900)
    check_stages(shape, 900, y, ref, view)
    yact_default = view["yact"].clone()
    monkeypatch.setenv("XMOE_FF1_PAIR", "0")
    y2 = layer.forward(x.cuda(), logits.cuda())
    torch.cuda.synchronize()
    assert layer.status(900) == 0
    m = torch.from_numpy(Hh.valid_row_mask(ref["pack"])).cuda()
    assert torch.equal(layer.view(900)["yact"][: len(m)][m], yact_default[: len(m)][m])
    assert torch.equal(y, y2)


def test_long_k_prefill_uses_wide_ff2_tile():
    # inter >= 2048 with prefill-sized experts: FF1 token-major kernel + FF2 with 256-token tiles,
    # ragged last tiles (counts not multiples of 128 or 256)
    shape = synth.scaled_shape(synth.SHAPES["mixtral"], hidden=256, inter=2048, num_experts=4)
    _, _, _, _, y, ref, view = run_case(shape, 700)
    assert view["token_tile"] == 128
    check_stages(shape, 700, y, ref, view)


def test_routed_rows_with_unused_slots_and_row_bound():
    # the expert-parallel receive path: a buffer of cap rows, the first m in use, expert id -1 beyond;
    # rows-only output must equal the routed forward on the m rows alone
    shape = synth.scaled_shape(synth.SHAPES["toy"], top_k=1, num_shared_experts=0)
    w, layer = Hh.build_layer(shape, token_tile=32)  # same tile for both calls: same summation order
    m, cap = 70, 256
    x, _ = synth.make_inputs(shape, w, cap)
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, shape.num_experts, (cap, 1), generator=g, dtype=torch.int32)
    idx[m:] = -1
    gate = torch.rand(cap, 1, generator=g).to(torch.bfloat16)
    xd, idxd, gd = x.cuda(), idx.cuda(), gate.cuda()
    y_ref = layer.forward_routed(xd[:m], idxd[:m], gd[:m])
    scale = layer.view(m)["act_scale"].clone()
    n_valid = torch.tensor([m], dtype=torch.int32, device="cuda")
    layer.forward_routed_rows(xd, idxd, gd, act_scale=scale, n_valid=n_valid)
    torch.cuda.synchronize()
    assert layer.status(cap) == 0
    v = layer.view(cap)
    rows = v["topk_row"][:m, 0].long()   # (the index arrays of the rows beyond n_valid are left as they were)
    assert int(v["counts"].sum()) == m
    assert torch.equal(v["out_rows"][rows], y_ref)


def test_tensor_pipe_probe_reports_plausible_rates():
    from xcaliber_b200 import ops
    nv = ops.probe_mma_rate("nvfp4", 65536)
    bf = ops.probe_mma_rate("bf16", 65536)
    # B200 nominal dense rates are 9000 / 2250 TFLOP/s; the probe must land in that neighbourhood
    assert 4000 < nv < 10000 and 1000 < bf < 2600 and 3.0 < nv / bf < 5.0, (nv, bf)


@pytest.mark.parametrize("rows,inter,keep", [(300, 2048, 512), (200, 256, 64), (128, 1024, 100), (64, 2048, 1),
                                             (64, 2048, 2047), (40, 4096, 1000)])
def test_activation_topk_exact_with_ties(rows, inter, keep):
    # few distinct magnitudes => many ties at the threshold: survivors must be the lowest indices
    import ctypes as C

    from xcaliber_b200 import _lib

    g = torch.Generator().manual_seed(1)
    y = (torch.randn(rows, inter, generator=g) * 4).round().clamp(-20, 20).to(torch.bfloat16)
    cap = (rows + 127) // 128 * 128
    counts = torch.tensor([rows], dtype=torch.int32, device="cuda")
    offsets = torch.tensor([0, cap], dtype=torch.int32, device="cuda")
    yd = torch.zeros(cap, inter, dtype=torch.bfloat16, device="cuda")
    yd[:rows] = y.cuda()
    _lib.check(_lib.lib().xmoe_act_topk(yd.data_ptr(), counts.data_ptr(), offsets.data_ptr(), 1, inter, keep, cap, None),
               "xmoe_act_topk")
    torch.cuda.synchronize()
    ref = O.act_topk_rows(O.bf16_bits(y), keep)
    np.testing.assert_array_equal(O.bf16_bits(yd[:rows].cpu()), ref)


@pytest.mark.parametrize("name,n", [("toy", 200), ("toy", 7), ("dsv3s", 300), ("qwen3s", 129), ("toysig", 65)])
def test_gate_gemm_and_gated_forward(name, n):
    # the gate GEMM inside the library: logits against an fp32 matmul, then the gated forward must equal
    # the plain forward fed with those logits, bit for bit
    shape = {"toy": synth.SHAPES["toy"],
             "toysig": synth.scaled_shape(synth.SHAPES["toy"], scoring="sigmoid", renormalize=False),
             "dsv3s": synth.scaled_shape(synth.SHAPES["dsv3"], hidden=512, inter=256, num_experts=64, act_topk_keep=0),
             "qwen3s": synth.scaled_shape(synth.SHAPES["qwen3"], hidden=512, inter=256, num_experts=128)}[name]
    from xcaliber_b200 import ops

    w, layer = Hh.build_layer(shape)
    x, _ = synth.make_inputs(shape, w, n)
    gw = w.router_weight.to(torch.bfloat16)
    lg = ops.gate_logits(x.cuda(), gw.cuda()).cpu()
    ref = (x.float() @ gw.float().T)
    # bf16 rounding of sums accumulated in another order (and with the tensor core's fp32 alignment): within
    # two bf16 steps of max(|ref|, rms), and mostly the same bits
    step = torch.maximum(ref.abs(), ref.pow(2).mean().sqrt()) * 2.0 ** -7
    assert ((lg.float() - ref).abs() <= step).all()
    assert (lg == ref.to(torch.bfloat16)).float().mean() > 0.9
    # ONE kernel for gate GEMM + router: with and without the logits written out, the routing arrays and the
    # output must equal the two-step path (gate_logits, then forward) bit for bit
    y2 = layer.forward(x.cuda(), lg.cuda())
    v2 = layer.view(n)
    idx2, w2 = v2["topk_idx"].clone(), v2["topk_w"].clone()
    for keep in (True, False):
        v2["topk_idx"].fill_(-5)
        y = layer.forward_gated(x.cuda(), gw.cuda(), keep_logits=keep)
        torch.cuda.synchronize()
        assert layer.status(n) == 0
        if keep:
            assert torch.equal(layer.last_logits.cpu(), lg)
        v = layer.view(n)
        assert torch.equal(v["topk_idx"], idx2) and torch.equal(Hh.bits_t(v["topk_w"]), Hh.bits_t(w2))
        assert torch.equal(y, y2)


@pytest.mark.parametrize("n", [9, 300])
def test_forward_scatter_writes_rows_token_major(n):
    # the layer without its combine: the FF2 epilogue stores row (token, slot) at rows_out[token * k_eff + slot];
    # the same bits as the packed rows of a plain forward, for router-made and for caller-supplied routing
    shape = synth.scaled_shape(synth.SHAPES["toy"], num_shared_experts=1)
    w, layer = Hh.build_layer(shape)
    x, logits = synth.make_inputs(shape, w, n)
    xd, ld = x.cuda(), logits.cuda()
    y = layer.forward(xd, ld)
    v = layer.view(n)
    packed = v["out_rows"][v["topk_row"].reshape(-1).long()].clone()           # [n * k_eff, H] token-major
    idx, gate = v["topk_idx"][:, : shape.top_k].contiguous().clone(), v["topk_w"][:, : shape.top_k].contiguous().clone()
    poison = torch.full((n * shape.k_eff + 3, shape.hidden), -7.0, dtype=torch.bfloat16, device="cuda")
    out = layer.forward_scatter(xd, poison.clone(), router_logits=ld)
    torch.cuda.synchronize()
    assert layer.status(n) == 0
    assert torch.equal(out[: n * shape.k_eff], packed) and (out[n * shape.k_eff:] == -7.0).all()
    out2 = layer.forward_scatter(xd, poison.clone(), topk_idx=idx, topk_w=gate)
    assert torch.equal(out2[: n * shape.k_eff], packed)
    # and the combine over those rows is the layer output
    from xcaliber_b200 import ops
    slots = torch.arange(n * shape.k_eff, dtype=torch.int32, device="cuda").reshape(n, shape.k_eff)
    assert torch.equal(ops.combine(out, slots), y)
