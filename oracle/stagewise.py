"""Stage-wise parity check of one fused-MoE layer call at checkpoint sizes.

TEST INFRASTRUCTURE ONLY (like the rest of oracle/): used by tests/ and by bench.py's parity spot check.

At the sizes of the published model shapes the CPU oracle cannot dequantise every expert within a test
run, so each stage is checked on its own, against what the kernel really consumed:
  routing, permutation, activation scale, NVFP4 packets    bit-exact, all tokens
  FF1 rows     sampled experts x sampled packed rows x sampled output columns (at least one column in
               every 128-column weight tile), full K, from the oracle's own packets (= the kernel's)
  FF2 rows     same sampling; the oracle reads the GPU's FF1 rows, i.e. exactly the kernel's input
  combine      y == bf16(fp32 sum of the GPU's FF2 rows in slot order), bit-exact, all tokens
Tolerance of the two GEMM stages: max rel 2e-2, mean 5e-3 (relative to max(|exp|, rms)).
`view` is the dict of workspace views of the call (device tensors), `ckpt` the checkpoint-format weights
(any device), `rw` a weights object whose router parts are on the CPU.
"""
import numpy as np
import torch

from . import moe_oracle as O

MAX_REL, MEAN_REL = 2e-2, 5e-3


def bits(t):
    return O.bf16_bits(t)


def assert_routing_equal(view, pk):
    """Routing indices, packed rows and counts must be bit-exact; gate weights within the reference's own 2^-8
    (benchmark.cu:622-624)."""
    np.testing.assert_array_equal(view["topk_idx"].cpu().numpy(), pk["idx"])
    np.testing.assert_array_equal(view["counts"].cpu().numpy(), pk["counts"])
    np.testing.assert_array_equal(view["offsets"].cpu().numpy(), pk["offsets"])
    np.testing.assert_array_equal(view["topk_off"].cpu().numpy(), pk["topk_off"])
    np.testing.assert_array_equal(view["topk_row"].cpu().numpy(), pk["topk_row"])
    rows = int(pk["offsets"][-1])
    live = pk["row_token"] >= 0
    np.testing.assert_array_equal(view["row_token"].cpu().numpy()[:rows][live], pk["row_token"][live])
    gw = O.bits_to_f32(bits(view["topk_w"]))
    ew = O.bits_to_f32(pk["w_bits"])
    assert np.abs(gw - ew).max() <= 2.0 ** -8

def cover_columns(width, n_cols, rng):
    """n_cols column indices of [0, width): one in every 128-block, the rest uniform; sorted, unique."""
    blocks = (width + 127) // 128
    cols = {min(width - 1, b * 128 + int(rng.integers(0, 128))) for b in range(blocks)}
    while len(cols) < min(n_cols, width):
        cols.add(int(rng.integers(0, width)))
    return np.array(sorted(cols), dtype=np.int64)


def pick_rows(count, cap, rng):
    """Packed-row indices of one expert: first rows, the ragged tail and a random fill."""
    if count <= cap:
        return np.arange(count, dtype=np.int64)
    sel = set(range(min(8, count))) | set(range(max(0, count - 8), count))
    while len(sel) < cap:
        sel.add(int(rng.integers(0, count)))
    return np.array(sorted(sel), dtype=np.int64)


def oracle_routing(shape, rw, logits):
    if shape.n_group > 1 or rw.router_bias is not None:
        idx, w_bits, _ = O.router_topk_grouped(logits, shape.top_k, shape.n_group, shape.topk_group, rw.router_bias,
                                               shape.renormalize, shape.routed_scale)
    else:
        idx, w_bits, _ = O.router_topk(logits, shape.top_k, shape.scoring, shape.renormalize, shape.routed_scale)
    return O.route_pack(idx, w_bits, shape.num_experts, shape.num_shared_experts)


def assert_packets_equal(view, pk, codes, sx, shape, n):
    rows_tok = torch.from_numpy(pk["topk_row"].reshape(-1).astype(np.int64)).to(view["xq"].device)
    tok = np.repeat(np.arange(n), shape.k_eff)
    xq = view["xq"][rows_tok].cpu().numpy()
    np.testing.assert_array_equal(xq, O.pack_nibbles(codes)[tok])
    sfx = view["sfx"].cpu().numpy()
    r = pk["topk_row"].reshape(-1)[:, None]
    c = np.arange(shape.hidden // 16)[None, :]
    nt = view["token_tile"]
    np.testing.assert_array_equal(sfx[r // nt, c // 4, (r % 32) * 16 + ((r % nt) // 32) * 4 + (c % 4)], sx[tok])


def check_combine_exact(y, view):
    rows, tr = view["out_rows"], view["topk_row"].long()
    acc = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
    for s in range(tr.shape[1]):
        acc = acc + rows[tr[:, s]].float()
    assert torch.equal(acc.to(torch.bfloat16), y), "combine differs from the slot-ordered fp32 sum of the FF2 rows"


def check_layer_stages(shape, ckpt, rw, x, logits, y, view, *, dense_view=None, seed=0, experts_cap=10, rows_cap=48,
                       ff1_cols=256, ff2_cols=256, exact_all_tokens=True):
    """Checks one layer call (x, logits on the CPU; y and `view` from the GPU) as described in the module
    docstring and raises AssertionError on the first mismatch. dense_view: the views of a call on the same
    weights with the activation top-k off, required when shape.act_topk_keep > 0 (the FF1 rows before
    sparsification, so that the top-k rule is checked exactly on the kernel's own values).
    Returns dict(pack, worst={ff1: (max, mean), ff2: (max, mean)}, experts=[...])."""
    n = x.shape[0]
    rng = np.random.default_rng(seed * 7919 + n)
    pk = oracle_routing(shape, rw, logits)
    assert_routing_equal(view, pk)
    xgs, xgs_inv = O.act_scale(x)
    sc = view["act_scale"].cpu().numpy()
    assert sc[0] == xgs and sc[1] == xgs_inv, "activation scale differs"
    codes, sx = O.act_quant(x, xgs)
    if exact_all_tokens:
        assert_packets_equal(view, pk, codes, sx, shape, n)
    check_combine_exact(y, view)

    sparse = 0 < shape.act_topk_keep < shape.inter
    assert not sparse or dense_view is not None, "the activation top-k needs the dense rows of a second call"
    live = np.nonzero(pk["counts"])[0]
    chosen = {int(live[np.argmax(pk["counts"][live])]), int(live[np.argmin(pk["counts"][live])])}
    chosen |= set(range(shape.num_experts, shape.e_tot))
    for e in rng.permutation(live):
        if len(chosen) >= experts_cap:
            break
        chosen.add(int(e))
    dev = view["yact"].device
    i_cols = cover_columns(shape.inter, ff1_cols, rng)
    h_cols = cover_columns(shape.hidden, ff2_cols, rng)
    i_cols_t, h_cols_t = torch.from_numpy(i_cols).to(dev), torch.from_numpy(h_cols).to(dev)
    worst = dict(ff1=(0.0, 0.0), ff2=(0.0, 0.0))
    for e in sorted(chosen):
        c, r0 = int(pk["counts"][e]), int(pk["offsets"][e])
        sel = r0 + pick_rows(c, rows_cap, rng)
        sel_t = torch.from_numpy(sel).to(dev)
        tok = pk["row_token"][sel]
        # FF1 on the sampled columns: gate rows i_cols and up rows I + i_cols of this expert
        wrows = torch.cat([i_cols_t, shape.inter + i_cols_t]).to(ckpt.w13_packed.device)
        w13 = torch.from_numpy(O.nvfp4_dequant(ckpt.w13_packed[e][wrows].cpu().numpy(),
                                               ckpt.w13_scale[e][wrows].cpu().numpy()))
        xa = torch.from_numpy(O.act_dequant(codes[tok], sx[tok], np.float32(1.0), with_global=False))
        exp_bits = O.expert_ff1(xa, w13, ckpt.w13_gs[e].cpu().numpy(), xgs_inv,
                                torch.from_numpy(O.bits_to_f32(pk["row_weight"][sel])), shape)
        got_rows = (dense_view if sparse else view)["yact"][sel_t]        # [rows, I] on the GPU
        mx, mean = O.rel_errors(got_rows[:, i_cols_t].float().cpu(), torch.from_numpy(O.bits_to_f32(exp_bits)))
        assert mx <= MAX_REL and mean <= MEAN_REL, f"expert {e}: FF1 rel err max {mx:.4g} mean {mean:.4g}"
        worst["ff1"] = (max(worst["ff1"][0], mx), max(worst["ff1"][1], mean))
        ff2_in = view["yact"][sel_t]
        if sparse:  # the kept set must be the oracle's rule applied to the kernel's own dense values
            np.testing.assert_array_equal(bits(ff2_in), O.act_topk_rows(bits(got_rows), shape.act_topk_keep))
        # FF2 on the sampled output features, from the kernel's own input rows
        hc = h_cols_t.to(ckpt.w2_qweight.device)
        w2 = torch.from_numpy(O.int4_dequant_gptq(ckpt.w2_qweight[e][:, hc].cpu().numpy(),
                                                  bits(ckpt.w2_scales[e][:, hc])))
        exp_out = O.expert_ff2(bits(ff2_in), w2)
        got_out = view["out_rows"][sel_t][:, h_cols_t].float().cpu()
        mx, mean = O.rel_errors(got_out, torch.from_numpy(O.bits_to_f32(exp_out)))
        assert mx <= MAX_REL and mean <= MEAN_REL, f"expert {e}: FF2 rel err max {mx:.4g} mean {mean:.4g}"
        worst["ff2"] = (max(worst["ff2"][0], mx), max(worst["ff2"][1], mean))
    return dict(pack=pk, worst=worst, experts=sorted(chosen))
