"""CPU oracle for the fused MoE hot path (router -> permute -> NVFP4 act quant -> FF1 -> FF2 -> combine).

TEST INFRASTRUCTURE ONLY. Nothing in the product package may import this module; only
tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py use it.

It restates, in numpy/torch on the CPU, the algorithm of the reference
(Pranshu-Bahadur/xCaliber; paths relative to that tree, S = xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a):

  router_topk          S/topk.cuh:44-140            bit-exact selection, fp32 weights
  route_pack           S/preamble.cuh:466-535  ==  S/benchmarks/benchmark.cu:172-183
  act_scale            S/preamble.cuh:98-128
  ue4m3_ceil/_decode   S/preamble.cuh:17-43
  act_quant            S/preamble.cuh:45-66, 567-599
  nvfp4 weight format  S/xR64FF1FF2/xR64FF1.cu:17-20, xR64FF2.cu:17-20
  int4-g128 format     xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/xR64ABSRepack.cu:3-24,
                       .../vllm/xcaliber_int4_vllm/method.py:194-203
  layer identity       co-design.md:75-90, S/xR64FF1FF2/xR64FF1.cu:356-386 (weight after SwiGLU)

Pinning status. Router selection, permutation, UE4M3/E2M1 arithmetic and the activation
quantiser are pinned (a) against the reference's own routing-by-construction check and its
analytic FF1 known-answer test, restated in tests/golden/, and (b) on a GPU box against the
reference's topk.cuh / preamble.cuh kernels compiled unmodified from the reference tree
(oracle/ref_kernels.cu -> oracle/_ref/). The layer OUTPUT has no higher-precision reference
in xCaliber (it only records new-vs-old deltas tied to sm_120 rounding): for outputs this
oracle is "parity unpinned" beyond the analytic FF1 test. Group-limited sigmoid routing,
clamped SwiGLU, activation top-k and shared experts do not exist in the reference; their
rules are defined in the docstrings below.
"""
from __future__ import annotations

import numpy as np
import torch

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_SIGNED = np.concatenate([E2M1, -E2M1]).astype(np.float32)   # indexed by the 4-bit code (bit 3 = sign)


# ---------------------------------------------------------------------------------------
# bit helpers
# ---------------------------------------------------------------------------------------
def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy array of its bit patterns."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))
    return (rounded >> 16).astype(np.uint16)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return bits_to_f32(f32_to_bf16_bits(x))


# ---------------------------------------------------------------------------------------
# router  (S/topk.cuh)
# ---------------------------------------------------------------------------------------
def _order_keys(bits: np.ndarray) -> np.ndarray:
    """topk.cuh:58-69: monotone map of bf16 bits (negatives flip all bits, others set the
    sign bit), expert id in the low half inverted so that ties pick the lower id."""
    raw = bits.astype(np.uint32)
    ordered = raw ^ (((np.uint32(0) - (raw >> 15)) | np.uint32(0x8000)) & np.uint32(0xFFFF))
    e = np.arange(bits.shape[-1], dtype=np.uint32)
    return (ordered << 16) | (np.uint32(0xFFFF) - e)


def router_topk(logits: torch.Tensor, top_k: int, scoring: str = "softmax", renormalize: bool = True,
                routed_scale: float = 1.0, expert_scale: torch.Tensor | None = None):
    """Flat top-k. Returns (idx int32 [N,k] in descending-logit order, weight bf16-bits uint16 [N,k],
    weight fp32 before the bf16 round)."""
    bits = bf16_bits(logits)
    keys = _order_keys(bits)
    order = np.argsort(-keys.astype(np.int64), axis=1, kind="stable")[:, :top_k]
    idx = order.astype(np.int32)
    x = bits_to_f32(np.take_along_axis(bits, order, axis=1)).astype(np.float32)
    if scoring == "sigmoid":
        w = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)
        denom = w.sum(axis=1, keepdims=True)
    else:
        w = np.exp((x - x[:, :1]).astype(np.float64)).astype(np.float32)
        if renormalize:
            denom = w.sum(axis=1, keepdims=True)
        else:
            allx = bits_to_f32(bits).astype(np.float64)
            denom = np.exp(allx - x[:, :1].astype(np.float64)).sum(axis=1, keepdims=True).astype(np.float32)
    if renormalize or scoring != "sigmoid":
        w = w / denom
    w = w * np.float32(routed_scale)
    if expert_scale is not None:
        w = w * bits_to_f32(bf16_bits(expert_scale))[idx]
    w = w.astype(np.float32)
    return idx, f32_to_bf16_bits(w), w


def sigmoid_lut() -> np.ndarray:
    """fp32 sigmoid of every bf16 bit pattern (double-precision evaluation, one rounding)."""
    x = bits_to_f32(np.arange(65536, dtype=np.uint16)).astype(np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        return (1.0 / (1.0 + np.exp(-x))).astype(np.float32)


def router_topk_grouped(logits: torch.Tensor, top_k: int, n_group: int, topk_group: int,
                        bias: torch.Tensor | None, renormalize: bool = True, routed_scale: float = 1.0,
                        expert_scale: torch.Tensor | None = None, lut: np.ndarray | None = None):
    """Group-limited sigmoid routing with selection bias (DeepSeek-V3 rule; not in the reference).

    score = lut[bf16 logit]; choice = fp32(score + bias); group score = fp32 sum of the group's
    two best choices; keep the topk_group best groups (ties: lower group); top_k best choices
    among kept groups (ties: lower expert); weight = score / (sum of the k scores, added in
    slot order in fp32) * routed_scale; bf16 round.
    """
    lut = sigmoid_lut() if lut is None else lut
    bits = bf16_bits(logits)
    n, e = bits.shape
    score = lut[bits]
    choice = score if bias is None else (score + bias.detach().cpu().numpy().astype(np.float32)).astype(np.float32)
    gs = e // n_group
    allowed = np.ones((n, e), dtype=bool)
    if n_group > 1:
        grp = choice.reshape(n, n_group, gs)
        top2 = -np.sort(-grp, axis=2)[:, :, :2]
        gscore = (top2[:, :, 0] + top2[:, :, 1]).astype(np.float32)
        gorder = np.argsort(-gscore, axis=1, kind="stable")[:, :topk_group]
        gmask = np.zeros((n, n_group), dtype=bool)
        np.put_along_axis(gmask, gorder, True, axis=1)
        allowed = np.repeat(gmask, gs, axis=1)
    masked = np.where(allowed, choice, -np.inf).astype(np.float32)
    order = np.argsort(-masked, axis=1, kind="stable")[:, :top_k]
    idx = order.astype(np.int32)
    s = np.take_along_axis(score, order, axis=1).astype(np.float32)
    denom = np.zeros(n, dtype=np.float32)
    for r in range(top_k):
        denom = (denom + s[:, r]).astype(np.float32)
    w = s / denom[:, None] if renormalize else s
    w = (w.astype(np.float32) * np.float32(routed_scale)).astype(np.float32)
    if expert_scale is not None:
        w = (w * bits_to_f32(bf16_bits(expert_scale))[idx]).astype(np.float32)
    return idx, f32_to_bf16_bits(w), w


# ---------------------------------------------------------------------------------------
# permutation  (S/preamble.cuh:466-535 == S/benchmarks/benchmark.cu:172-183)
# ---------------------------------------------------------------------------------------
def route_pack(idx: np.ndarray, w_bits: np.ndarray, num_experts: int, num_shared: int = 0):
    """Walk tokens in ascending order; the running per-expert hit count is the packed row p.

    Returns dict(counts[E_tot], offsets[E_tot+1] (expert starts, multiples of 128),
    topk_off[N,k_eff] (p), topk_row[N,k_eff] (offsets[e]+p), row_token[R], row_weight[R] (bf16 bits),
    idx[N,k_eff], w_bits[N,k_eff]) with shared experts appended as slots k.. (weight 1.0).
    """
    n, k = idx.shape
    e_tot = num_experts + num_shared
    if num_shared:
        sh = np.tile(np.arange(num_experts, e_tot, dtype=np.int32), (n, 1))
        idx = np.concatenate([idx, sh], axis=1)
        w_bits = np.concatenate([w_bits, np.full((n, num_shared), 0x3F80, dtype=np.uint16)], axis=1)
    k_eff = k + num_shared
    counts = np.bincount(idx.reshape(-1), minlength=e_tot).astype(np.int32)
    offsets = np.zeros(e_tot + 1, dtype=np.int32)
    offsets[1:] = np.cumsum((counts + 127) // 128 * 128)
    flat_e = idx.reshape(-1)
    # stable sort by expert keeps ascending (token, slot) order inside each expert
    order = np.argsort(flat_e, kind="stable")
    starts = np.zeros(e_tot + 1, dtype=np.int64)
    starts[1:] = np.cumsum(counts)
    p = np.empty(n * k_eff, dtype=np.int32)
    p[order] = (np.arange(n * k_eff) - starts[flat_e[order]]).astype(np.int32)
    topk_off = p.reshape(n, k_eff)
    topk_row = (offsets[idx] + topk_off).astype(np.int32)
    rows = int(offsets[-1])
    row_token = np.full(rows, -1, dtype=np.int32)
    row_weight = np.zeros(rows, dtype=np.uint16)
    row_token[topk_row.reshape(-1)] = np.repeat(np.arange(n, dtype=np.int32), k_eff)
    row_weight[topk_row.reshape(-1)] = w_bits.reshape(-1)
    return dict(counts=counts, offsets=offsets, topk_off=topk_off, topk_row=topk_row, row_token=row_token,
                row_weight=row_weight, idx=idx.astype(np.int32), w_bits=w_bits)


def to_reference_route_arrays(idx: np.ndarray, w_bits: np.ndarray, topk_off: np.ndarray, num_experts: int):
    """Convert to the reference's containers (preamble.cuh:457-461): topk_off u16 [N,k],
    expert_topk_W u16 [E,NP] and expert_token_idx u16 [E,NP+1] with slot 0 = count; NP = round_up(N,32)."""
    n, k = idx.shape
    np_ = (n + 31) & ~31
    etw = np.zeros((num_experts, np_), dtype=np.uint16)
    eti = np.zeros((num_experts, np_ + 1), dtype=np.uint16)
    for t in range(n):
        for s in range(k):
            e, p = int(idx[t, s]), int(topk_off[t, s])
            etw[e, p] = w_bits[t, s]
            eti[e, 1 + p] = t
    eti[:, 0] = np.bincount(idx.reshape(-1), minlength=num_experts).astype(np.uint16)
    return topk_off.astype(np.uint16), etw, eti


# ---------------------------------------------------------------------------------------
# NVFP4 activation quantisation  (S/preamble.cuh)
# ---------------------------------------------------------------------------------------
def act_scale(x: torch.Tensor):
    """preamble.cuh:98-128: XGS = 2688/amax (fp32), XGSINV = bf16(amax * (1/2688)); zero input -> 0, 0."""
    mag = bf16_bits(x) & np.uint16(0x7FFF)
    m = int(mag.max()) if mag.size else 0
    if m == 0:
        return np.float32(0.0), np.float32(0.0)
    amax = bits_to_f32(np.array([m], dtype=np.uint16))[0]
    xgs = np.float32(2688.0) / amax
    inv = bf16_round(np.array([amax * np.float32(1.0 / 2688.0)], dtype=np.float32))[0]
    return np.float32(xgs), np.float32(inv)


def ue4m3_ceil(x: np.ndarray) -> np.ndarray:
    """preamble.cuh:17-36, vectorised. x fp32 >= 0 -> UE4M3 byte, rounded up."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    e = ((bits >> 23) & 0xFF).astype(np.int32) - 120
    sub = np.minimum(np.ceil(x.astype(np.float64) * 512.0), 7).astype(np.uint32)
    m = ((bits >> 20) & 7).astype(np.int32) + ((bits & 0xFFFFF) != 0).astype(np.int32)
    carry = m == 8
    m = np.where(carry, 0, m)
    e2 = e + carry.astype(np.int32)
    normal = np.where(e2 >= 15, np.where(m > 6, 0x7E, 0x78 | m), (e2 << 3) | m).astype(np.uint32)
    out = np.where(e <= 0, sub, normal)
    out = np.where(x >= 448.0, 0x7E, out)
    out = np.where(x > 0, out, 0)
    return out.astype(np.uint8)


def ue4m3_decode(s: np.ndarray) -> np.ndarray:
    """preamble.cuh:38-43."""
    s = s.astype(np.uint32)
    e, m = s >> 3, s & 7
    normal = (((e + 120) << 23) | (m << 20)).astype(np.uint32).view(np.float32)
    return np.where(e == 0, m.astype(np.float32) * np.float32(1.0 / 512.0), normal).astype(np.float32)


def e2m1_rn_satfinite(v: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e2m1x2.f32 on one value: nearest E2M1, ties to the even mantissa,
    saturate at 6, sign bit from the input (so -0 keeps its sign)."""
    a = np.abs(v).astype(np.float32)
    code = ((a > 0.25).astype(np.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5)
            + (a > 5.0)).astype(np.uint8)
    return code | (np.signbit(v).astype(np.uint8) << 3)


def act_quant(x: torch.Tensor, xgs: np.float32):
    """preamble.cuh:567-599 per token and 16 K. Returns (codes u8 [N,H] one nibble per element,
    scale bytes u8 [N,H/16])."""
    bits = bf16_bits(x)
    n, h = bits.shape
    xf = bits_to_f32(bits)
    mag = (bits & np.uint16(0x7FFF)).reshape(n, h // 16, 16).max(axis=2)
    a = bits_to_f32(mag)
    t = (a * np.float32(xgs)).astype(np.float32) * np.float32(1.0 / 6.0)
    s = ue4m3_ceil(t.astype(np.float32))
    s = np.where(mag == 0, 0, s).astype(np.uint8)
    with np.errstate(divide="ignore", invalid="ignore"):
        qs = bf16_round((np.float32(xgs) / ue4m3_decode(s)).astype(np.float32))
    prod = bf16_round((xf.reshape(n, h // 16, 16) * qs[:, :, None]).astype(np.float32))
    codes = e2m1_rn_satfinite(prod)
    codes = np.where((mag == 0)[:, :, None], 0, codes).astype(np.uint8)
    return codes.reshape(n, h), s


def act_dequant(codes: np.ndarray, s: np.ndarray, xgs_inv: np.float32, with_global: bool = True) -> np.ndarray:
    val = E2M1_SIGNED[codes & 15]
    n, h = codes.shape
    out = val.reshape(n, h // 16, 16) * ue4m3_decode(s)[:, :, None]
    out = out.reshape(n, h).astype(np.float32)
    return out * np.float32(xgs_inv) if with_global else out


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """low nibble = lower K (preamble.cuh:60)."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def sf_tile_layout(s: np.ndarray, kb_pad: int | None = None) -> np.ndarray:
    """Scale bytes [rows, K/16] -> the tiled order the kernels use: [ceil(rows/128), kb_pad, 512]
    with byte (row%32)*16 + (row//32 % 4)*4 + (k16 % 4) inside the tile of (row//128, k16//4)."""
    rows, k16 = s.shape
    kb = (k16 + 3) // 4
    kb_pad = kb_pad or (kb + 3) // 4 * 4
    rb = (rows + 127) // 128
    out = np.zeros((rb, kb_pad, 512), dtype=np.uint8)
    r = np.arange(rows)[:, None]
    c = np.arange(k16)[None, :]
    out[r // 128, c // 4, (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4)] = s
    return out


# ---------------------------------------------------------------------------------------
# weight formats
# ---------------------------------------------------------------------------------------
def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(b)).view(torch.float8_e4m3fn).float().numpy()


def nvfp4_dequant(packed: np.ndarray, scale: np.ndarray, gs=None) -> np.ndarray:
    """packed u8 [rows, K/2] (low nibble = even K), scale e4m3 bits [rows, K/16] -> f32 [rows, K]
    = e2m1 * e4m3 (* gs when given)."""
    rows, kh = packed.shape
    codes = np.empty((rows, kh * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    val = E2M1_SIGNED[codes & 15]
    s = e4m3_decode(scale)
    out = (val.reshape(rows, kh // 8, 16) * s[:, :, None]).reshape(rows, kh * 2).astype(np.float32)
    return out if gs is None else out * np.float32(gs)


def int4_dequant_gptq(qweight: np.ndarray, scales_bits: np.ndarray) -> np.ndarray:
    """GPTQ i32 [K/8, O] uint4b8 + bf16-bit scales [G, O] -> bf16-rounded f32 weights [O, K]:
    w = bf16((u4 - 8) * s[k // 128])."""
    k8, o = qweight.shape
    u = qweight.astype(np.int64) & 0xFFFFFFFF
    nib = np.stack([(u >> (4 * j)) & 0xF for j in range(8)], axis=1)      # [K/8, 8, O]
    q = nib.reshape(k8 * 8, o).astype(np.float32) - 8.0                    # [K, O]
    s = bits_to_f32(scales_bits)                                           # [G, O]
    w = q * np.repeat(s, 128, axis=0)[: k8 * 8]
    return bf16_round(w.T.copy().astype(np.float32))


def repack_gptq_reference_layout(qweight: np.ndarray) -> np.ndarray:
    """The reference's own repack target (xR64ABSRepack.cu:3-24): [K/8, O] uint4b8 -> [O, K/8] s4
    (xor 0x88888888, transposed). Used only to show the two packings carry the same integers."""
    return (qweight.astype(np.int64) & 0xFFFFFFFF ^ 0x88888888).astype(np.uint32).T.copy()


# ---------------------------------------------------------------------------------------
# layer
# ---------------------------------------------------------------------------------------
def glu(g: torch.Tensor, u: torch.Tensor, activation: str, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """silu: silu(g)*u (co-design.md:75-90). swiglu_clamp (not in the reference):
    g=min(g,limit), u=clamp(u,-limit,limit), g*sigmoid(alpha*g)*(u+1). gelu_tanh: the INT4
    lane's alternative gate (xR64ABS.cuh:114-121)."""
    if activation == "swiglu_clamp":
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
        return g * torch.sigmoid(alpha * g) * (u + 1.0)
    if activation == "gelu_tanh":
        return torch.nn.functional.gelu(g, approximate="tanh") * u
    return torch.nn.functional.silu(g) * u


def ff1_rows(w13_packed: np.ndarray, w13_scale: np.ndarray, gs, codes: np.ndarray, sx: np.ndarray,
             xgs_inv, row_weight_bits: np.ndarray, activation: str = "silu", alpha: float = 1.702,
             limit: float = 7.0) -> np.ndarray:
    """FF1 of one expert on already-quantised rows (xR64FF1.cu:110-130, 356-386): G, U in fp32 from
    exact NVFP4 x NVFP4 products, each times weight_global_scale * XGSINV, GLU, times the routing
    weight, bf16. w13_packed u8 [2I, H/2], w13_scale e4m3 bits [2I, H/16], gs (gate, up),
    codes u8 [rows, H], sx u8 [rows, H/16] -> bf16 bits [rows, I]."""
    i = w13_packed.shape[0] // 2
    w13 = torch.from_numpy(nvfp4_dequant(w13_packed, w13_scale))
    xa = torch.from_numpy(act_dequant(codes, sx, np.float32(1.0), with_global=False))
    g = (xa @ w13[:i].t()) * (np.float32(gs[0]) * np.float32(xgs_inv))
    u = (xa @ w13[i:].t()) * (np.float32(gs[1]) * np.float32(xgs_inv))
    y = glu(g, u, activation, alpha, limit) * torch.from_numpy(bits_to_f32(row_weight_bits))[:, None]
    return f32_to_bf16_bits(y.float().numpy())


def expert_ff1(xa: torch.Tensor, w13: torch.Tensor, gs, xgs_inv, row_weight: torch.Tensor, shape) -> np.ndarray:
    """FF1 rows of one expert from dequantised operands, fp32 (xR64FF1.cu:110-130, 356-386): xa f32 [rows, H]
    (activation codes times block scales, without XGSINV), w13 f32 [2I, H] (without the tensor scales gs) ->
    bf16 bits [rows, I] of glu(G, U) * routing weight, BEFORE any activation top-k."""
    i = w13.shape[0] // 2
    g = (xa @ w13[:i].t()) * (np.float32(gs[0]) * np.float32(xgs_inv))
    u = (xa @ w13[i:].t()) * (np.float32(gs[1]) * np.float32(xgs_inv))
    y = glu(g, u, shape.activation, shape.swiglu_alpha, shape.swiglu_limit) * row_weight[:, None]
    return f32_to_bf16_bits(y.float().numpy())


def expert_ff2(yact_bits: np.ndarray, w2: torch.Tensor) -> np.ndarray:
    """FF2 rows of one expert: bf16 activations [rows, I] (bits) times the bf16-exact weights w2 f32 [H, I],
    fp32 accumulation, one bf16 round -> bits [rows, H]."""
    ya = torch.from_numpy(bits_to_f32(yact_bits))
    return f32_to_bf16_bits((ya @ w2.t()).float().numpy())


def act_topk_rows(y_bits: np.ndarray, keep: int) -> np.ndarray:
    """Keep the `keep` largest |y| per row (bf16 magnitudes, ties to the lower index), zero the rest."""
    mag = (y_bits & np.uint16(0x7FFF)).astype(np.int64)
    n, i = mag.shape
    key = mag * i + (i - 1 - np.arange(i))[None, :]
    order = np.argsort(-key, axis=1, kind="stable")[:, :keep]
    mask = np.zeros((n, i), dtype=bool)
    np.put_along_axis(mask, order, True, axis=1)
    return np.where(mask, y_bits, 0).astype(np.uint16)


def dense_expert_weights(weights, shape, device=None):
    """Every expert dequantised once to bf16, as a CPU deployment of the dequantise-then-bf16-matmul path does
    at load time: list of (w_gate [I,H], w_up [I,H], w_down [H,I]) bf16 CPU tensors with the tensor scales
    folded in. The arithmetic is plain torch and may run on `device` (e.g. the GPU that synthesised the
    weights) before the result is moved to the CPU; the values do not depend on where it runs (every product
    is rounded once, to bf16)."""
    dev = torch.device(device) if device is not None else weights.w13_packed.device
    lut = torch.from_numpy(E2M1_SIGNED).to(dev)
    i = shape.inter
    out = []
    for ex in range(shape.e_tot):
        pk = weights.w13_packed[ex].to(dev)
        rows, kh = pk.shape
        val = torch.stack([lut[(pk & 15).long()], lut[(pk >> 4).long()]], dim=-1).reshape(rows, kh // 8, 16)
        sc = weights.w13_scale[ex].to(dev).contiguous().view(torch.float8_e4m3fn).float()
        w13 = (val * sc[:, :, None]).reshape(rows, kh * 2)
        gs = weights.w13_gs[ex].to(dev).float()
        wg = (w13[:i] * gs[0]).to(torch.bfloat16).cpu()
        wu = (w13[i:] * gs[1]).to(torch.bfloat16).cpu()
        q = weights.w2_qweight[ex].to(dev)
        k8, o = q.shape
        nib = torch.stack([(q >> (4 * j)) & 0xF for j in range(8)], dim=1).reshape(k8 * 8, o).float() - 8.0
        s2 = weights.w2_scales[ex].to(dev).float().repeat_interleave(128, dim=0)[: k8 * 8]
        w2 = (nib * s2).to(torch.bfloat16).t().contiguous().cpu()
        out.append((wg, wu, w2))
    return out


def layer_forward(x: torch.Tensor, logits: torch.Tensor | None, weights, shape, *, precision: str = "f32",
                  routing=None, threads: int | None = None, expert_scale: torch.Tensor | None = None, dense=None):
    """Whole layer on the CPU. `weights` is a synth.LayerWeights (checkpoint formats), `shape` a
    synth.MoEShape. precision "f32": exact dequantised values, fp32 matmuls (parity oracle).
    precision "bf16": dequantise to bf16 and use bf16 matmuls (the dequantise-then-bf16-matmul
    path; used for the timed CPU baseline; `dense` = dense_expert_weights(...) skips the per-call
    dequantisation). Returns dict(y bf16 [N,H], plus routing / packing intermediates)."""
    if threads:
        torch.set_num_threads(threads)
    n, h = x.shape
    i, e, k = shape.inter, shape.num_experts, shape.top_k
    if routing is not None:
        idx, w_bits = routing
    elif shape.n_group > 1 or weights.router_bias is not None:
        idx, w_bits, _ = router_topk_grouped(logits, k, shape.n_group, shape.topk_group, weights.router_bias,
                                             shape.renormalize, shape.routed_scale, expert_scale)
    else:
        idx, w_bits, _ = router_topk(logits, k, shape.scoring, shape.renormalize, shape.routed_scale, expert_scale)
    pk = route_pack(idx, w_bits, e, shape.num_shared_experts)
    xgs, xgs_inv = act_scale(x)
    codes, sx = act_quant(x, xgs)
    xdq = torch.from_numpy(act_dequant(codes, sx, xgs_inv, with_global=False))   # [N,H] without XGSINV
    rows = int(pk["offsets"][-1])
    yact_bits = np.zeros((rows, i), dtype=np.uint16)
    out_rows = np.zeros((rows, h), dtype=np.uint16)
    if dense is None:
        w13p = weights.w13_packed.cpu().numpy()
        w13s = weights.w13_scale.cpu().numpy()
        w13g = weights.w13_gs.cpu().numpy()
        w2q = weights.w2_qweight.cpu().numpy()
        w2s = bf16_bits(weights.w2_scales)
    else:
        assert precision == "bf16"
    mm_dtype = torch.bfloat16 if precision == "bf16" else torch.float32
    for ex in range(shape.e_tot):
        c = int(pk["counts"][ex])
        if c == 0:
            continue
        r0 = int(pk["offsets"][ex])
        tok = torch.from_numpy(pk["row_token"][r0:r0 + c].astype(np.int64))
        rw = torch.from_numpy(bits_to_f32(pk["row_weight"][r0:r0 + c]))
        xa = xdq[tok]
        if dense is None:
            w13 = torch.from_numpy(nvfp4_dequant(w13p[ex], w13s[ex]))             # [2I,H] without gs
        if precision == "bf16":
            if dense is None:
                wg = (w13[:i] * float(w13g[ex, 0])).to(mm_dtype)
                wu = (w13[i:] * float(w13g[ex, 1])).to(mm_dtype)
            else:
                wg, wu, _ = dense[ex]
            xb = (xa * float(xgs_inv)).to(mm_dtype)
            g = (xb @ wg.t()).float()
            u = (xb @ wu.t()).float()
            y = glu(g, u, shape.activation, shape.swiglu_alpha, shape.swiglu_limit) * rw[:, None]
            yb = f32_to_bf16_bits(y.float().numpy())
        else:
            yb = expert_ff1(xa, w13, w13g[ex], xgs_inv, rw, shape)
        if shape.act_topk_keep and shape.act_topk_keep < i:
            yb = act_topk_rows(yb, shape.act_topk_keep)
        yact_bits[r0:r0 + c] = yb
        w2 = dense[ex][2] if dense is not None else torch.from_numpy(int4_dequant_gptq(w2q[ex], w2s[ex]))  # [H, I]
        ya = torch.from_numpy(bits_to_f32(yb))
        o = (ya.to(mm_dtype) @ w2.to(mm_dtype).t()).float()
        out_rows[r0:r0 + c] = f32_to_bf16_bits(o.numpy())
    acc = np.zeros((n, h), dtype=np.float32)
    for s in range(shape.k_eff):
        acc = (acc + bits_to_f32(out_rows[pk["topk_row"][:, s]])).astype(np.float32)
    y = torch.from_numpy(f32_to_bf16_bits(acc).view(np.int16)).view(torch.bfloat16)
    return dict(y=y, idx=pk["idx"], w_bits=pk["w_bits"], pack=pk, xgs=xgs, xgs_inv=xgs_inv, codes=codes, sx=sx,
                yact_bits=yact_bits, out_rows=out_rows)


def rel_errors(got: torch.Tensor, exp: torch.Tensor):
    """|got-exp| / max(|exp|, rms(exp)): the reference's floor convention
    (ff1_w4a4_swiglu_topk_reduce.cu:1233-1234 uses floor 1.0 on O(H) values; here the floor is
    the tensor RMS because the data are N(0,1)*N(0,0.02)). Returns (max, mean)."""
    g, e = got.float(), exp.float()
    floor = e.pow(2).mean().sqrt().clamp_min(1e-30)
    rel = (g - e).abs() / torch.maximum(e.abs(), floor)
    return float(rel.max()), float(rel.mean())
