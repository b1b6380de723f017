"""Seeded synthetic inputs for the fused MoE layer: configs, weight quantisers, routing data.

The reference ships no weight quantiser (its weights come from checkpoints or constant
fills, sm120a/benchmarks/benchmark.cu:209-221), so the formats are produced here:

* NVFP4 (FF1): E2M1 values in blocks of 16 along K, one E4M3 scale per block, one fp32
  scale per (expert, projection); tensors shaped like the checkpoint contract the
  reference documents at sm120a/xR64FF1FF2/xR64FF1.cu:17-20:
  ``w13_packed u8 [E, 2I, H/2]`` (low nibble = lower K), ``w13_scale e4m3 [E, 2I, H/16]``,
  ``w13_gs f32 [E, 2]`` (the dequant multiplier).
* INT4 group-128 (FF2): symmetric, ``u4 = q + 8``, packed the GPTQ way the reference's
  repack consumes (sm75/xR64/xR64ABSRepack.cu:3-24): ``qweight i32 [E, K/8, O]`` with
  nibble j of word (k8, o) holding K index 8*k8 + j, ``scales bf16 [E, K/128, O]``.

Everything is plain torch and runs on CPU or CUDA; nothing here touches the kernels.
"""
from __future__ import annotations

import dataclasses
import math

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


@dataclasses.dataclass(frozen=True)
class MoEShape:
    """One MoE layer shape. Names follow the reference (H hidden, I intermediate, E experts)."""

    name: str
    hidden: int
    inter: int
    num_experts: int
    top_k: int
    scoring: str = "softmax"          # "softmax" | "sigmoid"
    renormalize: bool = True
    num_shared_experts: int = 0
    n_group: int = 1
    topk_group: int = 1
    routed_scale: float = 1.0
    activation: str = "silu"           # "silu" | "swiglu_clamp" | "gelu_tanh"
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    act_topk_keep: int = 0             # entries kept per FF1 output row, 0 = dense
    router_bias: bool = False
    zipf_bias: float = 0.0             # >0: add a Zipf(zipf_bias)-skewed per-expert logit bias

    @property
    def e_tot(self) -> int:
        return self.num_experts + self.num_shared_experts

    @property
    def k_eff(self) -> int:
        return self.top_k + self.num_shared_experts


SHAPES = {
    "toy": MoEShape("toy", 1024, 512, 8, 2),
    "mixtral": MoEShape("mixtral", 4096, 14336, 8, 2),
    "qwen3": MoEShape("qwen3", 2048, 768, 128, 8, zipf_bias=1.1),
    "gptoss": MoEShape("gptoss", 2880, 2880, 128, 4, activation="swiglu_clamp"),
    "dsv3": MoEShape("dsv3", 7168, 2048, 256, 8, scoring="sigmoid", num_shared_experts=1, n_group=8, topk_group=4,
                     routed_scale=2.5, act_topk_keep=512, router_bias=True),
}


def scaled_shape(shape: MoEShape, **kw) -> MoEShape:
    return dataclasses.replace(shape, **kw)


# ---------------------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------------------
def _e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the E2M1 grid, saturating at 6; returns 4-bit codes (uint8)."""
    a = v.abs().float()
    # boundaries between consecutive magnitudes; ties go to the code with an even mantissa bit
    code = torch.zeros_like(a, dtype=torch.uint8)
    code += (a > 0.25).to(torch.uint8)
    code += (a >= 0.75).to(torch.uint8)
    code += (a > 1.25).to(torch.uint8)
    code += (a >= 1.75).to(torch.uint8)
    code += (a > 2.5).to(torch.uint8)
    code += (a >= 3.5).to(torch.uint8)
    code += (a > 5.0).to(torch.uint8)
    return code | ((v < 0).to(torch.uint8) << 3)


def quantize_nvfp4(w: torch.Tensor):
    """w: float [..., rows, K] (K % 16 == 0). One global scale per leading index.

    Returns (packed u8 [..., rows, K/2], scale e4m3-bits u8 [..., rows, K/16], gs f32 [...]).
    gs = amax/(6*448); block scale = e4m3_rn(amax_blk/(6*gs)); q = e2m1_rn(w/(dec(scale)*gs)).
    """
    w = w.float()
    *lead, rows, k = w.shape
    assert k % 16 == 0
    amax = w.abs().amax(dim=(-1, -2), keepdim=True).clamp_min(1e-30)
    gs = amax / (6.0 * 448.0)
    blocks = w.reshape(*lead, rows, k // 16, 16)
    amax_blk = blocks.abs().amax(dim=-1)
    s8 = (amax_blk / (6.0 * gs)).to(torch.float8_e4m3fn)
    s = s8.float()
    denom = (s * gs).unsqueeze(-1)
    q = _e2m1_codes(torch.where(denom > 0, blocks / denom.clamp_min(1e-30), torch.zeros_like(blocks)))
    q = q.reshape(*lead, rows, k)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), s8.view(torch.uint8).contiguous(), gs.reshape(*lead).contiguous()


def quantize_int4_g128(w: torch.Tensor):
    """w: float [E, O, K] (K % 128 == 0 not required; last group may be short).

    Returns (qweight i32 [E, ceil(K/8), O] GPTQ-packed uint4b8, scales bf16 [E, ceil(K/128), O]).
    s = bf16(amax_group/7), q = clamp(rn(w/s), -8, 7), stored as q + 8.
    """
    w = w.float()
    e, o, k = w.shape
    assert k % 8 == 0
    g = (k + 127) // 128
    pad = g * 128 - k
    wp = torch.nn.functional.pad(w, (0, pad)) if pad else w
    grp = wp.reshape(e, o, g, 128)
    s = (grp.abs().amax(dim=-1) / 7.0).to(torch.bfloat16)
    sf = s.float().clamp_min(1e-30).unsqueeze(-1)
    q = torch.clamp(torch.round(grp / sf), -8, 7).to(torch.int32) + 8
    q = q.reshape(e, o, g * 128)[..., :k]
    q = q.reshape(e, o, k // 8, 8)
    word = torch.zeros(e, o, k // 8, dtype=torch.int64, device=w.device)
    for j in range(8):
        word |= q[..., j].to(torch.int64) << (4 * j)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    qweight = word.permute(0, 2, 1).contiguous()          # [E, K/8, O]
    scales = s.permute(0, 2, 1).contiguous()              # [E, G, O]
    return qweight, scales


# ---------------------------------------------------------------------------------------
# layer weights and inputs
# ---------------------------------------------------------------------------------------
@dataclasses.dataclass
class LayerWeights:
    """Checkpoint-format weights of one layer (before kernel-side preparation)."""

    w13_packed: torch.Tensor   # u8 [E_tot, 2I, H/2]
    w13_scale: torch.Tensor    # u8 (e4m3 bits) [E_tot, 2I, H/16]
    w13_gs: torch.Tensor       # f32 [E_tot, 2]
    w2_qweight: torch.Tensor   # i32 [E_tot, I/8, H]  (GPTQ: [E, K/8, O])
    w2_scales: torch.Tensor    # bf16 [E_tot, ceil(I/128), H]
    router_weight: torch.Tensor  # bf16 [E, H]
    router_bias: torch.Tensor | None   # f32 [E] selection bias (grouped sigmoid routing)
    logit_bias: torch.Tensor | None    # f32 [E] added to the logits (load-imbalance skew)


def make_weights(shape: MoEShape, seed: int = 0, device: str | torch.device = "cpu",
                 std: float = 0.02) -> LayerWeights:
    """bf16 N(0, std) weights quantised to the two 4-bit formats, one expert at a time."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    dev = torch.device(device)
    h, i, et = shape.hidden, shape.inter, shape.e_tot
    w13_packed = torch.empty(et, 2 * i, h // 2, dtype=torch.uint8, device=dev)
    w13_scale = torch.empty(et, 2 * i, h // 16, dtype=torch.uint8, device=dev)
    w13_gs = torch.empty(et, 2, dtype=torch.float32, device=dev)
    g = (i + 127) // 128
    w2_q = torch.empty(et, i // 8, h, dtype=torch.int32, device=dev)
    w2_s = torch.empty(et, g, h, dtype=torch.bfloat16, device=dev)
    on_gpu = dev.type == "cuda"
    ggen = torch.Generator(device=dev).manual_seed(seed) if on_gpu else gen
    for e in range(et):
        w13 = (torch.randn(2, i, h, generator=ggen, device=dev) * std).to(torch.bfloat16)
        p, s, gs = quantize_nvfp4(w13)
        w13_packed[e] = p.reshape(2 * i, h // 2)
        w13_scale[e] = s.reshape(2 * i, h // 16)
        w13_gs[e] = gs
        w2 = (torch.randn(1, h, i, generator=ggen, device=dev) * std).to(torch.bfloat16)
        q, sc = quantize_int4_g128(w2)
        w2_q[e] = q[0]
        w2_s[e] = sc[0]
    router_w = (torch.randn(shape.num_experts, h, generator=gen) * std).to(torch.bfloat16).to(dev)
    rbias = None
    if shape.router_bias:
        rbias = (torch.randn(shape.num_experts, generator=gen) * 0.01).float().to(dev)
    lbias = None
    if shape.zipf_bias > 0:
        perm = torch.randperm(shape.num_experts, generator=gen)
        ranks = torch.empty(shape.num_experts)
        ranks[perm] = torch.arange(shape.num_experts, dtype=torch.float32)
        lbias = (-shape.zipf_bias * torch.log(ranks + 1.0)).float().to(dev)
    return LayerWeights(w13_packed, w13_scale, w13_gs, w2_q, w2_s, router_w, rbias, lbias)


def make_inputs(shape: MoEShape, weights: LayerWeights, n_tokens: int, seed: int = 0,
                device: str | torch.device = "cpu"):
    """x ~ N(0,1) bf16 [N,H]; logits = bf16(x @ Wr^T (+ skew bias)) computed once, fp32 accumulate."""
    gen = torch.Generator(device="cpu").manual_seed(seed + 1000003)
    x = torch.randn(n_tokens, shape.hidden, generator=gen).to(torch.bfloat16).to(device)
    logits = x.float() @ weights.router_weight.float().t()
    if weights.logit_bias is not None:
        logits = logits + weights.logit_bias
    return x, logits.to(torch.bfloat16)


def planted_routes(n_tokens: int, num_experts: int, top_k: int, mode: str = "uniform", seed: int = 0,
                   gate: str = "softmax"):
    """Routes fixed first, logits built so that they win: the construction of the reference's
    routing self-check (sm120a/benchmarks/benchmark.cu:94-183) restated with torch's RNG.

    Filler logits are below -3.75, winner r gets 4 - 0.5 r, so the expected top-k (in slot
    order), the expected weights and the expected packed rows follow by counting.
    Returns (logits bf16 [N,E], idx i32 [N,k], weights f32 [N,k]).
    """
    gen = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_experts, generator=gen)
    p = torch.empty(num_experts, dtype=torch.float64)
    p[perm] = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** 1.10
    idx = torch.empty(n_tokens, top_k, dtype=torch.int64)
    if mode == "uniform":
        for t in range(n_tokens):
            idx[t] = torch.randperm(num_experts, generator=gen)[:top_k]
    elif mode == "zipf":
        idx = torch.multinomial(p.expand(n_tokens, -1), top_k, replacement=False, generator=gen)
    elif mode == "burst":
        span = max(top_k * 3, max(8, num_experts // 16))
        for t0 in range(0, n_tokens, 16):
            centre = int(torch.multinomial(p, 1, generator=gen))
            local = [(centre + d - span // 2) % num_experts for d in range(span)]
            pl = torch.zeros(num_experts, dtype=torch.float64)
            pl[local] = 1.0
            mix = 0.75 * pl / pl.sum() + 0.25 * p / p.sum()
            n_here = min(16, n_tokens - t0)
            idx[t0:t0 + n_here] = torch.multinomial(mix.expand(n_here, -1), top_k, replacement=False, generator=gen)
    else:
        raise ValueError(mode)
    filler = torch.randint(0, 1024, (n_tokens, num_experts), generator=gen).float() / 4096.0 - 4.0
    logits = filler.clone()
    ranks = torch.arange(top_k, dtype=torch.float32)
    vals = 4.0 - 0.5 * ranks
    logits.scatter_(1, idx, vals.expand(n_tokens, -1))
    if gate == "sigmoid":
        w = torch.sigmoid(vals)
    else:
        w = torch.exp(vals - 4.0)
    w = (w / w.sum()).expand(n_tokens, -1).contiguous()
    return logits.to(torch.bfloat16), idx.to(torch.int32), w


def algorithmic_bytes(shape: MoEShape, n_tokens: int, live_experts: int) -> int:
    """HBM bytes one layer call has to move at minimum (weights of live experts once + activations)."""
    h, i = shape.hidden, shape.inter
    per_expert = 2 * i * h // 2 + 2 * i * h // 16 + 8 + h * i // 2 + 2 * h * math.ceil(i / 128)
    act = 4 * n_tokens * h + 2 * n_tokens * shape.num_experts + 6 * n_tokens * shape.k_eff
    return live_experts * per_expert + act


def algorithmic_flops(shape: MoEShape, n_tokens: int) -> int:
    """6*N*k*H*I (FF1 4*N*k*H*I + FF2 2*N*k*H*I), the reference's useful_tflops numerator."""
    return 6 * n_tokens * shape.k_eff * shape.hidden * shape.inter
