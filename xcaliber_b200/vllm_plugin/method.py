"""FusedMoE quant method backed by the B200 fused operator.

Surface and error behaviour mirror the reference's method classes
(vllm/xcaliber_int4_vllm/method.py:32-45 properties, :129-238 weight post-processing,
:240-264 apply_monolithic): monolithic (the operator owns routing), no expert map, no router
weight on the input, parallel sizes other than expert parallelism must be 1. Weights arrive in
vLLM's compressed-tensors NVFP4 parameter set (w13_weight_packed u8 [E, 2I, H/2],
w13_weight_scale e4m3 [E, 2I, H/16], w13_weight_global_scale f32 [E, 2], w2_* likewise); FF1
uses them as they are, FF2 is converted once at load time to int4 group-128 for the W4A16
down projection. At run time the layer goes through the registered PyTorch custom op
`torch.ops.xmoe_b200.forward` (torch_ops.py), the counterpart of the reference's `_C.forward`.
"""
from __future__ import annotations

import torch
from vllm.model_executor.layers.quantization.compressed_tensors.compressed_tensors_moe.compressed_tensors_moe_w4a4_nvfp4 import (  # noqa: E501
    CompressedTensorsW4A4Nvfp4MoEMethod,
)

from .. import ops, synth, torch_ops

_ACTIVATIONS = {"silu": "silu", "swigluoai": "swiglu_clamp", "gelu_tanh": "gelu_tanh"}


def _nvfp4_to_float(packed: torch.Tensor, scale_e4m3: torch.Tensor, dequant_gs: torch.Tensor) -> torch.Tensor:
    """[rows, K/2] u8 + [rows, K/16] e4m3 + scalar -> f32 [rows, K] (load-time helper)."""
    lut = torch.tensor(synth.E2M1_VALUES + tuple(-v for v in synth.E2M1_VALUES), device=packed.device)
    lo, hi = (packed & 0xF).long(), (packed >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).reshape(packed.shape[0], -1)
    s = scale_e4m3.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1)
    return vals * s * dequant_gs


def convert_w2_nvfp4_to_int4(w2_packed: torch.Tensor, w2_scale: torch.Tensor, w2_dequant_gs: torch.Tensor):
    """The down projection of an NVFP4 checkpoint -> the int4 group-128 contract of the W4A16 kernel (GPTQ
    packing, xR64ABSRepack.cu:3-24): u8 [E, H, I/2] + e4m3 [E, H, I/16] + f32 [E] -> (qweight i32 [E, I/8, H],
    scales bf16 [E, ceil(I/128), H]). One expert at a time (the float copy of an expert is transient)."""
    e, h, half_i = w2_packed.shape
    i = half_i * 2
    dev = w2_packed.device
    w2_q = torch.empty(e, i // 8, h, dtype=torch.int32, device=dev)
    w2_s = torch.empty(e, (i + 127) // 128, h, dtype=torch.bfloat16, device=dev)
    for ex in range(e):
        wf = _nvfp4_to_float(w2_packed[ex], w2_scale[ex], w2_dequant_gs[ex])
        q, s = synth.quantize_int4_g128(wf.unsqueeze(0))
        w2_q[ex], w2_s[ex] = q[0], s[0]
    return w2_q, w2_s


class XCaliberB200NVFP4MoE(CompressedTensorsW4A4Nvfp4MoEMethod):
    """create_weights is inherited (same parameters as stock vLLM, so checkpoints load unchanged)."""

    @classmethod
    def from_stock(cls, stock: CompressedTensorsW4A4Nvfp4MoEMethod) -> "XCaliberB200NVFP4MoE":
        self = cls.__new__(cls)
        self.__dict__.update(stock.__dict__)
        self._xc_layer = None
        return self

    # ---- properties the runner reads (reference: method.py:32-45) ---------------------------
    @property
    def is_monolithic(self) -> bool:
        return True

    @property
    def supports_internal_mk(self) -> bool:
        return True

    @property
    def supports_eplb(self) -> bool:
        return False

    def get_fused_moe_quant_config(self, layer):
        return None

    def maybe_make_prepare_finalize(self, *args, **kwargs):
        return None

    # ---- load time ------------------------------------------------------------------------------
    def process_weights_after_loading(self, layer) -> None:
        pc = self.moe.moe_parallel_config
        for name in ("tp_size", "dp_size", "pcp_size", "sp_size"):
            if getattr(pc, name, 1) != 1:
                raise RuntimeError(f"xcaliber_b200 fused MoE needs {name} == 1 (got {getattr(pc, name)})")
        if getattr(layer, "expert_map", None) is not None:
            raise RuntimeError("xcaliber_b200 fused MoE does not take an expert_map; use its own expert-parallel path")
        if getattr(layer, "apply_router_weight_on_input", False):
            raise RuntimeError("apply_router_weight_on_input is not supported: gate weights are applied after SwiGLU")
        act = _ACTIVATIONS.get(str(getattr(layer, "activation", "silu")).lower().split(".")[-1])
        if act is None:
            raise RuntimeError(f"unsupported activation {layer.activation!r}")
        e, two_i, half_h = layer.w13_weight_packed.shape
        h, i = half_h * 2, two_i // 2
        scoring = getattr(layer, "scoring_func", "softmax")
        n_group = int(getattr(layer, "num_expert_group", None) or 1)
        bias = getattr(layer, "e_score_correction_bias", None)
        shape = synth.MoEShape(
            "vllm", h, i, e, int(layer.top_k), scoring=scoring, renormalize=bool(getattr(layer, "renormalize", True)),
            n_group=n_group, topk_group=int(getattr(layer, "topk_group", None) or 1),
            routed_scale=float(getattr(layer, "routed_scaling_factor", 1.0) or 1.0), activation=act,
            swiglu_limit=float(getattr(layer, "swiglu_limit", None) or 7.0), router_bias=bias is not None)
        dev = layer.w13_weight_packed.device
        # compressed-tensors stores the quantisation multiplier; the kernels want the dequant one
        w13_gs = (1.0 / layer.w13_weight_global_scale.data.float()).reshape(e, 2)
        w2_gs = (1.0 / layer.w2_weight_global_scale.data.float()).reshape(e)
        w2_q, w2_s = convert_w2_nvfp4_to_int4(layer.w2_weight_packed.data, layer.w2_weight_scale.data, w2_gs)
        pw = ops.PreparedWeights.from_checkpoint(
            shape, layer.w13_weight_packed.data, layer.w13_weight_scale.data.view(torch.uint8), w13_gs, w2_q, w2_s,
            router_bias=None if bias is None else bias.data, expert_scale=getattr(layer, "_xcaliber_per_expert_scale", None),
            device=dev)
        self._xc_layer = ops.FusedMoE(shape, pw)
        # the stock parameters are no longer needed on the device
        for name in ("w2_weight_packed", "w2_weight_scale"):
            getattr(layer, name).data = torch.empty(0, device=dev, dtype=getattr(layer, name).dtype)

    # ---- run time (reference: method.py:240-264) ------------------------------------------
    def apply_monolithic(self, layer, x: torch.Tensor, router_logits: torch.Tensor, input_ids=None) -> torch.Tensor:
        if self._xc_layer is None:
            raise RuntimeError("weights were not post-processed: process_weights_after_loading has not run")
        if x.numel() == 0:
            return torch.empty_like(x)
        # the registered custom op (torch.ops.xmoe_b200.forward): output and scratch come from torch's allocator
        # inside the op, fp16 activations are served in bf16 there, as in the reference's bridge
        return torch_ops.forward(self._xc_layer, x.contiguous(), router_logits.to(torch.bfloat16).contiguous())

    def apply(self, *args, **kwargs):
        raise RuntimeError("xcaliber_b200 fused MoE is monolithic: the runner must call apply_monolithic")
