"""`torch.ops.xmoe_b200.*`: the fused MoE operator as a registered PyTorch custom op.

The counterpart of the reference's `_C` torch-extension module
(sm75/xR64/vllm/csrc/xr64_abs_bridge.cu:234-242: forward / repack_gptq / build_info) that its vLLM
method calls (vllm/xcaliber_int4_vllm/method.py:240-264). The ops are registered with TORCH_LIBRARY
by libxmoe_torch_ops.so (csrc/torch_op.cpp, host code over the C ABI of libxmoe_b200.so); they carry
Meta kernels, so torch.compile and fake-tensor tracing see their output shapes. There is no fallback:
a missing library raises.
"""
from __future__ import annotations

from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent / "libxmoe_torch_ops.so"
_loaded = False


def load() -> None:
    """Registers the ops (once per process)."""
    global _loaded
    if _loaded:
        return
    if not _LIB.exists():
        raise RuntimeError(f"{_LIB} is missing: build it with `python -m xcaliber_b200.csrc.build` (there is no fallback)")
    torch.ops.load_library(str(_LIB))
    _loaded = True


def cfg_lists(cfg) -> tuple[list[int], list[float]]:
    """The int and float fields of an XMoEConfig, in declaration order, as the op takes them."""
    ints = [int(getattr(cfg, name)) for name, ctype in cfg._fields_[:12]]
    floats = [float(getattr(cfg, name)) for name, ctype in cfg._fields_[12:]]
    return ints, floats


def forward(layer, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
    """`torch.ops.xmoe_b200.forward` on the weights of an ops.FusedMoE (output and scratch come from torch's
    allocator inside the op, like the reference's `_C.forward`)."""
    load()
    w = layer.weights
    ints, floats = cfg_lists(layer.cfg)
    return torch.ops.xmoe_b200.forward(x, router_logits, w.expert_scale, w.w13_packed, w.w13_sf, w.w13_gs, w.w2_q,
                                       w.w2_scale, w.router_bias, w.lut, ints, floats)


def repack_gptq(qweight: torch.Tensor) -> torch.Tensor:
    load()
    return torch.ops.xmoe_b200.repack_gptq(qweight)


def build_info() -> str:
    load()
    return torch.ops.xmoe_b200.build_info()
