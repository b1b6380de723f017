"""Plugin entry point: routes NVFP4 compressed-tensors MoE layers to the B200 fused operator.

Mirrors the reference's `register()` (vllm/xcaliber_int4_vllm/plugin.py:31-139): it wraps the
static method selection `CompressedTensorsMoEMethod.get_moe_method(quant_config, layer,
layer_name)` and returns this package's method class when the layer's weight scheme is NVFP4;
everything else falls through to vLLM's own choice. Written against vLLM 0.22 (the reference
targets 0.19 and no longer imports there).
"""
from __future__ import annotations

import logging

logger = logging.getLogger(__name__)
_PATCH_FLAG = "_xcaliber_b200_registered"


def register() -> None:
    from vllm.model_executor.layers.quantization.compressed_tensors.compressed_tensors_moe.compressed_tensors_moe import (  # noqa: E501
        CompressedTensorsMoEMethod,
    )

    if getattr(CompressedTensorsMoEMethod, _PATCH_FLAG, False):
        return
    original = CompressedTensorsMoEMethod.get_moe_method

    def get_moe_method(quant_config, layer, layer_name):
        method = original(quant_config, layer, layer_name)
        try:
            from vllm.model_executor.layers.quantization.compressed_tensors.compressed_tensors_moe.compressed_tensors_moe_w4a4_nvfp4 import (  # noqa: E501
                CompressedTensorsW4A4Nvfp4MoEMethod,
            )
        except ImportError:
            return method
        if isinstance(method, CompressedTensorsW4A4Nvfp4MoEMethod):
            from .method import XCaliberB200NVFP4MoE

            logger.info("xcaliber_b200: %s -> fused NVFP4 MoE operator (sm_100a)", layer_name)
            return XCaliberB200NVFP4MoE.from_stock(method)
        return method

    CompressedTensorsMoEMethod.get_moe_method = staticmethod(get_moe_method)
    setattr(CompressedTensorsMoEMethod, _PATCH_FLAG, True)
    logger.info("xcaliber_b200 vLLM plugin registered")
