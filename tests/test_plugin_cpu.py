"""The vLLM plugin slot: registration patches method selection once, and the method class
exposes the monolithic surface the vLLM runner calls (no GPU needed)."""
import pytest


def test_plugin_registers_and_method_surface():
    pytest.importorskip("vllm")
    try:
        from xcaliber_b200.vllm_plugin import plugin
        from vllm.model_executor.layers.quantization.compressed_tensors.compressed_tensors_moe.compressed_tensors_moe import (  # noqa: E501
            CompressedTensorsMoEMethod,
        )
    except ImportError as exc:  # a vLLM build without the compressed-tensors MoE methods
        pytest.skip(str(exc))
    before = CompressedTensorsMoEMethod.get_moe_method
    plugin.register()
    patched = CompressedTensorsMoEMethod.get_moe_method
    assert patched is not before and getattr(CompressedTensorsMoEMethod, "_xcaliber_b200_registered")
    plugin.register()
    assert CompressedTensorsMoEMethod.get_moe_method is patched          # idempotent
    from xcaliber_b200.vllm_plugin.method import XCaliberB200NVFP4MoE as M

    m = M.__new__(M)
    m._xc_layer = None
    assert m.is_monolithic and m.supports_internal_mk and not m.supports_eplb
    assert m.get_fused_moe_quant_config(None) is None
    import torch

    with pytest.raises(RuntimeError):
        m.apply_monolithic(None, torch.zeros(1, 8), torch.zeros(1, 4))
    with pytest.raises(RuntimeError):
        m.apply()
