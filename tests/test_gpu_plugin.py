"""The vLLM boundary on a GPU: the registered custom op, and the plugin's weight path end to end on a stand-in
FusedMoE layer that carries vLLM's compressed-tensors NVFP4 parameter set."""
import types

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests import helpers as Hh
from tests.test_gpu_layer import MAX_REL, MEAN_REL
from xcaliber_b200 import synth

pytestmark = pytest.mark.gpu


def test_custom_op_matches_c_abi_and_has_meta_kernels():
    from xcaliber_b200 import torch_ops

    shape = synth.SHAPES["toy"]
    w, layer = Hh.build_layer(shape)
    x, logits = synth.make_inputs(shape, w, 72)
    xd, ld = x.cuda(), logits.cuda()
    y_abi = layer.forward(xd, ld)
    y_op = torch_ops.forward(layer, xd, ld)
    assert torch.equal(y_op, y_abi)
    # fp16 activations are served in bf16 and handed back as fp16 (the reference bridge does the same)
    y16 = torch_ops.forward(layer, xd.to(torch.float16), ld)
    assert y16.dtype == torch.float16
    assert torch.equal(y16, layer.forward(xd.to(torch.float16).to(torch.bfloat16), ld).to(torch.float16))
    assert torch_ops.forward(layer, xd[:0], ld[:0]).shape == (0, shape.hidden)
    assert "sm_100a" in torch_ops.build_info()
    # shape inference without data: what torch.compile / fake tensors use
    ints, floats = torch_ops.cfg_lists(layer.cfg)
    wts = layer.weights
    meta = lambda t: None if t is None else torch.empty_like(t, device="meta")  # noqa: E731
    ym = torch.ops.xmoe_b200.forward(meta(xd), meta(ld), None, meta(wts.w13_packed), meta(wts.w13_sf), meta(wts.w13_gs),
                                     meta(wts.w2_q), meta(wts.w2_scale), None, None, ints, floats)
    assert ym.device.type == "meta" and ym.shape == xd.shape and ym.dtype == xd.dtype
    # argument errors surface as RuntimeError, like TORCH_CHECK in the reference bridge
    with pytest.raises(RuntimeError):
        torch_ops.forward(layer, xd[:, :-8].contiguous(), ld)
    # CUDA-graph capture of the op (output and scratch come from torch's capture-aware allocator)
    torch_ops.forward(layer, xd, ld)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y_cap = torch_ops.forward(layer, xd, ld)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_cap, y_abi)


def test_plugin_weight_path_and_apply_monolithic():
    pytest.importorskip("vllm")
    try:
        from xcaliber_b200.vllm_plugin import method as M
    except ImportError as exc:  # a vLLM build without the compressed-tensors NVFP4 MoE method
        pytest.skip(str(exc))
    shape = synth.scaled_shape(synth.SHAPES["toy"], hidden=512, inter=384, num_experts=8, top_k=2)
    e, h, i = shape.num_experts, shape.hidden, shape.inter
    base = synth.make_weights(shape, seed=2, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(7)
    w2 = (torch.randn(e, h, i, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    w2_packed, w2_scale, w2_gs = synth.quantize_nvfp4(w2)

    # the parameters vLLM's compressed-tensors NVFP4 MoE method creates
    # (compressed_tensors_moe_w4a4_nvfp4.py: create_weights); global scales are stored as the quantisation multiplier
    layer = torch.nn.Module()
    par = lambda t: torch.nn.Parameter(t, requires_grad=False)  # noqa: E731
    layer.w13_weight_packed = par(base.w13_packed.clone())
    layer.w13_weight_scale = par(base.w13_scale.clone().view(torch.float8_e4m3fn))
    layer.w13_weight_global_scale = par(1.0 / base.w13_gs)
    layer.w13_input_global_scale = par(torch.ones(e, 2, device="cuda"))
    layer.w2_weight_packed = par(w2_packed.clone())
    layer.w2_weight_scale = par(w2_scale.clone().view(torch.float8_e4m3fn))
    layer.w2_weight_global_scale = par(1.0 / w2_gs)
    layer.w2_input_global_scale = par(torch.ones(e, device="cuda"))
    layer.top_k, layer.activation, layer.renormalize, layer.scoring_func = shape.top_k, "silu", True, "softmax"
    layer.expert_map, layer.apply_router_weight_on_input = None, False

    m = M.XCaliberB200NVFP4MoE.__new__(M.XCaliberB200NVFP4MoE)
    m._xc_layer = None
    par_cfg = types.SimpleNamespace(tp_size=1, dp_size=1, pcp_size=1, sp_size=1, ep_size=1)
    m.moe = types.SimpleNamespace(moe_parallel_config=par_cfg)
    # what the oracle dequantises: the same conversion of the down projection, computed here first because the
    # method frees the stock w2 parameters
    # (the dequant multipliers are the reciprocals of the stored ones, as the method computes them)
    w2_dq = (1.0 / layer.w2_weight_global_scale.data.float()).reshape(e)
    w13_dq = (1.0 / layer.w13_weight_global_scale.data.float()).reshape(e, 2)
    w2_q, w2_s = M.convert_w2_nvfp4_to_int4(w2_packed, w2_scale.view(torch.float8_e4m3fn), w2_dq)
    m.process_weights_after_loading(layer)
    assert layer.w2_weight_packed.numel() == 0

    w_cpu = synth.LayerWeights(base.w13_packed.cpu(), base.w13_scale.cpu(), w13_dq.cpu(), w2_q.cpu(), w2_s.cpu(),
                               base.router_weight.cpu(), None, None)
    for n in (5, 300):
        x, logits = synth.make_inputs(shape, w_cpu, n, seed=n)
        y = m.apply_monolithic(layer, x.cuda(), logits.cuda().float())   # vLLM hands over fp32 or bf16 logits
        ref = O.layer_forward(x, logits, w_cpu, shape)
        mx, mean = O.rel_errors(y.float().cpu(), ref["y"].float())
        assert mx <= MAX_REL and mean <= MEAN_REL, (n, mx, mean)
    assert m.apply_monolithic(layer, x.cuda()[:0], logits.cuda()[:0]).shape == (0, h)
    # refusals of the reference's method (method.py:130-154) keep their meaning
    layer.expert_map = torch.zeros(e, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        m.process_weights_after_loading(layer)
    layer.expert_map = None
    par_cfg.tp_size = 2
    with pytest.raises(RuntimeError):
        m.process_weights_after_loading(layer)
