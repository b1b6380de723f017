// PyTorch custom-op registration of the fused MoE operator: `torch.ops.xmoe_b200.{forward, repack_gptq,
// prep_nvfp4_sf, build_info}`. This is the vLLM-facing counterpart of the reference's torch extension module
// (xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/vllm/csrc/xr64_abs_bridge.cu:61-242: `_C.forward`,
// `_C.repack_gptq`, `_C.build_info`), registered through TORCH_LIBRARY instead of pybind11 so that the
// dispatcher, torch.compile (through the Meta kernels below) and CUDA-graph capture see a real operator
// rather than an opaque Python call. It contains no compute: every op checks its tensors the way the
// reference's bridge does (device, dtype, contiguity, shapes), allocates output and scratch with torch's
// allocator (as xr64_abs_bridge.cu:160-173 does; the caching allocator makes that capture-safe) and calls
// the C ABI of libxmoe_b200.so on the current stream.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <string>
#include <vector>

#include "../../include/xmoe_b200.h"

namespace {

void check_cuda_contig(const at::Tensor& t, const at::Tensor& like, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
    TORCH_CHECK(t.device() == like.device(), name, " must live on the same device as x");
}

// cfg_ints: hidden, inter, num_experts, top_k, num_shared_experts, scoring, renormalize, n_group, topk_group,
//           activation, act_topk_keep, token_tile (the int fields of xmoe_config, in order)
// cfg_floats: routed_scale, swiglu_alpha, swiglu_limit
xmoe_config make_cfg(at::IntArrayRef ci, at::ArrayRef<double> cf) {
    TORCH_CHECK(ci.size() == 12 && cf.size() == 3, "cfg_ints needs 12 entries and cfg_floats 3");
    xmoe_config c;
    int32_t* p = &c.hidden;
    for (int i = 0; i < 12; ++i) p[i] = (int32_t)ci[i];
    c.routed_scale = (float)cf[0];
    c.swiglu_alpha = (float)cf[1];
    c.swiglu_limit = (float)cf[2];
    return c;
}

const void* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

at::Tensor forward_cuda(const at::Tensor& x, const at::Tensor& router_logits,
                        const c10::optional<at::Tensor>& per_expert_scale, const at::Tensor& w13_packed,
                        const at::Tensor& w13_sf, const at::Tensor& w13_gs, const at::Tensor& w2_q,
                        const at::Tensor& w2_scale, const c10::optional<at::Tensor>& router_bias,
                        const c10::optional<at::Tensor>& sigmoid_lut, at::IntArrayRef cfg_ints,
                        at::ArrayRef<double> cfg_floats) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2, "x must be a contiguous CUDA tensor [N, H]");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "x must be bf16 or fp16");
    c10::cuda::CUDAGuard guard(x.device());
    const xmoe_config cfg = make_cfg(cfg_ints, cfg_floats);
    check_cuda_contig(router_logits, x, "router_logits");
    check_cuda_contig(w13_packed, x, "w13_packed");
    check_cuda_contig(w13_sf, x, "w13_sf");
    check_cuda_contig(w13_gs, x, "w13_gs");
    check_cuda_contig(w2_q, x, "w2_q");
    check_cuda_contig(w2_scale, x, "w2_scale");
    const int64_t n = x.size(0), h = x.size(1);
    const int64_t e_tot = (int64_t)cfg.num_experts + cfg.num_shared_experts;
    TORCH_CHECK(h == cfg.hidden, "x must be [N, hidden]");
    TORCH_CHECK(router_logits.dim() == 2 && router_logits.size(0) == n && router_logits.size(1) == cfg.num_experts,
                "router_logits must be [N, num_experts]");
    TORCH_CHECK(w13_packed.scalar_type() == at::kByte && w13_packed.dim() == 3 && w13_packed.size(0) == e_tot &&
                    w13_packed.size(1) == 2 * (int64_t)cfg.inter && w13_packed.size(2) == h / 2,
                "w13_packed must be u8 [E_tot, 2I, H/2]");
    TORCH_CHECK(w13_gs.scalar_type() == at::kFloat && w13_gs.numel() == 2 * e_tot, "w13_gs must be f32 [E_tot, 2]");
    TORCH_CHECK(w2_q.scalar_type() == at::kInt && w2_q.dim() == 3 && w2_q.size(0) == e_tot && w2_q.size(1) == h &&
                    w2_q.size(2) == cfg.inter / 8,
                "w2_q must be i32 [E_tot, H, I/8] (repack_gptq output)");
    TORCH_CHECK(w2_scale.scalar_type() == at::kBFloat16 && w2_scale.dim() == 3 && w2_scale.size(0) == e_tot &&
                    w2_scale.size(1) == (cfg.inter + 127) / 128 && w2_scale.size(2) == h,
                "w2_scale must be bf16 [E_tot, ceil(I/128), H]");
    TORCH_CHECK((int64_t)w13_sf.numel() * (int64_t)w13_sf.element_size() ==
                    (int64_t)xmoe_nvfp4_sf_bytes((int32_t)(2 * e_tot), cfg.inter, cfg.hidden),
                "w13_sf must be the output of prep_nvfp4_sf");
    if (per_expert_scale.has_value() && per_expert_scale->defined()) {
        check_cuda_contig(*per_expert_scale, x, "per_expert_scale");
        TORCH_CHECK(per_expert_scale->scalar_type() == at::kBFloat16 && per_expert_scale->numel() == cfg.num_experts,
                    "per_expert_scale must be bf16 [num_experts]");
    }
    if (router_bias.has_value() && router_bias->defined()) {
        check_cuda_contig(*router_bias, x, "router_bias");
        TORCH_CHECK(router_bias->scalar_type() == at::kFloat && router_bias->numel() == cfg.num_experts,
                    "router_bias must be f32 [num_experts]");
    }
    if (sigmoid_lut.has_value() && sigmoid_lut->defined()) {
        check_cuda_contig(*sigmoid_lut, x, "sigmoid_lut");
        TORCH_CHECK(sigmoid_lut->scalar_type() == at::kFloat && sigmoid_lut->numel() == 65536,
                    "sigmoid_lut must be f32 [65536]");
    }
    if (n == 0) return at::empty_like(x);
    // fp16 callers are served in bf16 like the reference's bridge (xr64_abs_bridge.cu:127-137)
    const at::Tensor xb = x.scalar_type() == at::kBFloat16 ? x : x.to(at::kBFloat16);
    const at::Tensor lb =
        router_logits.scalar_type() == at::kBFloat16 ? router_logits : router_logits.to(at::kBFloat16).contiguous();
    const size_t ws_bytes = xmoe_workspace_bytes(&cfg, (int32_t)n);
    TORCH_CHECK(ws_bytes > 0, "unsupported MoE configuration");
    at::Tensor raw = at::empty({(int64_t)ws_bytes + 1024}, x.options().dtype(at::kByte));
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw.data_ptr()) + 1023) & ~(uintptr_t)1023);
    at::Tensor y = at::empty_like(xb);
    xmoe_weights w;
    w.w13_packed = w13_packed.data_ptr();
    w.w13_sf = w13_sf.data_ptr();
    w.w13_gs = w13_gs.data_ptr<float>();
    w.w2_q = w2_q.data_ptr();
    w.w2_scale = w2_scale.data_ptr();
    w.router_bias = static_cast<const float*>(opt_ptr(router_bias));
    w.expert_scale = opt_ptr(per_expert_scale);
    w.sigmoid_lut = static_cast<const float*>(opt_ptr(sigmoid_lut));
    const int rc = xmoe_forward(&cfg, &w, xb.data_ptr(), lb.data_ptr(), (int32_t)n, y.data_ptr(), ws, ws_bytes,
                                c10::cuda::getCurrentCUDAStream(x.get_device()).stream());
    TORCH_CHECK(rc == XMOE_OK, "xmoe_forward: ", xmoe_status_string(rc));
    return x.scalar_type() == at::kBFloat16 ? y : y.to(x.scalar_type());
}

at::Tensor forward_meta(const at::Tensor& x, const at::Tensor&, const c10::optional<at::Tensor>&, const at::Tensor&,
                        const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                        const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, at::IntArrayRef,
                        at::ArrayRef<double>) {
    return at::empty_like(x);
}

at::Tensor repack_gptq_cuda(const at::Tensor& qweight) {
    TORCH_CHECK(qweight.is_cuda() && qweight.is_contiguous() && qweight.scalar_type() == at::kInt && qweight.dim() == 3,
                "qweight must be a contiguous CUDA int32 tensor [E, K/8, O]");
    c10::cuda::CUDAGuard guard(qweight.device());
    const int64_t e = qweight.size(0), k8 = qweight.size(1), o = qweight.size(2);
    at::Tensor out = at::empty({e, o, k8}, qweight.options());
    const int rc = xmoe_repack_gptq(qweight.data_ptr(), out.data_ptr(), (int32_t)e, (int32_t)(k8 * 8), (int32_t)o,
                                    c10::cuda::getCurrentCUDAStream(qweight.get_device()).stream());
    TORCH_CHECK(rc == XMOE_OK, "xmoe_repack_gptq: ", xmoe_status_string(rc));
    return out;
}
at::Tensor repack_gptq_meta(const at::Tensor& q) { return at::empty({q.size(0), q.size(2), q.size(1)}, q.options()); }

at::Tensor prep_nvfp4_sf_cuda(const at::Tensor& scale, int64_t rows_per_mat) {
    TORCH_CHECK(scale.is_cuda() && scale.is_contiguous() && scale.element_size() == 1 && scale.dim() >= 2,
                "scale must be a contiguous CUDA tensor of E4M3 bytes [..., rows, K/16]");
    c10::cuda::CUDAGuard guard(scale.device());
    const int64_t k = scale.size(-1) * 16;
    TORCH_CHECK(rows_per_mat > 0 && scale.numel() % (rows_per_mat * scale.size(-1)) == 0, "rows_per_mat does not divide the tensor");
    const int64_t n_mats = scale.numel() / (rows_per_mat * scale.size(-1));
    const size_t bytes = xmoe_nvfp4_sf_bytes((int32_t)n_mats, (int32_t)rows_per_mat, (int32_t)k);
    at::Tensor out = at::empty({(int64_t)bytes}, scale.options().dtype(at::kByte));
    const int rc = xmoe_prep_nvfp4_sf(scale.data_ptr(), out.data_ptr(), (int32_t)n_mats, (int32_t)rows_per_mat, (int32_t)k,
                                      c10::cuda::getCurrentCUDAStream(scale.get_device()).stream());
    TORCH_CHECK(rc == XMOE_OK, "xmoe_prep_nvfp4_sf: ", xmoe_status_string(rc));
    return out;
}
at::Tensor prep_nvfp4_sf_meta(const at::Tensor& scale, int64_t rows_per_mat) {
    const int64_t n_mats = scale.numel() / (rows_per_mat * scale.size(-1));
    return at::empty({(int64_t)xmoe_nvfp4_sf_bytes((int32_t)n_mats, (int32_t)rows_per_mat, (int32_t)(scale.size(-1) * 16))},
                     scale.options().dtype(at::kByte));
}

std::string build_info() { return xmoe_build_info(); }

}  // namespace

TORCH_LIBRARY(xmoe_b200, m) {
    m.def(
        "forward(Tensor x, Tensor router_logits, Tensor? per_expert_scale, Tensor w13_packed, Tensor w13_sf, "
        "Tensor w13_gs, Tensor w2_q, Tensor w2_scale, Tensor? router_bias, Tensor? sigmoid_lut, int[] cfg_ints, "
        "float[] cfg_floats) -> Tensor");
    m.def("repack_gptq(Tensor qweight) -> Tensor");
    m.def("prep_nvfp4_sf(Tensor scale_e4m3, int rows_per_mat) -> Tensor");
    m.def("build_info() -> str", &build_info);
}

TORCH_LIBRARY_IMPL(xmoe_b200, CUDA, m) {
    m.impl("forward", &forward_cuda);
    m.impl("repack_gptq", &repack_gptq_cuda);
    m.impl("prep_nvfp4_sf", &prep_nvfp4_sf_cuda);
}

TORCH_LIBRARY_IMPL(xmoe_b200, Meta, m) {
    m.impl("forward", &forward_meta);
    m.impl("repack_gptq", &repack_gptq_meta);
    m.impl("prep_nvfp4_sf", &prep_nvfp4_sf_meta);
}
