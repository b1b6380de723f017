"""Host side of the fused MoE operator: the Python mirror of the reference's `_C` module
(sm75/xR64/vllm/csrc/xr64_abs_bridge.cu:61-242: forward / repack_gptq / build_info) on top
of the C ABI. torch is used for device memory and streams only; all compute is in
libxmoe_b200.so, and a missing library or a failed call raises.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

import torch

from . import _lib
from ._lib import XMoEConfig, XMoEWeights, XMoEWorkspaceView, check
from .synth import MoEShape

_ACT = {"silu": 0, "swiglu_clamp": 1, "gelu_tanh": 2}
_SCORE = {"softmax": 0, "sigmoid": 1}


def build_info() -> str:
    return _lib.lib().xmoe_build_info().decode()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def make_config(shape: MoEShape, token_tile: int = 0) -> XMoEConfig:
    return XMoEConfig(
        hidden=shape.hidden, inter=shape.inter, num_experts=shape.num_experts, top_k=shape.top_k,
        num_shared_experts=shape.num_shared_experts, scoring=_SCORE[shape.scoring],
        renormalize=int(shape.renormalize), n_group=shape.n_group, topk_group=shape.topk_group,
        activation=_ACT[shape.activation], act_topk_keep=shape.act_topk_keep, token_tile=token_tile,
        routed_scale=shape.routed_scale, swiglu_alpha=shape.swiglu_alpha, swiglu_limit=shape.swiglu_limit)


def sigmoid_lut(device) -> torch.Tensor:
    host = torch.empty(65536, dtype=torch.float32)
    _lib.lib().xmoe_fill_sigmoid_lut(host.data_ptr())
    return host.to(device)


def repack_gptq(qweight: torch.Tensor) -> torch.Tensor:
    """GPTQ int32 [E, K/8, O] (uint4b8) -> int32 [E, O, K/8] in the FF2 kernel's nibble order.
    Same call shape as the reference's `_C.repack_gptq` (xr64_abs_bridge.cu:61-79)."""
    if qweight.dim() != 3 or qweight.dtype != torch.int32 or not qweight.is_cuda:
        raise RuntimeError("repack_gptq expects a CUDA int32 tensor [E, K/8, O]")
    q = qweight.contiguous()
    e, k8, o = q.shape
    out = torch.empty(e, o, k8, dtype=torch.int32, device=q.device)
    check(_lib.lib().xmoe_repack_gptq(q.data_ptr(), out.data_ptr(), e, k8 * 8, o, _stream()), "xmoe_repack_gptq")
    return out


def prep_nvfp4_sf(scale_e4m3: torch.Tensor, rows_per_mat: int) -> torch.Tensor:
    """E4M3 block scales u8 [..., rows, K/16] -> tiled scale factors for the block-scaled MMA.
    The leading dims times (rows / rows_per_mat) matrices are padded to 128 rows each."""
    s = scale_e4m3.contiguous().view(torch.uint8)
    k = s.shape[-1] * 16
    n_mats = s.numel() // (rows_per_mat * s.shape[-1])
    nbytes = _lib.lib().xmoe_nvfp4_sf_bytes(n_mats, rows_per_mat, k)
    out = torch.empty(nbytes, dtype=torch.uint8, device=s.device)
    check(_lib.lib().xmoe_prep_nvfp4_sf(s.data_ptr(), out.data_ptr(), n_mats, rows_per_mat, k, _stream()),
          "xmoe_prep_nvfp4_sf")
    return out


@dataclasses.dataclass
class PreparedWeights:
    """Device-resident weights in kernel layout. Keeps every tensor alive."""

    w13_packed: torch.Tensor
    w13_sf: torch.Tensor
    w13_gs: torch.Tensor
    w2_q: torch.Tensor
    w2_scale: torch.Tensor
    router_bias: torch.Tensor | None = None
    expert_scale: torch.Tensor | None = None
    lut: torch.Tensor | None = None

    @classmethod
    def from_checkpoint(cls, shape: MoEShape, w13_packed, w13_scale, w13_gs, w2_qweight, w2_scales,
                        router_bias=None, expert_scale=None, device="cuda") -> "PreparedWeights":
        dev = torch.device(device)
        w13_packed = w13_packed.to(dev).contiguous()
        sf = prep_nvfp4_sf(w13_scale.to(dev), shape.inter)
        w2_q = repack_gptq(w2_qweight.to(dev))
        lut = None
        rb = None
        if router_bias is not None or shape.n_group > 1:
            lut = sigmoid_lut(dev)
            rb = None if router_bias is None else router_bias.to(dev).float().contiguous()
        es = None if expert_scale is None else expert_scale.to(dev).to(torch.bfloat16).contiguous()
        return cls(w13_packed, sf, w13_gs.to(dev).float().contiguous(), w2_q,
                   w2_scales.to(dev).to(torch.bfloat16).contiguous(), rb, es, lut)

    def as_struct(self) -> XMoEWeights:
        return XMoEWeights(_ptr(self.w13_packed), _ptr(self.w13_sf), _ptr(self.w13_gs), _ptr(self.w2_q),
                           _ptr(self.w2_scale), _ptr(self.router_bias), _ptr(self.expert_scale), _ptr(self.lut))


class FusedMoE:
    """One MoE layer bound to prepared weights. `forward(x, router_logits)` is the call the
    reference exposes as `_C.forward` (xr64_abs_bridge.cu:81-232); scratch is cached per
    batch size instead of being allocated per call."""

    def __init__(self, shape: MoEShape, weights: PreparedWeights, token_tile: int = 0):
        self.shape = shape
        self.weights = weights
        self.cfg = make_config(shape, token_tile)
        self._wstruct = weights.as_struct()
        self._ws: dict[tuple[int, bool], torch.Tensor] = {}
        self.kernel_launches_per_forward = 8 + (1 if 0 < shape.act_topk_keep < shape.inter else 0)

    # -- workspace ---------------------------------------------------------------------
    def workspace(self, n: int, host_io: bool = False) -> torch.Tensor:
        key = (n, host_io)
        ws = self._ws.get(key)
        if ws is None:
            fn = _lib.lib().xmoe_workspace_bytes_host_io if host_io else _lib.lib().xmoe_workspace_bytes
            nbytes = fn(C.byref(self.cfg), n)
            if nbytes == 0:
                raise RuntimeError("unsupported MoE configuration")
            raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=self.weights.w13_packed.device)
            off = (-raw.data_ptr()) % 1024
            ws = raw[off:off + nbytes]
            self._ws[key] = ws
        return ws

    def view(self, n: int, host_io: bool = False) -> dict:
        """Typed torch views of the workspace intermediates of the last forward with n tokens."""
        ws = self.workspace(n, host_io)
        v = XMoEWorkspaceView()
        check(_lib.lib().xmoe_workspace_view_get(C.byref(self.cfg), n, ws.data_ptr(), ws.numel(), C.byref(v)),
              "xmoe_workspace_view_get")
        base = ws.data_ptr()
        sh = self.shape

        def t(ptr, nbytes, dtype, *dims):
            return ws[ptr - base: ptr - base + nbytes].view(dtype).reshape(*dims)

        r, ke = v.packed_rows, v.k_eff
        return dict(
            status=t(v.status, 4, torch.int32, 1), act_scale=t(v.act_scale, 12, torch.float32, 3),
            topk_idx=t(v.topk_idx, n * ke * 4, torch.int32, n, ke), topk_w=t(v.topk_w, n * ke * 2, torch.bfloat16, n, ke),
            topk_off=t(v.topk_off, n * ke * 4, torch.int32, n, ke), topk_row=t(v.topk_row, n * ke * 4, torch.int32, n, ke),
            counts=t(v.counts, sh.e_tot * 4, torch.int32, sh.e_tot),
            offsets=t(v.offsets, (sh.e_tot + 1) * 4, torch.int32, sh.e_tot + 1),
            row_token=t(v.row_token, r * 4, torch.int32, r), row_weight=t(v.row_weight, r * 2, torch.bfloat16, r),
            xq=t(v.xq, r * sh.hidden // 2, torch.uint8, r, sh.hidden // 2),
            sfx=t(v.sfx, (r // v.token_tile) * v.kb_pad * 512, torch.uint8, r // v.token_tile, v.kb_pad, 512),
            yact=t(v.yact, r * sh.inter * 2, torch.bfloat16, r, sh.inter),
            out_rows=t(v.out_rows, r * sh.hidden * 2, torch.bfloat16, r, sh.hidden),
            token_tile=v.token_tile, packed_rows=r, k_eff=ke, kb_pad=v.kb_pad)

    # -- calls ---------------------------------------------------------------------------
    def _check_x(self, x: torch.Tensor, logits: torch.Tensor | None):
        if x.dim() != 2 or x.shape[1] != self.shape.hidden or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise RuntimeError("x must be a contiguous bf16 tensor [N, hidden]")
        if logits is not None and (logits.shape != (x.shape[0], self.shape.num_experts)
                                   or logits.dtype != torch.bfloat16 or not logits.is_contiguous()):
            raise RuntimeError("router_logits must be a contiguous bf16 tensor [N, num_experts]")

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        self._check_x(x, router_logits)
        n = x.shape[0]
        y = torch.empty_like(x) if out is None else out
        if n == 0:
            return y
        ws = self.workspace(n)
        check(_lib.lib().xmoe_forward(C.byref(self.cfg), C.byref(self._wstruct), x.data_ptr(), router_logits.data_ptr(),
                                      n, y.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "xmoe_forward")
        return y

    def forward_gated(self, x: torch.Tensor, gate_weight: torch.Tensor, out: torch.Tensor | None = None,
                      keep_logits: bool = False) -> torch.Tensor:
        """The layer with the router gate inside: gate_weight bf16 [num_experts, hidden]. One kernel runs the gate
        GEMM and the router; the logits reach HBM only with keep_logits (then in `self.last_logits`, bf16
        [N, num_experts])."""
        self._check_x(x, None)
        n = x.shape[0]
        y = torch.empty_like(x) if out is None else out
        if n == 0:
            return y
        gw = gate_weight.to(torch.bfloat16).contiguous()
        self.last_logits = (torch.empty(n, self.shape.num_experts, dtype=torch.bfloat16, device=x.device)
                            if keep_logits else None)
        ws = self.workspace(n)
        check(_lib.lib().xmoe_forward_gated(C.byref(self.cfg), C.byref(self._wstruct), x.data_ptr(), gw.data_ptr(),
                                            _ptr(self.last_logits), n, y.data_ptr(), ws.data_ptr(), ws.numel(),
                                            _stream()), "xmoe_forward_gated")
        return y

    def forward_routed(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                       act_scale: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Routing supplied by the caller (the reference's `operator(...)`, xR64ABSBinding.cu:8-121).
        act_scale: optional device f32 [2] (XGS, XGSINV) used instead of this batch's own amax."""
        self._check_x(x, None)
        n = x.shape[0]
        y = torch.empty_like(x) if out is None else out
        if n == 0:
            return y
        idx = topk_idx.to(torch.int32).contiguous()
        w = topk_w.to(torch.bfloat16).contiguous()
        ws = self.workspace(n)
        check(_lib.lib().xmoe_forward_routed(C.byref(self.cfg), C.byref(self._wstruct), x.data_ptr(), idx.data_ptr(),
                                             w.data_ptr(), _ptr(act_scale), n, y.data_ptr(), ws.data_ptr(),
                                             ws.numel(), _stream()),
              "xmoe_forward_routed")
        return y

    def forward_routed_rows(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                            act_scale: torch.Tensor | None = None, n_valid: torch.Tensor | None = None) -> None:
        """forward_routed without the final combine: the FF2 rows stay in the workspace
        (view(n)["out_rows"], indexed by view(n)["topk_row"]). topk_idx / topk_w must already be
        int32 / bf16 and contiguous; an expert id of -1 marks a slot that is not in use. n_valid
        (device int32 [1], optional): only the first n_valid rows are in use."""
        n = x.shape[0]
        if n == 0:
            return
        if topk_idx.dtype != torch.int32 or topk_w.dtype != torch.bfloat16:
            raise TypeError("topk_idx must be int32 and topk_w bf16")
        ws = self.workspace(n)
        check(_lib.lib().xmoe_forward_routed_bounded(C.byref(self.cfg), C.byref(self._wstruct), x.data_ptr(),
                                                     topk_idx.data_ptr(), topk_w.data_ptr(), _ptr(act_scale), n,
                                                     _ptr(n_valid), None, ws.data_ptr(), ws.numel(), _stream()),
              "xmoe_forward_routed_bounded")

    def forward_scatter(self, x: torch.Tensor, rows_out: torch.Tensor, router_logits: torch.Tensor | None = None,
                        topk_idx: torch.Tensor | None = None, topk_w: torch.Tensor | None = None,
                        act_scale: torch.Tensor | None = None) -> torch.Tensor:
        """The layer without its combine: FF2 row (token, slot) lands at rows_out[token * k_eff + slot] (bf16
        [>= N * k_eff, hidden], contiguous), written by the FF2 epilogue itself. Routing from router_logits, or
        supplied (topk_idx int32 / topk_w bf16, both [N, top_k], contiguous)."""
        self._check_x(x, router_logits)
        n = x.shape[0]
        if n == 0:
            return rows_out
        if rows_out.dtype != torch.bfloat16 or not rows_out.is_contiguous() or \
                rows_out.numel() < n * self.shape.k_eff * self.shape.hidden:
            raise RuntimeError("rows_out must be a contiguous bf16 buffer of at least N * k_eff rows")
        ws = self.workspace(n)
        check(_lib.lib().xmoe_forward_scatter(C.byref(self.cfg), C.byref(self._wstruct), x.data_ptr(), _ptr(router_logits),
                                              _ptr(topk_idx), _ptr(topk_w), _ptr(act_scale), n, rows_out.data_ptr(),
                                              ws.data_ptr(), ws.numel(), _stream()), "xmoe_forward_scatter")
        return rows_out

    def forward_host(self, x_host: torch.Tensor, logits_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        """Host (pinned) buffers in and out; copies and the stream sync happen inside the C call."""
        n = x_host.shape[0]
        ws = self.workspace(n, host_io=True)
        check(_lib.lib().xmoe_forward_host(C.byref(self.cfg), C.byref(self._wstruct), x_host.data_ptr(),
                                           logits_host.data_ptr(), n, y_host.data_ptr(), ws.data_ptr(), ws.numel(),
                                           _stream()), "xmoe_forward_host")
        return y_host

    def forward_host_async(self, x_host: torch.Tensor, logits_host: torch.Tensor, y_host: torch.Tensor, slot: int = 0,
                           stream: "torch.cuda.Stream | None" = None) -> None:
        """forward_host without the final synchronisation, on `stream` (default: the current one). `slot` selects
        one of several independent workspaces so that calls on different streams can be in flight together;
        y_host is valid after the caller has synchronised the stream. Buffers must be pinned."""
        n = x_host.shape[0]
        key = (n, ("host_io", slot))
        ws = self._ws.get(key)
        if ws is None:
            nbytes = _lib.lib().xmoe_workspace_bytes_host_io(C.byref(self.cfg), n)
            raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=self.weights.w13_packed.device)
            off = (-raw.data_ptr()) % 1024
            ws = self._ws[key] = raw[off:off + nbytes]
        s = stream.cuda_stream if stream is not None else _stream()
        check(_lib.lib().xmoe_forward_host_async(C.byref(self.cfg), C.byref(self._wstruct), x_host.data_ptr(),
                                                 logits_host.data_ptr(), n, y_host.data_ptr(), ws.data_ptr(),
                                                 ws.numel(), s), "xmoe_forward_host_async")

    def status(self, n: int, host_io: bool = False) -> int:
        """Device status word of the last forward with n tokens (0 = ok). Synchronises."""
        ws = self.workspace(n, host_io)
        out = C.c_uint32(0)
        rc = _lib.lib().xmoe_read_status(ws.data_ptr(), C.byref(out), _stream())
        if rc not in (0, 5):
            check(rc, "xmoe_read_status")
        return out.value


def router_topk(logits: torch.Tensor, shape: MoEShape, weights: "PreparedWeights | None" = None,
                idx_stride: int | None = None):
    """Router stage alone: (topk_idx i32 [N, stride], topk_w bf16 [N, stride])."""
    n, e = logits.shape
    stride = idx_stride or shape.top_k
    idx = torch.empty(n, stride, dtype=torch.int32, device=logits.device)
    w = torch.empty(n, stride, dtype=torch.bfloat16, device=logits.device)
    bias = lut = es = None
    if weights is not None:
        bias, lut, es = weights.router_bias, weights.lut, weights.expert_scale
    check(_lib.lib().xmoe_router_topk(logits.data_ptr(), _ptr(bias), _ptr(lut), _ptr(es), n, e, shape.top_k, stride,
                                      _SCORE[shape.scoring], int(shape.renormalize), shape.n_group, shape.topk_group,
                                      shape.routed_scale, idx.data_ptr(), w.data_ptr(), _stream()), "xmoe_router_topk")
    return idx, w


def gate_logits(x: torch.Tensor, gate_weight: torch.Tensor) -> torch.Tensor:
    """Gate GEMM alone: bf16 [N, E] = x [N, H] @ gate_weight [E, H]^T (fp32 accumulation)."""
    n, h = x.shape
    e = gate_weight.shape[0]
    out = torch.empty(n, e, dtype=torch.bfloat16, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    check(_lib.lib().xmoe_gate_logits(x.data_ptr(), gate_weight.data_ptr(), n, h, e, out.data_ptr(), status.data_ptr(),
                                      _stream()), "xmoe_gate_logits")
    if int(status.item()):
        raise RuntimeError(f"gate GEMM device status {int(status.item()):#x}")
    return out


def act_amax(x: torch.Tensor) -> torch.Tensor:
    """Activation scale stage alone: device f32 [4] = XGS, XGSINV, amax, 0."""
    scratch = torch.zeros(2, dtype=torch.int32, device=x.device)
    scale = torch.zeros(4, dtype=torch.float32, device=x.device)
    check(_lib.lib().xmoe_act_amax(x.data_ptr(), x.numel(), scratch.data_ptr(), scale.data_ptr(), _stream()),
          "xmoe_act_amax")
    return scale


def act_scale_from_amax(amax: torch.Tensor) -> torch.Tensor:
    scale = torch.zeros(4, dtype=torch.float32, device=amax.device)
    check(_lib.lib().xmoe_act_scale_from_amax(amax.data_ptr(), scale.data_ptr(), _stream()),
          "xmoe_act_scale_from_amax")
    return scale


def combine(rows: torch.Tensor, topk_row: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Combine stage alone: y[t] = sum_s rows[topk_row[t, s]] (fp32, slot order), bf16."""
    n, k = topk_row.shape
    h = rows.shape[1]
    y = torch.empty(n, h, dtype=torch.bfloat16, device=rows.device) if out is None else out
    if n:
        check(_lib.lib().xmoe_combine(rows.data_ptr(), topk_row.data_ptr(), n, h, k, k, y.data_ptr(), _stream()),
              "xmoe_combine")
    return y


STAGE_NAMES = ("router", "route_pack", "act_amax", "act_quant", "ff1", "act_topk", "ff2", "combine")


def probe_mma_rate(kind: str = "nvfp4", n_mma: int = 65536) -> float:
    """Dense TFLOP/s at which the GPU retires resident-operand tcgen05.mma instructions (M 128, N 256):
    the tensor-pipe ceiling used as a roofline denominator where no library GEMM exists (NVFP4)."""
    out = C.c_double(0.0)
    check(_lib.lib().xmoe_probe_mma_rate({"nvfp4": 0, "bf16": 1}[kind], n_mma, C.byref(out), _stream()),
          "xmoe_probe_mma_rate")
    return out.value


def profile_begin(max_steps: int) -> None:
    check(_lib.lib().xmoe_profile_begin(max_steps), "xmoe_profile_begin")


def profile_read() -> tuple[dict, int]:
    """(stage -> summed ms over the recorded forwards, number of forwards). Synchronises."""
    buf = (C.c_float * 8)()
    steps = C.c_int32(0)
    check(_lib.lib().xmoe_profile_read(buf, C.byref(steps)), "xmoe_profile_read")
    return dict(zip(STAGE_NAMES, list(buf))), steps.value


def forward(x, router_logits, per_expert_scale, layer: FusedMoE):
    """Functional spelling close to the reference's `_C.forward(x, router_logits, per_expert_scale, ...)`."""
    if per_expert_scale is not None and layer.weights.expert_scale is None:
        raise RuntimeError("per_expert_scale must be bound when the weights are prepared")
    return layer.forward(x, router_logits.to(torch.bfloat16))
