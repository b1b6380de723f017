"""ctypes binding of libxmoe_b200.so (the C ABI declared in include/xmoe_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# XMOE_B200_LIB selects another build of the library (e.g. one compiled with debug defines).
_LIB_PATH = Path(os.environ.get("XMOE_B200_LIB") or Path(__file__).resolve().parent / "libxmoe_b200.so")
_lib = None

STATUS_NAMES = {0: "OK", 1: "ERR_ARG", 2: "ERR_SHAPE", 3: "ERR_WORKSPACE", 4: "ERR_CUDA", 5: "ERR_TIMEOUT",
                6: "ERR_LIMIT"}


class XMoEConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("inter", C.c_int32), ("num_experts", C.c_int32), ("top_k", C.c_int32),
        ("num_shared_experts", C.c_int32), ("scoring", C.c_int32), ("renormalize", C.c_int32),
        ("n_group", C.c_int32), ("topk_group", C.c_int32), ("activation", C.c_int32),
        ("act_topk_keep", C.c_int32), ("token_tile", C.c_int32),
        ("routed_scale", C.c_float), ("swiglu_alpha", C.c_float), ("swiglu_limit", C.c_float),
    ]


class XMoEWeights(C.Structure):
    _fields_ = [
        ("w13_packed", C.c_void_p), ("w13_sf", C.c_void_p), ("w13_gs", C.c_void_p), ("w2_q", C.c_void_p),
        ("w2_scale", C.c_void_p), ("router_bias", C.c_void_p), ("expert_scale", C.c_void_p),
        ("sigmoid_lut", C.c_void_p),
    ]


class XMoEWorkspaceView(C.Structure):
    _fields_ = [
        ("status", C.c_void_p), ("act_scale", C.c_void_p), ("topk_idx", C.c_void_p), ("topk_w", C.c_void_p),
        ("topk_off", C.c_void_p), ("topk_row", C.c_void_p), ("counts", C.c_void_p), ("offsets", C.c_void_p),
        ("row_token", C.c_void_p), ("row_weight", C.c_void_p), ("xq", C.c_void_p), ("sfx", C.c_void_p),
        ("yact", C.c_void_p), ("out_rows", C.c_void_p),
        ("k_eff", C.c_int32), ("packed_rows", C.c_int32), ("kb_pad", C.c_int32), ("token_tile", C.c_int32),
    ]


EP_MAX_WORLD = 8
EP_CTL_BYTES = 512


class XMoEEpBuffers(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("hidden", C.c_int32), ("experts_per_rank", C.c_int32),
        ("cap_rows", C.c_int32), ("ret_cap", C.c_int32),
        ("ctl", C.c_void_p * EP_MAX_WORLD), ("recv_x", C.c_void_p * EP_MAX_WORLD),
        ("recv_meta", C.c_void_p * EP_MAX_WORLD), ("ret_rows", C.c_void_p * EP_MAX_WORLD),
    ]


# name -> (restype, argtypes); every symbol of include/xmoe_b200.h
_P, _I, _F, _SZ = C.c_void_p, C.c_int32, C.c_float, C.c_size_t
SIGNATURES = {
    "xmoe_build_info": (C.c_char_p, []),
    "xmoe_status_string": (C.c_char_p, [C.c_int]),
    "xmoe_packed_rows": (_SZ, [C.POINTER(XMoEConfig), _I]),
    "xmoe_workspace_bytes": (_SZ, [C.POINTER(XMoEConfig), _I]),
    "xmoe_workspace_bytes_host_io": (_SZ, [C.POINTER(XMoEConfig), _I]),
    "xmoe_forward": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _I, _P, _P, _SZ, _P]),
    "xmoe_forward_host": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _I, _P, _P, _SZ, _P]),
    "xmoe_forward_host_async": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _I, _P, _P, _SZ, _P]),
    "xmoe_read_status": (C.c_int, [_P, C.POINTER(C.c_uint32), _P]),
    "xmoe_forward_routed": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _P, _P, _I, _P, _P, _SZ,
                                      _P]),
    "xmoe_forward_routed_bounded": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _P, _P, _I, _P, _P,
                                              _P, _SZ, _P]),
    "xmoe_forward_scatter": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _P, _P, _P, _I, _P, _P,
                                       _SZ, _P]),
    "xmoe_gate_logits": (C.c_int, [_P, _P, _I, _I, _I, _P, _P, _P]),
    "xmoe_forward_gated": (C.c_int, [C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P, _P, _I, _P, _P, _SZ, _P]),
    "xmoe_probe_mma_rate": (C.c_int, [_I, _I, C.POINTER(C.c_double), _P]),
    "xmoe_profile_begin": (C.c_int, [_I]),
    "xmoe_profile_read": (C.c_int, [C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "xmoe_workspace_view_get": (C.c_int, [C.POINTER(XMoEConfig), _I, _P, _SZ, C.POINTER(XMoEWorkspaceView)]),
    "xmoe_router_topk": (C.c_int, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P]),
    "xmoe_route_pack_scratch_bytes": (_SZ, [_I, _I, _I]),
    "xmoe_route_pack": (C.c_int, [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "xmoe_route_pack_static_max_tokens": (_I, []),
    "xmoe_route_pack_static": (C.c_int, [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "xmoe_act_amax": (C.c_int, [_P, _SZ, _P, _P, _P]),
    "xmoe_act_scale_from_amax": (C.c_int, [_P, _P, _P]),
    "xmoe_act_quant_pack": (C.c_int, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "xmoe_ff1": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P]),
    "xmoe_act_topk": (C.c_int, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "xmoe_ff2": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "xmoe_combine": (C.c_int, [_P, _P, _I, _I, _I, _I, _P, _P]),
    "xmoe_ep_post_counts": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, _P, _P]),
    "xmoe_ep_dispatch": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "xmoe_ep_wait_data": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, _P, _P, _P]),
    "xmoe_ep_return": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, _P, _I, _P]),
    "xmoe_ep_forward_local": (C.c_int, [C.POINTER(XMoEEpBuffers), C.POINTER(XMoEConfig), C.POINTER(XMoEWeights), _P, _P,
                                        _P, _P, _I, _P, _P, _SZ, _P]),
    "xmoe_ep_dispatch_quantised": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "xmoe_ep_wait_ret": (C.c_int, [C.POINTER(XMoEEpBuffers), _P]),
    "xmoe_ep_status": (C.c_int, [C.POINTER(XMoEEpBuffers), _P, C.POINTER(C.c_uint32)]),
    "xmoe_nvfp4_sf_bytes": (_SZ, [_I, _I, _I]),
    "xmoe_prep_nvfp4_sf": (C.c_int, [_P, _P, _I, _I, _I, _P]),
    "xmoe_repack_gptq": (C.c_int, [_P, _P, _I, _I, _I, _P]),
    "xmoe_repack_int4_kmajor": (C.c_int, [_P, _P, _SZ, _P]),
    "xmoe_fill_sigmoid_lut": (None, [_P]),
}


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """Load the shared library once. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m xcaliber_b200.csrc.build` "
                "(there is no fallback path)")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class XMoEError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        msg = lib().xmoe_status_string(status).decode()
        super().__init__(f"{what}: {STATUS_NAMES.get(status, status)} ({msg})")


def check(status: int, what: str) -> None:
    if status != 0:
        raise XMoEError(status, what)
