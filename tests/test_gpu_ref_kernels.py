"""Pins the CPU oracle and the CUDA path against the REFERENCE's own kernels (topk.cuh and
preamble.cuh, compiled unmodified for sm_100a into oracle/_ref/libref_kernels.so by
oracle/build_oracle.py): router, route pack, activation scale and NVFP4 activation packets."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from xcaliber_b200 import ops, synth

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_kernels.so"


@pytest.fixture(scope="module")
def ref():
    if not REF.exists():
        pytest.skip("oracle/_ref/libref_kernels.so not built (reference tree absent at build time)")
    return C.CDLL(str(REF))


def _p(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("n,e,k,sigmoid", [(64, 8, 2, 0), (300, 128, 8, 0), (77, 128, 4, 1), (1, 64, 6, 0)])
def test_router_and_route_pack_match_reference_kernels(ref, n, e, k, sigmoid):
    torch.manual_seed(n + e)
    # coarse grid => exact bf16 ties are common
    logits = (torch.randint(-24, 24, (n, e)).float() / 8).to(torch.bfloat16).cuda()
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    idx_r = torch.zeros(n, k, dtype=torch.int32, device="cuda")
    w_r = torch.zeros(n, k, dtype=torch.int16, device="cuda")
    assert ref.ref_topk(_p(logits), _p(idx_r), _p(w_r), None, n, e, k, C.c_float(1.0), sigmoid, s) == 0
    np_ = (n + 31) & ~31
    off_r = torch.zeros(n, k, dtype=torch.int16, device="cuda")
    etw_r = torch.zeros(e, np_, dtype=torch.int16, device="cuda")
    eti_r = torch.zeros(e, np_ + 1, dtype=torch.int16, device="cuda")
    assert ref.ref_route_pack(_p(idx_r), _p(w_r), _p(off_r), _p(etw_r), _p(eti_r), n, np_, k, e, s) == 0
    torch.cuda.synchronize()
    # oracle
    idx_o, wb_o, w_o = O.router_topk(logits.cpu(), k, "sigmoid" if sigmoid else "softmax")
    np.testing.assert_array_equal(idx_r.cpu().numpy(), idx_o)
    wr = O.bits_to_f32(w_r.cpu().numpy().view(np.uint16))
    assert np.abs(wr - w_o).max() <= 2.0 ** -8
    pk = O.route_pack(idx_o, w_r.cpu().numpy().view(np.uint16), e)
    off, etw, eti = O.to_reference_route_arrays(pk["idx"], pk["w_bits"], pk["topk_off"], e)
    np.testing.assert_array_equal(off_r.cpu().numpy().view(np.uint16), off)
    np.testing.assert_array_equal(etw_r.cpu().numpy().view(np.uint16), etw)
    np.testing.assert_array_equal(eti_r.cpu().numpy().view(np.uint16), eti)
    # this library's router kernel: same indices, weights within the reference's own tolerance
    shape = synth.MoEShape("t", 64, 64, e, k, scoring="sigmoid" if sigmoid else "softmax")
    idx_m, w_m = ops.router_topk(logits, shape)
    np.testing.assert_array_equal(idx_m.cpu().numpy(), idx_o)
    wm = w_m.float().cpu().numpy()
    assert np.abs(wm - wr).max() <= 2.0 ** -8


@pytest.mark.parametrize("n,e,k,h", [(64, 8, 2, 1024), (100, 32, 4, 256), (33, 16, 8, 2880)])
def test_activation_quant_matches_reference_kernels(ref, n, e, k, h):
    torch.manual_seed(h + n)
    x = torch.randn(n, h)
    x[1, 32:48] = 0
    x[2] *= 1e-3
    x = x.to(torch.bfloat16).cuda()
    logits = torch.randn(n, e).to(torch.bfloat16).cuda()
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    idx_r = torch.zeros(n, k, dtype=torch.int32, device="cuda")
    w_r = torch.zeros(n, k, dtype=torch.int16, device="cuda")
    ref.ref_topk(_p(logits), _p(idx_r), _p(w_r), None, n, e, k, C.c_float(1.0), 0, s)
    np_ = (n + 31) & ~31
    off_r = torch.zeros(n, k, dtype=torch.int16, device="cuda")
    etw_r = torch.zeros(e, np_, dtype=torch.int16, device="cuda")
    eti_r = torch.zeros(e, np_ + 1, dtype=torch.int16, device="cuda")
    ref.ref_route_pack(_p(idx_r), _p(w_r), _p(off_r), _p(etw_r), _p(eti_r), n, np_, k, e, s)
    pairs = n * h // 2
    blocks = max(1, min(4096, (pairs + 2047) // 2048))
    partial = torch.zeros(4096, dtype=torch.int32, device="cuda")
    scale = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert ref.ref_act_scale(_p(x), C.c_ulonglong(pairs), _p(partial), blocks, _p(scale), s) == 0
    x4 = torch.zeros(e, np_, h // 8, dtype=torch.int32, device="cuda")
    sx = torch.zeros(e, np_, h // 64, dtype=torch.int32, device="cuda")
    assert ref.ref_act_pack(_p(x), _p(scale), _p(idx_r), _p(off_r), _p(x4), _p(sx), n, np_, h, k, s) == 0
    torch.cuda.synchronize()
    # activation scale, bit for bit
    sc = scale.cpu().numpy()
    xgs_ref = sc[:1].view(np.float32)[0]
    inv_ref = O.bits_to_f32(np.array([sc[1] & 0xFFFF], dtype=np.uint16))[0]
    xgs, inv = O.act_scale(x.cpu())
    assert xgs_ref == xgs and inv_ref == inv
    mine = ops.act_amax(x).cpu().numpy()
    assert mine[0] == xgs and mine[1] == inv
    # packets: undo the reference's fragment order (preamble.cuh:612-627) and compare with the oracle
    codes, sbytes = O.act_quant(x.cpu(), xgs)
    packed = O.pack_nibbles(codes).view(np.uint32).reshape(n, h // 64, 8)        # one u32 per 8 K
    sq = sbytes.reshape(n, h // 64, 4).copy().view(np.uint32).reshape(n, h // 64)
    x4n = x4.cpu().numpy().view(np.uint32).reshape(e, -1)
    sxn = sx.cpu().numpy().view(np.uint32).reshape(e, -1)
    idx = idx_r.cpu().numpy()
    off = off_r.cpu().numpy().view(np.uint16)
    for t in range(n):
        for slot in range(k):
            ex, p = int(idx[t, slot]), int(off[t, slot])
            for kt in range(h // 64):
                for q8 in range(8):
                    word = (p >> 4) * (h << 1) + (kt << 7) + (p & 7) * 16 + (q8 & 3) * 4 + ((p >> 3) & 1) * 2 + (q8 >> 2)
                    assert x4n[ex, word] == packed[t, kt, q8], (t, slot, kt, q8)
                sword = (p >> 5) * ((h >> 6) << 5) + kt * 32 + (p & 7) * 4 + ((p >> 3) & 3)
                assert sxn[ex, sword] == sq[t, kt], (t, slot, kt)
