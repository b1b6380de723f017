"""xmoe_route_pack_static: the route pack for callers that cannot allocate device memory.

Some users of this library reach the routing step at a point where they have no way to get
scratch memory: an inference server that gave every free byte of HBM to its cache pool, or a
call site that must not risk the device-wide synchronisation a cudaMalloc can cause. The static
entry point keeps its histograms in a fixed array inside the library instead. This test calls it
through the C ABI, twice in a row with different inputs (the array keeps the first call's
contents, so the second call checks that stale data does no harm), and requires bit-identical
outputs to the ordinary xmoe_route_pack. It also checks the size limit. The file sorts last on
purpose: it runs after every other test and must also pass alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

from xcaliber_b200 import _lib

pytestmark = pytest.mark.gpu


def _route(n, e, k, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(n)]).to(torch.int32).cuda()
    w = torch.rand(n, k, generator=g).to(torch.bfloat16).cuda()
    return idx, w


def _outputs(n, e_tot, k_eff):
    rows = n * k_eff + min(e_tot, n * k_eff) * 127 + 128
    return dict(
        counts=torch.full((e_tot,), -7, dtype=torch.int32, device="cuda"),
        offsets=torch.full((e_tot + 1,), -7, dtype=torch.int32, device="cuda"),
        topk_off=torch.full((n, k_eff), -7, dtype=torch.int32, device="cuda"),
        topk_row=torch.full((n, k_eff), -7, dtype=torch.int32, device="cuda"),
        row_token=torch.full((rows,), -7, dtype=torch.int32, device="cuda"),
        row_weight=torch.zeros(rows, dtype=torch.bfloat16, device="cuda"),
        status=torch.zeros(4, dtype=torch.int32, device="cuda"),
    )


def _run(static, idx, w, e, k, n_shared):
    lib = _lib.lib()
    n = idx.shape[0]
    k_eff = k + n_shared
    idx_w = torch.zeros(n, k_eff, dtype=torch.int32, device="cuda")
    w_w = torch.zeros(n, k_eff, dtype=torch.bfloat16, device="cuda")
    idx_w[:, :k], w_w[:, :k] = idx, w
    o = _outputs(n, e + n_shared, k_eff)
    stream = torch.cuda.current_stream().cuda_stream
    tail = [o["counts"].data_ptr(), o["offsets"].data_ptr(), o["topk_off"].data_ptr(), o["topk_row"].data_ptr(),
            o["row_token"].data_ptr(), o["row_weight"].data_ptr(), o["status"].data_ptr(), stream]
    if static:
        rc = lib.xmoe_route_pack_static(idx_w.data_ptr(), w_w.data_ptr(), n, e, k, k_eff, n_shared, *tail)
    else:
        scratch = torch.empty(lib.xmoe_route_pack_scratch_bytes(n, e, n_shared), dtype=torch.uint8, device="cuda")
        rc = lib.xmoe_route_pack(idx_w.data_ptr(), w_w.data_ptr(), n, e, k, k_eff, n_shared, scratch.data_ptr(), *tail)
    torch.cuda.synchronize()
    assert rc == 0
    o["idx"], o["w"] = idx_w, w_w
    return o


def test_static_route_pack_matches_on_two_calls_in_a_row():
    # first call: many chunks, many experts; second: fewer of both, so stale histogram entries
    # of the first call lie beyond what the second call uses
    for n, e, k, n_shared, seed in [(3000, 128, 8, 0, 1), (700, 16, 2, 1, 2)]:
        idx, w = _route(n, e, k, seed)
        ref = _run(False, idx, w, e, k, n_shared)
        got = _run(True, idx, w, e, k, n_shared)
        assert int(got["status"][0]) == 0
        rows = int(ref["offsets"][-1])
        live = torch.zeros(ref["row_token"].numel(), dtype=torch.bool, device="cuda")
        live[ref["topk_row"].reshape(-1).long()] = True
        for name in ("counts", "offsets", "topk_off", "topk_row", "idx", "w"):
            assert torch.equal(got[name], ref[name]), name
        assert torch.equal(got["row_token"][live], ref["row_token"][live])
        assert torch.equal(got["row_weight"][live], ref["row_weight"][live])
        assert rows == int(got["offsets"][-1])


def test_static_route_pack_rejects_sizes_beyond_its_array():
    lib = _lib.lib()
    limit = lib.xmoe_route_pack_static_max_tokens()
    assert limit == 16384
    n = limit + 1
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    rc = lib.xmoe_route_pack_static(p, p, n, 8, 2, 2, 0, p, p, p, p, p, p, p, torch.cuda.current_stream().cuda_stream)
    assert rc == 6  # XMOE_ERR_LIMIT, nothing launched
    torch.cuda.synchronize()
    assert b"fixed scratch array" in lib.xmoe_status_string(rc)
