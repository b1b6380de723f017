"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol the
header declares, sizes its workspace sensibly and rejects bad arguments before touching CUDA."""
import ctypes as C
import re
from pathlib import Path

import pytest

from xcaliber_b200 import _lib, ops, synth

ROOT = Path(__file__).resolve().parent.parent


def test_every_declared_symbol_is_exported(built_lib):
    header = (ROOT / "include" / "xmoe_b200.h").read_text()
    declared = set(re.findall(r"\b(xmoe_[a-z0-9_]+)\s*\(", header))
    declared -= {"xmoe_config", "xmoe_weights", "xmoe_workspace_view"}
    assert len(declared) >= 25
    for name in sorted(declared):
        assert hasattr(built_lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= declared


def test_struct_layouts_match_header(built_lib):
    assert C.sizeof(_lib.XMoEConfig) == 15 * 4
    assert C.sizeof(_lib.XMoEWeights) == 8 * 8
    assert C.sizeof(_lib.XMoEWorkspaceView) == 14 * 8 + 4 * 4
    assert b"sm_100a" in built_lib.xmoe_build_info()


def test_workspace_sizes(built_lib):
    cfg = ops.make_config(synth.SHAPES["mixtral"])
    rows = built_lib.xmoe_packed_rows(C.byref(cfg), 4096)
    assert rows == (4096 * 2 + 8 * 127 + 127) // 128 * 128
    small = built_lib.xmoe_workspace_bytes(C.byref(cfg), 16)
    big = built_lib.xmoe_workspace_bytes(C.byref(cfg), 4096)
    assert 0 < small < big
    assert big >= rows * (14336 * 2 + 4096 * 2 + 2048)
    assert built_lib.xmoe_workspace_bytes_host_io(C.byref(cfg), 4096) > big
    # decode batches only reserve rows for experts that can be live
    assert built_lib.xmoe_packed_rows(C.byref(ops.make_config(synth.SHAPES["qwen3"])), 1) == 1024


@pytest.mark.parametrize("field,value", [("hidden", 1000), ("inter", 100), ("num_experts", 2048), ("top_k", 9),
                                         ("top_k", 0), ("num_shared_experts", 9), ("scoring", 3), ("activation", 5),
                                         ("token_tile", 48), ("n_group", 33)])
def test_bad_configs_are_rejected(built_lib, field, value):
    cfg = ops.make_config(synth.SHAPES["toy"])
    setattr(cfg, field, value)
    assert built_lib.xmoe_workspace_bytes(C.byref(cfg), 8) == 0
    w = _lib.XMoEWeights()
    rc = built_lib.xmoe_forward(C.byref(cfg), C.byref(w), None, None, 8, None, None, 0, None)
    assert rc in (1, 2)


def test_null_pointers_and_empty_batch(built_lib):
    cfg = ops.make_config(synth.SHAPES["toy"])
    w = _lib.XMoEWeights()
    assert built_lib.xmoe_forward(C.byref(cfg), C.byref(w), None, None, 0, None, None, 0, None) == 0   # N == 0: no-op
    assert built_lib.xmoe_forward(C.byref(cfg), C.byref(w), None, None, 8, None, None, 0, None) == 1   # ERR_ARG
    assert built_lib.xmoe_forward(C.byref(cfg), C.byref(w), None, None, -1, None, None, 0, None) == 1
    assert built_lib.xmoe_router_topk(None, None, None, None, 4, 8, 2, 2, 0, 1, 1, 1, 1.0, None, None, None) == 1
    assert built_lib.xmoe_status_string(3).startswith(b"workspace")
    with pytest.raises(_lib.XMoEError):
        _lib.check(2, "probe")


def test_sigmoid_lut_matches_oracle(built_lib):
    import numpy as np
    import torch

    from oracle import moe_oracle as O

    host = torch.empty(65536, dtype=torch.float32)
    built_lib.xmoe_fill_sigmoid_lut(host.data_ptr())
    ref = O.sigmoid_lut()
    got = host.numpy()
    finite = np.isfinite(ref)
    assert (got[finite] == ref[finite]).mean() > 0.9999
    assert np.abs(got[finite] - ref[finite]).max() <= 2 ** -24


def _kwalk_lib(tmp_path_factory):
    import subprocess

    out = tmp_path_factory.mktemp("kwalk") / "libkwalk_host.so"
    src = Path(__file__).resolve().parent / "kwalk_host.cpp"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", str(src), "-o", str(out)], check=True)
    lib = C.CDLL(str(out))
    lib.kwalk_segments.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_int), C.c_int]
    lib.kwalk_segments.restype = C.c_int
    return lib


def test_k_walk_covers_every_unit_once(tmp_path_factory):
    """The scheduler the FF2 kernel runs on the device (tiles cut along K, and whole tiles with a balanced stride),
    compiled for the host: over many tile lists and grids every K unit of every tile belongs to exactly one segment,
    a CTA's ring numbering (it0) counts the units it walked before, a non-final segment comes first, and the CTAs a
    finishing segment names as helpers hold exactly the units before its own."""
    lib = _kwalk_lib(tmp_path_factory)
    buf = (C.c_int * (6 * 4096))()

    def segments(tiles, k_walk, grid, cta, split):
        n = lib.kwalk_segments(tiles, k_walk, grid, cta, split, buf, 4096)
        assert 0 <= n <= 4096
        return [tuple(buf[6 * i + j] for j in range(6)) for i in range(n)]

    cases = [(t, k, g) for t in (1, 2, 3, 7, 64, 148, 149, 256, 300) for k in (2, 4, 6, 16, 24, 112) for g in (1, 4, 132, 148)]
    for tiles, k_walk, grid in cases:
        for split in (0, 1):
            owner = {}
            per_cta = {}
            for cta in range(grid):
                segs = per_cta[cta] = segments(tiles, k_walk, grid, cta, split)
                walked = 0
                for i, (tile, ks0, ks1, it0, first_helper, finishes) in enumerate(segs):
                    assert 0 <= tile < tiles and 0 <= ks0 < ks1 <= k_walk
                    assert it0 == walked, (tiles, k_walk, grid, cta, split, segs)
                    walked += ks1 - ks0
                    assert finishes == (ks1 == k_walk)
                    assert finishes or i == 0, "a partial sum must not wait behind other work"
                    if split:
                        assert ks0 % 2 == 0, "a segment never starts inside a two-unit weight stage"
                    for u in range(ks0, ks1):
                        assert (tile, u) not in owner, "K unit covered twice"
                        owner[(tile, u)] = cta
            assert len(owner) == tiles * k_walk, "K unit not covered"
            for cta, segs in per_cta.items():
                for tile, ks0, ks1, it0, first_helper, finishes in segs:
                    if not split or not finishes:
                        continue
                    helpers = sorted({owner[(tile, u)] for u in range(ks0)})
                    assert helpers == list(range(first_helper, cta)), (tiles, k_walk, grid, cta, segs)
                    for h in helpers:  # each helper holds ONE non-final segment of this tile
                        hs = [s for s in per_cta[h] if s[0] == tile]
                        assert len(hs) == 1 and hs[0][5] == 0


@pytest.mark.parametrize("shape,n,tile", [
    ("mixtral", 16, 32), ("mixtral", 64, 32), ("mixtral", 128, 128), ("mixtral", 4096, 128),
    ("qwen3", 256, 32), ("qwen3", 512, 128), ("gptoss", 512, 32), ("gptoss", 1024, 128),
    # shared experts take every token, but the routed experts decide: 16 rows per routed expert at 512 tokens
    ("dsv3", 16, 32), ("dsv3", 512, 32), ("dsv3", 1024, 128),
])
def test_token_tile_rule(built_lib, shape, n, tile):
    """The token tile a call pads every expert's rows to: 128 from 24 rows per routed expert on average, else 32
    (the workspace view reports the library's choice; nothing here touches the GPU)."""
    cfg = ops.make_config(synth.SHAPES[shape])
    nbytes = built_lib.xmoe_workspace_bytes(C.byref(cfg), n)
    view = _lib.XMoEWorkspaceView()
    fake = 1 << 20  # only addresses are computed
    assert built_lib.xmoe_workspace_view_get(C.byref(cfg), n, C.c_void_p(fake), nbytes, C.byref(view)) == 0
    assert view.token_tile == tile
    assert view.packed_rows % 128 == 0 and view.k_eff == cfg.top_k + cfg.num_shared_experts
