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
