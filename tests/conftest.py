"""pytest configuration: the `gpu` marker and shared helpers.

CPU tests (`-m "not gpu"`) cover the oracle against the golden vectors, the host logic and
that the C-ABI library loads and exports every declared symbol. GPU tests (`-m gpu`) are the
parity tests proper: they call the CUDA path through the C ABI and compare with the oracle.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The oracle allocates and frees many large numpy temporaries. Keep freed blocks inside the heap instead of
# returning them to the kernel (no mmap for large blocks, no trimming): on hosts where first touch of a page
# is slow the CPU suite otherwise spends most of its time in page faults.
try:
    import ctypes

    _libc = ctypes.CDLL("libc.so.6")
    _libc.mallopt(-4, 0)          # M_MMAP_MAX = 0
    _libc.mallopt(-1, 1 << 40)    # M_TRIM_THRESHOLD
except OSError:
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    from xcaliber_b200 import _lib

    if not _lib.lib_path().exists():
        from xcaliber_b200.csrc import build

        build.build()
    return _lib.lib()
