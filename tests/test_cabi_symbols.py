"""The shared library loads on a machine without a GPU and exports every function the header declares."""
import ctypes
import os
import re

import pytest

from tests.conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "aeon_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aeonb_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported_and_bound():
    from aeon_b200 import _lib
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 39
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "not exported: " + n
        assert n in _lib.PROTOTYPES, "no ctypes prototype: " + n
    assert sorted(_lib.PROTOTYPES) == names
    assert lib.aeonb_version().startswith(b"aeon_b200")


def test_struct_sizes_match_the_header_layout():
    from aeon_b200 import _lib
    # natural alignment on x86-64: computed by hand from the header
    assert ctypes.sizeof(_lib.ImageDesc) == 152
    assert ctypes.sizeof(_lib.ImageLayout) == 128
    assert ctypes.sizeof(_lib.JpegDesc) == 128
    assert ctypes.sizeof(_lib.SpecgramDesc) == 24
    assert ctypes.sizeof(_lib.SpecgramConfig) == 32


def test_calls_without_a_gpu_fail_with_a_message_not_a_crash():
    import torch
    from aeon_b200 import _lib
    lib = _lib.load()
    if torch.cuda.is_available():
        return
    h = ctypes.c_void_p()
    assert lib.aeonb_ctx_create(0, None, ctypes.byref(h)) < 0
    assert lib.aeonb_last_error()


@pytest.mark.timeout(120)
@pytest.mark.parametrize("threads", [1, 2, 3, 5, 14])
def test_worker_pool_light_and_full_dispatches_complete(threads):
    """The pool that stages the batches: thousands of alternating light (three threads) and full dispatches must all
    complete and run every job exactly once."""
    from aeon_b200 import _lib
    rounds = 20000
    want = sum((n * (n - 1)) // 2 for n in (1 + it % 300 for it in range(rounds)))
    assert _lib.load().aeonb_selftest_worker_pool(threads, rounds) == want
