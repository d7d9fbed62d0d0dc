"""aeon's C++ loader API (include/aeon_b200.hpp, header-only over the C ABI): the loop of aeon's
examples/cpp_iterator/iterator.cpp, compiled here with g++ against the header and the shared library.

Without a GPU the program must build, link and fail with aeon-style exceptions; with one it must deliver the
batches the Python DataLoader delivers for the same configuration."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from tests.conftest import ROOT

SRC = os.path.join(ROOT, "tests", "cpp", "iterator_example.cpp")


def build(tmp_path):
    exe = str(tmp_path / "iterator_example")
    libdir = os.path.join(ROOT, "aeon_b200")
    from aeon_b200 import _lib
    _lib.load()   # the library must be built
    subprocess.run(["g++", "-std=c++11", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC, "-o", exe,
                    "-L" + libdir, "-laeon_b200", "-Wl,-rpath," + libdir], check=True)
    return exe


def data_dir(tmp_path, golden_dir):
    d = tmp_path / "data"
    d.mkdir()
    for f in ("flowers.jpg", "img_2112_70.jpg"):
        shutil.copy(os.path.join(golden_dir, f), d / f)
    return str(d)


def test_cpp_header_builds_and_reports_errors_as_exceptions(tmp_path, golden_dir):
    import torch
    exe = build(tmp_path)
    r = subprocess.run([exe, data_dir(tmp_path, golden_dir), "20"], capture_output=True, text=True)
    if not torch.cuda.is_available():
        assert r.returncode == 1 and "failed: " in r.stdout   # no device: std::runtime_error, not a crash
    else:
        assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_iterator_matches_python_dataloader(tmp_path, golden_dir):
    exe = build(tmp_path)
    d = data_dir(tmp_path, golden_dir)
    r = subprocess.run([exe, d, "20"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    out = r.stdout
    assert "batch size: 4" in out and "batch count: 5" in out and "record count: 20" in out
    assert "buffer image uint8_t [ 32 32 3 ] bytes 3072" in out and "buffer label int32_t [ 1 ] bytes 4" in out
    assert "batches: 5 position 5" in out and "again: 5" in out
    assert "error: Required Argument: " in out   # a missing required key throws, with aeon's message
    rows = [ln.split() for ln in out.splitlines() if ln.startswith("\tbatch")]
    assert len(rows) == 5
    from aeon_b200.dataloader import DataLoader
    cfg = {"manifest_root": d, "manifest_filename": os.path.join(d, "manifest_cpp_iterator.txt"), "batch_size": 4,
           "iteration_mode": "ONCE", "etl": [{"type": "image", "height": 32, "width": 32, "channel_major": False},
                                               {"type": "label", "binary": False}],
           "augmentation": [{"type": "image", "flip_enable": True}]}
    dl = DataLoader(cfg)
    for i, batch in enumerate(dl):
        b = dict(batch)
        words = rows[i]
        assert int(words[words.index("label") + 1]) == int(b["label"][0, 0])
        # the flip is drawn from an unseeded engine; it permutes the pixels of a row and keeps their sum
        assert int(words[words.index("sum") + 1]) == int(b["image"][0].astype(np.int64).sum())
        assert int(words[words.index("items") + 1]) == 4 and "elements: 2]" in " ".join(words)
    dl.close()
