"""The allocation-free image entry point must give exactly what the regular one gives.

Some callers of this library cannot allocate GPU or pinned memory while they run: code inside a
framework phase that forbids allocator calls, processes with a memory budget fixed at start-up,
and latency-critical loops.  aeonb_image_batch_noalloc keeps its descriptor copy in a fixed array
inside the library instead.  Two calls in a row are checked (the array keeps the previous call's
contents), against the regular entry point, bit for bit.  This file is collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import image_ops as ops
from tests.synth import gradient_image

pytestmark = pytest.mark.gpu


def _params(rng, w, h, photometric):
    cw, ch = int(rng.integers(8, w + 1)), int(rng.integers(8, h + 1))
    kw = dict(cropbox=(int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch),
              output_size=(96, 80), flip=bool(rng.integers(2)))
    if photometric:
        kw.update(contrast=0.8, brightness=1.2, saturation=0.7, hue=int(rng.integers(-18, 19)),
                  lighting=[0.1, -0.05, 0.02], color_noise_std=0.1)
    return ops.ImageParams(**kw)


def test_noalloc_entry_matches_regular_entry_twice(ctx):
    from aeon_b200 import _lib as L, kernels as K
    lib = ctx.lib
    rng = np.random.default_rng(77)
    dev = torch.device("cuda", ctx.device)
    torch.cuda.set_device(ctx.device)
    lay = K.make_layout(96, 80, L.F32, True, True, [0.4, 0.5, 0.6], [0.2, 0.3, 0.25])
    stream = ctx.torch_stream
    for call, (n, photometric) in enumerate([(12, True), (5, False)]):  # the second call is smaller: stale
        srcs = [gradient_image(rng, int(rng.integers(64, 200)), int(rng.integers(64, 200))) for _ in range(n)]
        params = [_params(rng, s.shape[1], s.shape[0], photometric) for s in srcs]
        with torch.cuda.stream(stream):                                  # descriptors of call 1 must not leak in
            tsrc = [torch.from_numpy(s).to(dev) for s in srcs]
            want = torch.zeros((n, 3, 80, 96), dtype=torch.float32, device=dev)
            got = torch.full((n, 3, 80, 96), -1.0, dtype=torch.float32, device=dev)
            K.image_batch(ctx, tsrc, params, want, lay)
            descs = (L.ImageDesc * n)()
            for i in range(n):
                K.fill_desc(descs[i], tsrc[i], params[i], got.data_ptr() + i * got.stride(0) * 4, lib)
            L.check(lib.aeonb_image_batch_noalloc(descs, n, C.byref(lay), C.c_void_p(stream.cuda_stream)))
            stream.synchronize()
        assert torch.equal(got, want), "call %d differs" % call
        for i in range(n):  # and both agree with the oracle
            ref = ops.load_image(ops.transform_single_image(srcs[i], params[i]), True, True, "float",
                                 [0.4, 0.5, 0.6], [0.2, 0.3, 0.25])
            assert np.abs(got[i].cpu().numpy() - ref).max() <= 1e-6


def test_noalloc_entry_rejects_oversized_batches(ctx):
    from aeon_b200 import _lib as L, kernels as K
    n = 513
    descs = (L.ImageDesc * n)()
    lay = K.make_layout(8, 8, L.U8)
    status = ctx.lib.aeonb_image_batch_noalloc(descs, n, C.byref(lay), None)
    assert status == L.ERR_INVALID
    assert b"at most 512" in ctx.lib.aeonb_last_error()


def test_noalloc_entry_with_pinned_descriptors(ctx):
    """Descriptors in pinned host memory: the copy is then truly asynchronous, and the array must stay unchanged until the
    stream has consumed it -- which the test honours by synchronising before it touches the array again."""
    from aeon_b200 import _lib as L, kernels as K
    lib = ctx.lib
    rng = np.random.default_rng(78)
    dev = torch.device("cuda", ctx.device)
    torch.cuda.set_device(ctx.device)
    lay = K.make_layout(96, 80, L.U8, False)
    stream = ctx.torch_stream
    n = 7
    srcs = [gradient_image(rng, int(rng.integers(64, 200)), int(rng.integers(64, 200))) for _ in range(n)]
    params = [_params(rng, s.shape[1], s.shape[0], True) for s in srcs]
    pinned = torch.zeros(n * C.sizeof(L.ImageDesc), dtype=torch.uint8).pin_memory()
    descs = (L.ImageDesc * n).from_address(pinned.data_ptr())
    with torch.cuda.stream(stream):
        tsrc = [torch.from_numpy(s).to(dev) for s in srcs]
        want = torch.zeros((n, 80, 96, 3), dtype=torch.uint8, device=dev)
        got = torch.full((n, 80, 96, 3), 9, dtype=torch.uint8, device=dev)
        K.image_batch(ctx, tsrc, params, want, lay)
        for i in range(n):
            K.fill_desc(descs[i], tsrc[i], params[i], got.data_ptr() + i * got.stride(0), lib)
        L.check(lib.aeonb_image_batch_noalloc(descs, n, C.byref(lay), C.c_void_p(stream.cuda_stream)))
        stream.synchronize()
    assert torch.equal(got, want)
    for i in range(n):
        assert np.array_equal(got[i].cpu().numpy(), ops.transform_single_image(srcs[i], params[i]))
