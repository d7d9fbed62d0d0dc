"""Parity of host entropy decode + GPU JPEG back end with cv2.imdecode and the numpy oracle (bit-exact)."""
import os

import numpy as np
import pytest

from oracle import jpeg as ojpeg
from tests.synth import gradient_image, jpeg_bytes

pytestmark = pytest.mark.gpu


def decode_gpu(ctx, blobs, pixel_stride=3):
    from aeon_b200 import kernels as K
    outs, _ = K.jpeg_decode_batch(ctx, blobs, pixel_stride)
    return [o.cpu().numpy()[..., :3] for o in outs]


@pytest.mark.parametrize("pixel_stride", [3, 4])
def test_batch_420_matches_opencv(ctx, pixel_stride):
    import cv2
    rng = np.random.default_rng(21)
    blobs = []
    for _ in range(16):
        h, w = (int(v) for v in rng.integers(256, 513, 2))
        blobs.append(jpeg_bytes(gradient_image(rng, h, w), 90))
    got = decode_gpu(ctx, blobs, pixel_stride)
    for i, b in enumerate(blobs):
        ref = cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR)
        assert np.array_equal(got[i], ref), "image %d" % i


def test_sampling_modes_odd_sizes_restart_and_grey(ctx):
    import cv2
    rng = np.random.default_rng(22)
    cases = []
    for (h, w) in [(8, 8), (1, 1), (17, 16), (37, 53), (64, 80), (33, 47), (15, 130), (200, 9)]:
        for extra in ([], [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422],
                      [cv2.IMWRITE_JPEG_RST_INTERVAL, 3]):
            cases.append(jpeg_bytes(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), int(rng.integers(30, 100)), extra))
    cases.append(jpeg_bytes(gradient_image(rng, 45, 30)[..., 0], 85))
    got = decode_gpu(ctx, cases)
    for i, b in enumerate(cases):
        ref = cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR)
        assert np.array_equal(got[i], ref), "case %d" % i
        assert np.array_equal(got[i], ojpeg.decode(b)), "oracle case %d" % i


def test_reference_fixtures(ctx, golden_dir):
    """aeon's own test images: img_2112_70.jpg (480x360) and flowers.jpg (restart interval 38)."""
    import cv2
    blobs = [open(os.path.join(golden_dir, n), "rb").read() for n in ("img_2112_70.jpg", "flowers.jpg")]
    got = decode_gpu(ctx, blobs)
    for g, b in zip(got, blobs):
        assert np.array_equal(g, cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR))


def test_corrupt_streams_raise(ctx):
    from aeon_b200 import kernels as K
    from aeon_b200._lib import AeonError
    for blob in (b"", b"\x00" * 64, b"\xff\xd8\xff\xd9"):
        with pytest.raises(AeonError, match="Decoding image failed"):
            K.jpeg_entropy_decode(blob)


def test_region_decode_equals_the_same_pixels_of_the_full_decode(ctx):
    """Only the MCUs a crop box can touch are decoded; inside the box the pixels must equal the full decode."""
    import ctypes as C
    import cv2
    import torch
    from aeon_b200 import _lib as L, kernels as K
    rng = np.random.default_rng(23)
    dev = torch.device("cuda", ctx.device)
    for (h, w), extra in [((300, 420), []), ((97, 131), []), ((256, 256), [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422]),
                          ((64, 64), [cv2.IMWRITE_JPEG_RST_INTERVAL, 5])]:
        blob = jpeg_bytes(gradient_image(rng, h, w), 90, extra)
        ref = cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_COLOR)
        info = K.jpeg_parse(blob)
        for _ in range(6):
            cw, ch = int(rng.integers(1, w + 1)), int(rng.integers(1, h + 1))
            cx, cy = int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1))
            roi = (C.c_int32 * 4)()
            L.check(ctx.lib.aeonb_jpeg_roi_for_crop(C.byref(info), cx, cy, cw, ch, roi))
            mw, mh = 8 * info.hs[0], 8 * info.vs[0]
            rx, ry = roi[0] * mw, roi[1] * mh
            rw, rh = min(w, roi[2] * mw) - rx, min(h, roi[3] * mh) - ry
            assert rx <= cx and ry <= cy and rx + rw >= cx + cw and ry + rh >= cy + ch
            d = (L.JpegDesc * 1)()
            d[0].width, d[0].height, d[0].ncomp = rw, rh, info.ncomp
            coefs, quants, keep = [], [], []
            for c in range(info.ncomp):
                bw, bh = (roi[2] - roi[0]) * info.hs[c], (roi[3] - roi[1]) * info.vs[c]
                coefs.append(np.zeros(bw * bh * 64, np.int16))
                quants.append(np.zeros(64, np.uint16))
                d[0].hs[c], d[0].vs[c], d[0].blocks_w[c], d[0].blocks_h[c] = info.hs[c], info.vs[c], bw, bh
            cp = (C.c_void_p * 3)(*[c.ctypes.data for c in coefs])
            qp = (C.c_void_p * 3)(*[q.ctypes.data for q in quants])
            buf = (C.c_char * len(blob)).from_buffer_copy(blob)
            L.check(ctx.lib.aeonb_jpeg_entropy_decode_roi(buf, len(blob), roi, cp, qp))
            with torch.cuda.stream(ctx.torch_stream):
                for c in range(info.ncomp):
                    ct, qt = torch.from_numpy(coefs[c]).to(dev), torch.from_numpy(quants[c].view(np.int16)).to(dev)
                    keep += [ct, qt]
                    d[0].coef[c], d[0].quant[c] = ct.data_ptr(), qt.data_ptr()
                pitch = (rw * 3 + 15) // 16 * 16
                out = torch.zeros((rh, pitch), dtype=torch.uint8, device=dev)
                d[0].dst, d[0].dst_pitch, d[0].dst_pixel_stride = out.data_ptr(), pitch, 3
                L.check(ctx.lib.aeonb_jpeg_backend_batch(ctx.handle, d, 1))
                ctx.synchronize()
            got = out.cpu().numpy()[:, :rw * 3].reshape(rh, rw, 3)
            assert np.array_equal(got[cy - ry:cy - ry + ch, cx - rx:cx - rx + cw], ref[cy:cy + ch, cx:cx + cw]), (h, w, cx, cy, cw, ch)


def test_progressive_streams_match_opencv(ctx):
    """Progressive files (SOF2) are entropy-decoded on the host, scan by scan; the GPU back end is the same."""
    import cv2
    rng = np.random.default_rng(29)
    cases = []
    for (h, w) in [(64, 64), (37, 53), (200, 150), (8, 8), (1, 1), (375, 500), (33, 47)]:
        for extra in ([], [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422], [cv2.IMWRITE_JPEG_RST_INTERVAL, 3]):
            cases.append(jpeg_bytes(gradient_image(rng, h, w), int(rng.integers(30, 100)), [cv2.IMWRITE_JPEG_PROGRESSIVE, 1] + extra))
    cases.append(jpeg_bytes(gradient_image(rng, 45, 30)[..., 0], 85, [cv2.IMWRITE_JPEG_PROGRESSIVE, 1]))
    assert all(b"\xff\xc2" in c for c in cases)
    got = decode_gpu(ctx, cases)
    for i, b in enumerate(cases):
        assert np.array_equal(got[i], cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR)), "case %d" % i


def test_exif_orientation_is_applied_as_opencv_does(ctx):
    import cv2
    from tests.synth import with_exif_orientation
    rng = np.random.default_rng(30)
    cases = []
    for o in range(1, 9):
        h, w = (int(v) for v in rng.integers(20, 200, 2))
        cases.append(with_exif_orientation(jpeg_bytes(gradient_image(rng, h, w), 90), o, big_endian=bool(o % 2)))
    got = decode_gpu(ctx, cases)
    for i, b in enumerate(cases):
        ref = cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR)
        assert got[i].shape == ref.shape and np.array_equal(got[i], ref), "orientation %d" % (i + 1)


def test_440_and_411_sampling(ctx):
    """4:4:0 (libjpeg's vertical-only triangle filter) and 4:1:1 (replication), baseline and progressive, odd sizes."""
    import cv2
    rng = np.random.default_rng(33)
    cases = []
    for (h, w) in [(8, 8), (1, 1), (17, 16), (37, 53), (64, 80), (33, 47), (15, 130), (200, 9), (375, 500)]:
        for factor in (cv2.IMWRITE_JPEG_SAMPLING_FACTOR_440, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_411):
            for extra in ([], [cv2.IMWRITE_JPEG_PROGRESSIVE, 1], [cv2.IMWRITE_JPEG_RST_INTERVAL, 2]):
                cases.append(jpeg_bytes(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), int(rng.integers(30, 100)),
                                        [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, factor] + extra))
    got = decode_gpu(ctx, cases)
    for i, b in enumerate(cases):
        assert np.array_equal(got[i], cv2.imdecode(np.frombuffer(b, np.uint8), cv2.IMREAD_COLOR)), "case %d" % i
