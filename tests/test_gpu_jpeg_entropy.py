"""Device entropy decoders (a thread block per JPEG stream decoding segments speculatively; one warp per stream for streams with
restart markers) against the host decoder and against the oracle: identical coefficient planes."""
import ctypes as C
import os

import numpy as np
import pytest

from tests.synth import gradient_image, jpeg_bytes

pytestmark = pytest.mark.gpu


def host_planes(blob, roi=None):
    from aeon_b200 import _lib as L
    from aeon_b200 import kernels as K
    if roi is None:
        info, coefs, quants = K.jpeg_entropy_decode(blob)
        return info, coefs, quants
    lib = L.load()
    info = K.jpeg_parse(blob)
    nb = [(roi[2] - roi[0]) * info.hs[c] * (roi[3] - roi[1]) * info.vs[c] for c in range(info.ncomp)]
    coefs = [np.zeros(max(n * 64, 1), np.int16) for n in nb] + [np.zeros(1, np.int16)] * (3 - info.ncomp)
    quants = [np.zeros(64, np.uint16) for _ in range(3)]
    cp = (C.c_void_p * 3)(*[c.ctypes.data for c in coefs])
    qp = (C.c_void_p * 3)(*[q.ctypes.data for q in quants])
    buf = (C.c_char * len(blob)).from_buffer_copy(blob)
    r = (C.c_int32 * 4)(*roi)
    L.check(lib.aeonb_jpeg_entropy_decode_roi(buf, len(blob), r, cp, qp))
    return info, coefs[:info.ncomp], quants[:info.ncomp]


@pytest.fixture(params=[True, False], ids=["block-parallel", "one-warp"])
def parallel(request):
    return request.param


def check(ctx, blobs, rois=None, parallel=True):
    from aeon_b200 import kernels as K
    got = K.jpeg_entropy_decode_device(ctx, blobs, rois, parallel)
    for i, blob in enumerate(blobs):
        info, planes, quant, status = got[i]
        assert status == 0, "record %d status %d" % (i, status)
        hinfo, hcoefs, hquants = host_planes(blob, None if rois is None else rois[i])
        assert info.ncomp == hinfo.ncomp
        for c in range(info.ncomp):
            assert np.array_equal(planes[c].cpu().numpy(), hcoefs[c][:planes[c].numel()]), "record %d component %d" % (i, c)
            assert np.array_equal(quant[c], hquants[c])


def test_sampling_modes_sizes_and_restarts(ctx, parallel):
    import cv2
    rng = np.random.default_rng(61)
    blobs = []
    for (h, w) in [(8, 8), (1, 1), (17, 16), (37, 53), (64, 80), (33, 47), (15, 130), (200, 9), (256, 256)]:
        for extra in ([], [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_440],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_411],
                      [cv2.IMWRITE_JPEG_RST_INTERVAL, 3], [cv2.IMWRITE_JPEG_OPTIMIZE, 1]):
            blobs.append(jpeg_bytes(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), int(rng.integers(30, 101)), extra))
    blobs.append(jpeg_bytes(gradient_image(rng, 45, 30)[..., 0], 85))
    check(ctx, blobs, parallel=parallel)


def test_noise_at_quality_100_exercises_long_codes_and_stuffing(ctx, parallel):
    rng = np.random.default_rng(62)
    blobs = [jpeg_bytes(rng.integers(0, 256, (96, 160, 3), dtype=np.uint8), 100) for _ in range(4)]
    assert any(b"\xff\x00" in b for b in blobs)
    check(ctx, blobs, parallel=parallel)


def test_natural_batch_and_reference_fixtures(ctx, golden_dir, parallel):
    rng = np.random.default_rng(63)
    blobs = [jpeg_bytes(gradient_image(rng, int(rng.integers(256, 513)), int(rng.integers(256, 513))), 90) for _ in range(32)]
    blobs += [open(os.path.join(golden_dir, n), "rb").read() for n in ("img_2112_70.jpg", "flowers.jpg")]
    check(ctx, blobs, parallel=parallel)


def test_regions(ctx, parallel):
    from aeon_b200 import kernels as K
    rng = np.random.default_rng(64)
    blobs, rois = [], []
    for _ in range(12):
        h, w = (int(v) for v in rng.integers(100, 400, 2))
        blob = jpeg_bytes(gradient_image(rng, h, w), 85)
        info = K.jpeg_parse(blob)
        mcux, mcuy = info.blocks_w[0] // info.hs[0], info.blocks_h[0] // info.vs[0]
        x0, y0 = int(rng.integers(0, mcux)), int(rng.integers(0, mcuy))
        x1, y1 = int(rng.integers(x0 + 1, mcux + 1)), int(rng.integers(y0 + 1, mcuy + 1))
        blobs.append(blob)
        rois.append((x0, y0, x1, y1))
    check(ctx, blobs, rois, parallel)


def test_malformed_stream_sets_status_and_returns(ctx, parallel):
    """A scan of 0xFF filler and one of random bytes: the kernel flags them (or decodes garbage) and terminates."""
    from aeon_b200 import kernels as K
    rng = np.random.default_rng(65)
    good = jpeg_bytes(gradient_image(rng, 128, 128), 90)
    sos = good.index(b"\xff\xda")
    head = good[:sos + 14]
    truncated = good[:sos + 14 + 200] + b"\xff\xd9"
    noise = head + bytes(rng.integers(0, 255, 3000, dtype=np.uint8)) + b"\xff\xd9"
    got = K.jpeg_entropy_decode_device(ctx, [good, truncated, noise], None, parallel)
    assert got[0][3] == 0
    assert got[1][3] in (0, 1) and got[2][3] in (0, 1)
    # and the context is still usable
    check(ctx, [good], parallel=parallel)


def test_large_picture_and_many_streams(ctx, parallel):
    """A 2048x1536 picture (segments of several KB per thread) and a launch of 600 small streams (more blocks than fit at once)."""
    rng = np.random.default_rng(66)
    big = jpeg_bytes(gradient_image(rng, 1536, 2048), 92)
    assert len(big) > 400_000
    check(ctx, [big], parallel=parallel)
    small = [jpeg_bytes(gradient_image(rng, int(rng.integers(16, 64)), int(rng.integers(16, 64))), 80) for _ in range(40)]
    check(ctx, [small[i % 40] for i in range(600)], parallel=parallel)


def test_device_decoder_against_the_oracle_planes(ctx, golden_dir, parallel):
    """Both device kernels against oracle/jpeg.py's own Huffman decoder (not only against the library's host decoder)."""
    import cv2
    from aeon_b200 import kernels as K
    from oracle import jpeg as ojpeg
    rng = np.random.default_rng(67)
    blobs = [jpeg_bytes(gradient_image(rng, 40, 56), 90), jpeg_bytes(gradient_image(rng, 33, 47), 75, [cv2.IMWRITE_JPEG_RST_INTERVAL, 2]),
             jpeg_bytes(rng.integers(0, 256, (24, 24, 3), dtype=np.uint8), 100, [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444]),
             open(os.path.join(golden_dir, "img_2112_70.jpg"), "rb").read()]
    got = K.jpeg_entropy_decode_device(ctx, blobs, None, parallel)
    for i, blob in enumerate(blobs):
        info, planes, quant, status = got[i]
        co = ojpeg.entropy_decode(blob)
        assert status == 0 and (info.width, info.height, info.ncomp) == (co.width, co.height, co.ncomp)
        for c in range(info.ncomp):
            mine = planes[c].cpu().numpy().reshape(info.blocks_h[c], info.blocks_w[c], 8, 8).transpose(0, 1, 3, 2)  # column-major blocks
            assert np.array_equal(mine, co.blocks[c]), (i, c)


def test_streams_with_more_segments_than_the_smallest_segment_allows(ctx, golden_dir):
    """Streams longer than threads x smallest segment get longer segments, and their last, short segment can end a few
    bits before a checkpoint position.  The fixture is a 90 KB stream of the benchmark's generator (507 segments of 176
    bytes) whose last segment ends 8 bits before its second checkpoint: a run that stepped over that position with its
    last symbol once left a note there that a later run fell into step with, and the stream was reported as malformed
    although every coefficient was right."""
    blob = open(os.path.join(golden_dir, "entropy_stream_507_segments.jpg"), "rb").read()
    check(ctx, [blob])
    info = host_planes(blob)[0]
    mcux, mcuy = info.blocks_w[0] // info.hs[0], info.blocks_h[0] // info.vs[0]
    check(ctx, [blob] * 4, rois=[(0, 0, mcux, mcuy), (3, 5, mcux - 2, mcuy), (0, mcuy - 1, mcux, mcuy), (0, 0, mcux, mcuy - 1)])
    rng = np.random.default_rng(77)
    big = []
    for k in range(24):   # 84-140 KB: segments of 164 to 280 bytes, last segments of every length
        h, w = int(rng.integers(440, 513)), int(rng.integers(440, 513))
        img = np.clip(gradient_image(rng, h, w).astype(np.int16) + rng.integers(-28 - k, 29 + k, (h, w, 3)), 0, 255).astype(np.uint8)
        big.append(jpeg_bytes(img, 92))
    assert min(len(b) for b in big) > 84000
    check(ctx, big)
