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
