"""Pins of the numpy oracle: aeon's golden vectors and known answers, and the OpenCV binary (cv2 4.13)."""
import os

import cv2
import numpy as np
import pytest

from oracle import cv2_path as cvp
from oracle import image_ops as ops
from tests.synth import gradient_image

GOLD_MEAN, GOLD_STD = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]


def _fixture(golden_dir):
    return cv2.imdecode(np.fromfile(os.path.join(golden_dir, "img_2112_70.jpg"), np.uint8), cv2.IMREAD_COLOR)


def test_reference_golden_train(golden_dir):
    """aeon test/test_provider.cpp:96-179."""
    img = _fixture(golden_dir)
    p = ops.ImageParams(cropbox=(50, 50, 171, 201), output_size=(224, 224), flip=True)
    got = ops.load_image(ops.transform_single_image(img, p), True, True, "float", GOLD_MEAN, GOLD_STD)
    gold = np.fromfile(os.path.join(golden_dir, "augment_output_linear_train.bin"), np.float32).reshape(3, 224, 224)
    assert np.abs(got - gold).max() <= 1e-5   # the reference's own bound is 1e-3


def test_reference_golden_eval(golden_dir):
    """aeon test/test_provider.cpp:181-261: resize_short 256 (-> 341x256), centre crop (58,16,224x224)."""
    img = _fixture(golden_dir)
    p = ops.ImageParams(cropbox=(58, 16, 224, 224), output_size=(224, 224), resize_short_size=256)
    got = ops.load_image(ops.transform_single_image(img, p), True, True, "float", GOLD_MEAN, GOLD_STD)
    gold = np.fromfile(os.path.join(golden_dir, "augment_output_linear_eval.bin"), np.float32).reshape(3, 224, 224)
    assert np.abs(got - gold).max() <= 1e-5


def test_reference_contrast_and_brightness_known_answers():
    """aeon test/test_image.cpp:1367-1480."""
    def three(b, g, r):
        img = np.zeros((1, 3, 3), np.uint8)
        img[0, 0], img[0, 1], img[0, 2] = b, g, r
        return img
    img = three((0, 0, 0), (127, 127, 127), (255, 255, 255))
    assert ops.cbsjitter(img, 0.5, 1.0, 1.0, 0)[0, :, 0].tolist() == [64, 127, 191]
    assert ops.cbsjitter(img, 0.1, 1.0, 1.0, 0)[0, :, 0].tolist() == [115, 127, 140]
    img = three((0, 0, 0), (127, 127, 127), (255, 255, 255))
    assert ops.cbsjitter(img, 1.0, 0.5, 1.0, 0)[0, :, 0].tolist() == [0, 64, 128]
    assert ops.cbsjitter(img, 1.0, 0.1, 1.0, 0)[0, :, 0].tolist() == [0, 13, 26]
    assert ops.cbsjitter(img, 1.0, 1.5, 1.0, 0)[0, :, 0].tolist() == [0, 190, 255]


def test_resize_linear_matches_opencv_on_many_shapes():
    rng = np.random.default_rng(1)
    for _ in range(40):
        h, w = (int(v) for v in rng.integers(1, 300, 2))
        ow, oh = (int(v) for v in rng.integers(1, 300, 2))
        src = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        assert np.array_equal(ops.resize_linear_u8(src, ow, oh), cv2.resize(src, (ow, oh), interpolation=cv2.INTER_LINEAR))
    src = rng.integers(0, 256, (128, 96, 3), dtype=np.uint8)
    assert np.array_equal(ops.resize_linear_u8(src, 48, 64), cv2.resize(src, (48, 64), interpolation=cv2.INTER_LINEAR))
    assert np.array_equal(ops.resize_nearest_u8(src, 37, 51), cv2.resize(src, (37, 51), interpolation=cv2.INTER_NEAREST))


def test_resize_nearest_matches_opencv_for_every_source_width():
    """INTER_NEAREST tap positions for every source length 1..599 against a handful of output lengths: the pairs where
    d * src/dst is a whole number decide between the two ways of forming the scale factor."""
    for src_len in range(1, 600):
        row = (np.arange(src_len) % 251).astype(np.uint8).reshape(1, src_len, 1).repeat(3, axis=2)
        col = np.ascontiguousarray(row.transpose(1, 0, 2))
        for dst_len in (7, 56, 96, 112, 224, 300):
            assert np.array_equal(ops.resize_nearest_u8(row, dst_len, 1), cv2.resize(row, (dst_len, 1), interpolation=cv2.INTER_NEAREST))
            assert np.array_equal(ops.resize_nearest_u8(col, 1, dst_len), cv2.resize(col, (1, dst_len), interpolation=cv2.INTER_NEAREST))


def test_colour_matrix_transform_matches_opencv():
    rng = np.random.default_rng(2)
    img = rng.integers(0, 256, (64, 257, 3), dtype=np.uint8)
    for _ in range(10):
        m = ops.color_matrix(rng.uniform(0.3, 2.0), rng.uniform(0.0, 2.0))
        assert np.array_equal(ops.transform_u8(img, m), cv2.transform(img, m))


def _all_triples():
    v = np.arange(256, dtype=np.uint8)
    a, b, c = np.meshgrid(v, v, v, indexing="ij")
    return np.stack([a, b, c], -1)


def test_bgr2hsv_matches_opencv_exhaustively():
    img = _all_triples().reshape(4096, 4096, 3)
    assert np.array_equal(ops.bgr2hsv_u8(img), cv2.cvtColor(img, cv2.COLOR_BGR2HSV))


@pytest.mark.parametrize("width", [4096, 1])
def test_hsv2bgr_matches_opencv_exhaustively(width):
    """width 4096 exercises OpenCV's truncating vector body, width 1 its rounding scalar tail."""
    hsv = _all_triples().reshape(-1, width, 3)
    assert np.array_equal(ops.hsv2bgr_u8(hsv), cv2.cvtColor(hsv, cv2.COLOR_HSV2BGR))


def test_hsv_body_and_tail_boundary():
    rng = np.random.default_rng(3)
    for w in (31, 32, 33, 57, 64, 100, 224, 300):
        hsv = rng.integers(0, 256, (5, w, 3), dtype=np.uint8)
        assert np.array_equal(ops.hsv2bgr_u8(hsv), cv2.cvtColor(hsv, cv2.COLOR_HSV2BGR)), w


def test_hue_wrap_examples():
    """C remainder stored through a uint8_t: (5,-18)->243, (0,-1)->255, (18,-18)->0, (179,+18)->17."""
    for h, hue, want in [(5, -18, 243), (0, -1, 255), (18, -18, 0), (179, 18, 17)]:
        t = np.fmod(np.int32(h + hue), 180).astype(np.int32) & 0xFF
        assert int(t) == want


def test_full_pipeline_matches_opencv_call_sequence():
    rng = np.random.default_rng(4)
    for _ in range(25):
        h, w = (int(v) for v in rng.integers(40, 400, 2))
        src = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        cw, ch = int(rng.integers(8, w + 1)), int(rng.integers(8, h + 1))
        p = ops.ImageParams(cropbox=(int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch),
                            output_size=(int(rng.integers(16, 300)), int(rng.integers(16, 300))), flip=bool(rng.integers(2)),
                            contrast=rng.uniform(0.6, 1.4), brightness=rng.uniform(0.6, 1.4), saturation=rng.uniform(0.6, 1.4),
                            hue=int(rng.integers(-18, 19)), lighting=list(rng.normal(0, 0.1, 3).astype(np.float32)),
                            color_noise_std=0.1)
        a, b = ops.transform_single_image(src, p), cvp.transform_single_image(src, p)
        assert np.array_equal(a, b)
        fa = ops.load_image(a, True, True, "float", [0.4, 0.5, 0.6], [0.2, 0.3, 0.0])
        fb = cvp.load_image(b, True, True, "float", [0.4, 0.5, 0.6], [0.2, 0.3, 0.0])
        assert np.abs(fa - fb).max() <= 1e-6


def test_expand_padding_and_video_layout():
    rng = np.random.default_rng(5)
    src = gradient_image(rng, 20, 30)
    p = ops.ImageParams(expand_ratio=2.0, expand_offset=(7, 3), expand_size=(60, 40), cropbox=(0, 0, 60, 40), output_size=(60, 40))
    out = ops.transform_single_image(src, p)
    assert np.array_equal(out[3:23, 7:37], src) and out[:3].sum() == 0 and out[:, :7].sum() == 0
    frames = [np.full((4, 5, 3), i, np.uint8) for i in range(3)]
    v = ops.load_video(frames, 5)            # aeon test/test_video.cpp:119-180 layout: C x T x H x W
    assert v.shape == (3, 5, 4, 5) and v[:, 2].min() == 2 and not v[:, 3:].any()


def test_rotation_matches_opencv_warp_affine():
    """image::rotate (src/image.cpp:53-75): the restated fixed-point warpAffine against the OpenCV binary."""
    import cv2
    rng = np.random.default_rng(77)
    for (h, w, angle) in [(40, 60, 7), (97, 131, -13), (64, 64, 20), (200, 150, 3), (33, 70, -20), (256, 384, 45), (50, 50, 90),
                          (31, 17, 180), (120, 80, -1), (1, 1, 5), (2, 300, 11)]:
        img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        ref = cv2.warpAffine(img, cv2.getRotationMatrix2D((w // 2, h // 2), angle, 1.0), (w, h), flags=cv2.INTER_LINEAR,
                             borderMode=cv2.BORDER_CONSTANT, borderValue=(0, 0, 0, 0))
        assert np.array_equal(ops.rotate(img, angle), ref), (h, w, angle)
    img = rng.integers(0, 256, (20, 30, 3), dtype=np.uint8)
    assert ops.rotate(img, 0) is img


def test_nearest_rotation_and_pixel_mask_transform_match_opencv():
    """image::rotate with interpolate == false, and pixel_mask::transformer::transform (src/etl_pixel_mask.cpp:62-92) as
    the same OpenCV calls; the reference's own mask tests (test/test_pixel_mask.cpp:76-209) ask that a black / white
    checkerboard stays black / white through scale up, scale down and rotation, and that values survive the loader."""
    import cv2
    rng = np.random.default_rng(79)
    for _ in range(60):
        h, w = int(rng.integers(1, 300)), int(rng.integers(1, 300))
        angle = int(rng.integers(-180, 181)) or 9
        img = rng.integers(0, 256, (h, w, 1) if rng.integers(2) else (h, w, 3), dtype=np.uint8)
        ref = cv2.warpAffine(img, cv2.getRotationMatrix2D((w // 2, h // 2), angle, 1.0), (w, h), flags=cv2.INTER_NEAREST,
                             borderMode=cv2.BORDER_CONSTANT, borderValue=(0, 0, 0, 0))
        assert np.array_equal(ops.rotate(img, angle, interpolate=False), ref.reshape(img.shape)), (h, w, angle)
    board = (((np.add.outer(np.arange(256), np.arange(256)) % 2) * 255).astype(np.uint8))[..., None]
    for out_size, angle in (((300, 300), 0), ((100, 100), 0), ((256, 256), 45)):
        p = ops.ImageParams()
        p.cropbox, p.output_size, p.angle = (0, 0, 256, 256), out_size, angle
        tx = ops.transform_pixel_mask(board, p)
        assert tx.shape == (out_size[1], out_size[0], 1) and set(np.unique(tx)) <= {0, 255}
    for _ in range(20):
        h, w = int(rng.integers(40, 200)), int(rng.integers(40, 200))
        mask = rng.integers(0, 21, (h, w, 1), dtype=np.uint8)
        p = ops.ImageParams()
        cw, ch = int(rng.integers(8, w + 1)), int(rng.integers(8, h + 1))
        p.cropbox = (int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch)
        p.output_size, p.angle, p.flip = (int(rng.integers(8, 120)), int(rng.integers(8, 120))), int(rng.integers(-30, 31)), bool(rng.integers(2))
        ref = mask[..., 0]
        if p.angle:
            ref = cv2.warpAffine(ref, cv2.getRotationMatrix2D((w // 2, h // 2), p.angle, 1.0), (w, h), flags=cv2.INTER_NEAREST,
                                 borderMode=cv2.BORDER_CONSTANT, borderValue=(0, 0, 0, 0))
        x, y = p.cropbox[:2]
        ref = cv2.resize(ref[y:y + ch, x:x + cw], p.output_size, interpolation=cv2.INTER_NEAREST)
        if p.flip:
            ref = cv2.flip(ref, 1)
        assert np.array_equal(ops.transform_pixel_mask(mask, p)[..., 0], ref)
    cols = np.broadcast_to(np.arange(256, dtype=np.uint8), (256, 256))[..., None]
    p = ops.ImageParams()
    p.cropbox, p.output_size = (0, 0, 256, 256), (256, 256)
    loaded = ops.load_image(ops.transform_pixel_mask(cols, p), True, False, "int32_t")
    assert loaded.dtype == np.int32 and np.array_equal(loaded[0], np.broadcast_to(np.arange(256), (256, 256)))


def test_area_resize_matches_opencv_in_all_three_regimes():
    """cv::resize INTER_AREA: whole-factor boxes (2x2 and others), weighted cells, and the enlarging / mixed case."""
    import cv2
    rng = np.random.default_rng(78)
    cases = [(37, 53, 20, 31), (100, 130, 64, 64), (64, 64, 32, 32), (90, 90, 30, 30), (50, 70, 49, 69), (64, 96, 16, 32),
             (60, 60, 30, 20), (33, 47, 33, 20), (20, 31, 37, 53), (64, 64, 100, 130), (32, 32, 64, 64), (30, 40, 45, 41),
             (40, 30, 20, 45), (45, 50, 90, 25), (17, 19, 17, 19), (8, 9, 1, 1), (5, 5, 7, 3), (300, 411, 224, 224),
             (448, 448, 224, 224), (96, 96, 32, 32), (1, 1, 4, 4), (2, 3, 1, 1)]
    cases += [tuple(int(v) for v in rng.integers(1, 120, 4)) for _ in range(60)]
    for (sh, sw, dh, dw) in cases:
        img = rng.integers(0, 256, (sh, sw, 3), dtype=np.uint8)
        assert np.array_equal(ops.resize_area_u8(img, dw, dh), cv2.resize(img, (dw, dh), interpolation=cv2.INTER_AREA)), (sh, sw, dh, dw)


def test_cubic_resize_matches_opencvs_own_implementation():
    """cv::resize INTER_CUBIC as OpenCV's own code computes it (IPP, which this cv2 build would otherwise hand 8-bit cubic
    resizes to, is switched off for the comparison): three- and one-channel pictures, shrinking, enlarging, tiny sizes."""
    import cv2
    rng = np.random.default_rng(81)
    cases = [(300, 411, 224, 224), (1, 6, 18, 119), (45, 81, 15, 104), (41, 28, 65, 107), (39, 118, 70, 23), (37, 53, 20, 31),
             (100, 130, 64, 64), (1, 1, 5, 5), (3, 2, 9, 1), (8, 9, 1, 1)]
    cases += [tuple(int(v) for v in rng.integers(1, 130, 4)) for _ in range(80)]
    old = cv2.ipp.useIPP()
    cv2.ipp.setUseIPP(False)
    try:
        for (sh, sw, dh, dw) in cases:
            for cn in (3, 1):
                img = rng.integers(0, 256, (sh, sw, cn), dtype=np.uint8)
                ref = cv2.resize(img, (dw, dh), interpolation=cv2.INTER_CUBIC).reshape(dh, dw, cn)
                assert np.array_equal(ops.resize_cubic_u8(img, dw, dh), ref), (sh, sw, dh, dw, cn)
    finally:
        cv2.ipp.setUseIPP(old)


def test_lanczos4_resize_matches_opencv():
    import cv2
    rng = np.random.default_rng(83)
    cases = [(37, 53, 20, 31), (100, 130, 64, 64), (20, 31, 37, 53), (64, 64, 100, 130), (30, 40, 45, 41), (17, 19, 17, 40), (50, 50, 25, 25),
             (9, 9, 30, 30), (1, 1, 5, 5), (3, 2, 9, 1), (300, 411, 224, 224)]
    cases += [tuple(int(v) for v in rng.integers(1, 100, 4)) for _ in range(40)]
    for (sh, sw, dh, dw) in cases:
        img = rng.integers(0, 256, (sh, sw, 3), dtype=np.uint8)
        assert np.array_equal(ops.resize_lanczos4_u8(img, dw, dh), cv2.resize(img, (dw, dh), interpolation=cv2.INTER_LANCZOS4)), (sh, sw, dh, dw)
