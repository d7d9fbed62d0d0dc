"""Rotation pre-pass (image::rotate, src/image.cpp:53-75) through the C ABI against the oracle: bit-exact."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import image_ops as ops

pytestmark = pytest.mark.gpu


def rotate_gpu(ctx, images, angles, src_stride=3, dst_stride=3, nearest=False):
    from aeon_b200 import _lib as L
    dev = torch.device("cuda", ctx.device)
    n = len(images)
    descs = (L.RotateDesc * n)()
    keep, outs = [], []
    for i, (img, angle) in enumerate(zip(images, angles)):
        h, w = img.shape[:2]
        if src_stride == 4:
            img = np.concatenate([img, np.full((h, w, 1), 201, np.uint8)], -1)
        src = torch.from_numpy(np.ascontiguousarray(img)).to(dev)
        pitch = (w * dst_stride + 15) // 16 * 16
        dst = torch.full((h, pitch), 123, dtype=torch.uint8, device=dev)
        d = descs[i]
        d.src, d.src_pitch, d.src_pixel_stride = src.data_ptr(), w * src_stride, src_stride
        d.width, d.height, d.angle, d.nearest = w, h, int(angle), int(nearest)
        d.dst, d.dst_pitch, d.dst_pixel_stride = dst.data_ptr(), pitch, dst_stride
        keep += [src, dst]
        outs.append(torch.as_strided(dst, (h, w, dst_stride), (pitch, dst_stride, 1)))
    torch.cuda.synchronize(dev)
    L.check(ctx.lib.aeonb_rotate_batch(ctx.handle, descs, n))
    ctx.synchronize()
    return [o.cpu().numpy()[..., :3] for o in outs]


@pytest.mark.parametrize("strides", [(3, 3), (4, 3), (3, 4)])
def test_rotation_matches_oracle(ctx, strides):
    rng = np.random.default_rng(91)
    cases = [(40, 60, 7), (97, 131, -13), (64, 64, 20), (200, 150, 3), (33, 70, -20), (256, 384, 45), (50, 50, 90), (31, 17, 180),
             (120, 80, -1), (1, 1, 5), (2, 300, 11), (375, 500, 19), (512, 512, -20)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for h, w, _ in cases]
    got = rotate_gpu(ctx, images, [a for _, _, a in cases], *strides)
    for img, (h, w, angle), g in zip(images, cases, got):
        assert np.array_equal(g, ops.rotate(img, angle)), (h, w, angle)


def test_rotation_matches_opencv_binary(ctx):
    import cv2
    rng = np.random.default_rng(92)
    images = [rng.integers(0, 256, (int(rng.integers(20, 300)), int(rng.integers(20, 300)), 3), dtype=np.uint8) for _ in range(24)]
    angles = [int(a) for a in rng.integers(-45, 46, len(images))]
    got = rotate_gpu(ctx, images, angles)
    for img, angle, g in zip(images, angles, got):
        h, w = img.shape[:2]
        ref = cv2.warpAffine(img, cv2.getRotationMatrix2D((w // 2, h // 2), angle, 1.0), (w, h), flags=cv2.INTER_LINEAR,
                             borderMode=cv2.BORDER_CONSTANT, borderValue=(0, 0, 0, 0))
        assert np.array_equal(g, ref), (h, w, angle)


def test_rotation_without_interpolation_for_masks(ctx):
    """image::rotate(.., interpolate = false) as the pixelmask / depthmap transformers call it (src/etl_pixel_mask.cpp:71-73):
    against the oracle and against cv2.warpAffine(INTER_NEAREST) itself; grey pictures stored as B = G = R."""
    import cv2
    rng = np.random.default_rng(93)
    images, angles = [], []
    for _ in range(24):
        h, w = int(rng.integers(1, 300)), int(rng.integers(1, 300))
        grey = rng.integers(0, 256, (h, w, 1), dtype=np.uint8)
        images.append(np.repeat(grey, 3, axis=2) if rng.integers(2) else rng.integers(0, 256, (h, w, 3), dtype=np.uint8))
        angles.append(int(rng.integers(-180, 181)) or 13)
    got = rotate_gpu(ctx, images, angles, nearest=True)
    for img, angle, g in zip(images, angles, got):
        h, w = img.shape[:2]
        ref = cv2.warpAffine(img, cv2.getRotationMatrix2D((w // 2, h // 2), angle, 1.0), (w, h), flags=cv2.INTER_NEAREST,
                             borderMode=cv2.BORDER_CONSTANT, borderValue=(0, 0, 0, 0))
        assert np.array_equal(g, ops.rotate(img, angle, interpolate=False)), (h, w, angle)
        assert np.array_equal(g, ref.reshape(img.shape)), (h, w, angle)


def test_bad_arguments(ctx):
    from aeon_b200 import _lib as L
    d = (L.RotateDesc * 1)()
    assert ctx.lib.aeonb_rotate_batch(ctx.handle, d, 1) == L.ERR_INVALID
    assert ctx.lib.aeonb_rotate_batch(ctx.handle, d, 0) == 0
