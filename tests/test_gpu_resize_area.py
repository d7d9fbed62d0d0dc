"""INTER_AREA / INTER_CUBIC resize pass through the C ABI against the oracle (which is pinned to cv2.resize): bit-exact."""
import numpy as np
import pytest
import torch

from oracle import image_ops as ops

pytestmark = pytest.mark.gpu


def resize_gpu(ctx, jobs, src_stride=3, dst_stride=3, interp=None, channels=3):
    """jobs: list of (image, canvas_xy, crop_xywh, out_wh); the canvas is zero outside the image."""
    from aeon_b200 import _lib as L
    dev = torch.device("cuda", ctx.device)
    descs = (L.ResizeDesc * len(jobs))()
    keep, outs = [], []
    for i, (img, (cx, cy), (x, y, w, h), (ow, oh)) in enumerate(jobs):
        ih, iw = img.shape[:2]
        if src_stride == 4:
            img = np.concatenate([img, np.full((ih, iw, 1), 99, np.uint8)], -1)
        src = torch.from_numpy(np.ascontiguousarray(img)).to(dev)
        pitch = (ow * dst_stride + 15) // 16 * 16
        dst = torch.full((oh, pitch), 55, dtype=torch.uint8, device=dev)
        d = descs[i]
        d.src, d.src_pitch, d.src_pixel_stride, d.src_w, d.src_h = src.data_ptr(), iw * src_stride, src_stride, iw, ih
        d.canvas_x, d.canvas_y, d.crop_x, d.crop_y, d.crop_w, d.crop_h = cx, cy, x, y, w, h
        d.interp, d.out_w, d.out_h, d.channels = (L.INTERP_AREA if interp is None else interp), ow, oh, channels
        d.dst, d.dst_pitch, d.dst_pixel_stride = dst.data_ptr(), pitch, dst_stride
        keep += [src, dst]
        outs.append(torch.as_strided(dst, (oh, ow, dst_stride), (pitch, dst_stride, 1)))
    torch.cuda.synchronize(dev)
    L.check(ctx.lib.aeonb_resize_batch(ctx.handle, descs, len(jobs)))
    ctx.synchronize()
    return [o.cpu().numpy()[..., :3] for o in outs]


def window(img, canvas_xy, crop):
    """The crop box of the zero canvas on which the image sits."""
    (cx, cy), (x, y, w, h) = canvas_xy, crop
    canvas = np.zeros((max(cy + img.shape[0], y + h), max(cx + img.shape[1], x + w), 3), np.uint8)
    canvas[cy:cy + img.shape[0], cx:cx + img.shape[1]] = img
    return canvas[y:y + h, x:x + w]


@pytest.mark.parametrize("strides", [(3, 3), (4, 3), (3, 4)])
def test_all_regimes_match_the_oracle(ctx, strides):
    rng = np.random.default_rng(79)
    shapes = [(37, 53, 20, 31), (100, 130, 64, 64), (64, 64, 32, 32), (90, 90, 30, 30), (50, 70, 49, 69), (64, 96, 16, 32),
              (60, 60, 30, 20), (20, 31, 37, 53), (64, 64, 100, 130), (30, 40, 45, 41), (40, 30, 20, 45), (17, 19, 17, 19), (8, 9, 1, 1),
              (300, 411, 224, 224), (448, 448, 224, 224), (1, 1, 4, 4)]
    shapes += [tuple(int(v) for v in rng.integers(1, 150, 4)) for _ in range(40)]
    jobs = []
    for (sh, sw, dh, dw) in shapes:
        img = rng.integers(0, 256, (sh, sw, 3), dtype=np.uint8)
        jobs.append((img, (0, 0), (0, 0, sw, sh), (dw, dh)))
    got = resize_gpu(ctx, jobs, *strides)
    for (img, _, _, (dw, dh)), g in zip(jobs, got):
        assert np.array_equal(g, ops.resize_area_u8(img, dw, dh)), (img.shape, dw, dh)


def test_crop_windows_and_expanded_canvas(ctx):
    rng = np.random.default_rng(80)
    jobs = []
    for _ in range(24):
        ih, iw = (int(v) for v in rng.integers(40, 200, 2))
        img = rng.integers(0, 256, (ih, iw, 3), dtype=np.uint8)
        cx, cy = (int(v) for v in rng.integers(0, 30, 2))                 # the picture's place on an expanded canvas
        cw, ch = iw + cx + int(rng.integers(0, 30)), ih + cy + int(rng.integers(0, 30))
        w, h = int(rng.integers(8, cw + 1)), int(rng.integers(8, ch + 1))
        x, y = int(rng.integers(0, cw - w + 1)), int(rng.integers(0, ch - h + 1))
        jobs.append((img, (cx, cy), (x, y, w, h), (int(rng.integers(8, 120)), int(rng.integers(8, 120)))))
    got = resize_gpu(ctx, jobs)
    for (img, cxy, crop, (ow, oh)), g in zip(jobs, got):
        assert np.array_equal(g, ops.resize_area_u8(window(img, cxy, crop), ow, oh))


def test_cubic_matches_the_oracle(ctx):
    from aeon_b200 import _lib as L
    rng = np.random.default_rng(82)
    shapes = [(300, 411, 224, 224), (1, 6, 18, 119), (45, 81, 15, 104), (41, 28, 65, 107), (39, 118, 70, 23), (37, 53, 20, 31),
              (100, 130, 64, 64), (1, 1, 5, 5), (3, 2, 9, 1), (8, 9, 1, 1)]
    shapes += [tuple(int(v) for v in rng.integers(1, 150, 4)) for _ in range(50)]
    jobs = [(rng.integers(0, 256, (sh, sw, 3), dtype=np.uint8), (0, 0), (0, 0, sw, sh), (dw, dh)) for (sh, sw, dh, dw) in shapes]
    got = resize_gpu(ctx, jobs, interp=L.INTERP_CUBIC)
    for (img, _, _, (dw, dh)), g in zip(jobs, got):
        assert np.array_equal(g, ops.resize_cubic_u8(img, dw, dh)), (img.shape, dw, dh)
    # a grey picture carried as B = G = R: the reference resizes a one-channel row, whose vector part is shorter
    grey = [(np.repeat(rng.integers(0, 256, (sh, sw, 1), dtype=np.uint8), 3, 2), (0, 0), (0, 0, sw, sh), (dw, dh)) for (sh, sw, dh, dw) in shapes[:30]]
    got = resize_gpu(ctx, grey, interp=L.INTERP_CUBIC, channels=1)
    for (img, _, _, (dw, dh)), g in zip(grey, got):
        want = ops.resize_cubic_u8(img[..., :1], dw, dh)
        assert np.array_equal(g, np.repeat(want, 3, 2)), (img.shape, dw, dh)


def test_lanczos4_matches_the_oracle(ctx):
    from aeon_b200 import _lib as L
    rng = np.random.default_rng(84)
    shapes = [(37, 53, 20, 31), (100, 130, 64, 64), (20, 31, 37, 53), (64, 64, 100, 130), (30, 40, 45, 41), (17, 19, 17, 40), (9, 9, 30, 30),
              (1, 1, 5, 5), (3, 2, 9, 1), (300, 411, 224, 224)]
    shapes += [tuple(int(v) for v in rng.integers(1, 120, 4)) for _ in range(30)]
    jobs = [(rng.integers(0, 256, (sh, sw, 3), dtype=np.uint8), (0, 0), (0, 0, sw, sh), (dw, dh)) for (sh, sw, dh, dw) in shapes]
    got = resize_gpu(ctx, jobs, interp=L.INTERP_LANCZOS4)
    for (img, _, _, (dw, dh)), g in zip(jobs, got):
        assert np.array_equal(g, ops.resize_lanczos4_u8(img, dw, dh)), (img.shape, dw, dh)
