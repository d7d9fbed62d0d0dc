"""Parity of the image augmentation/packing kernel with the CPU oracle, through the C ABI.

Bar: bit-exact for uint8 outputs (geometry and photometric alike, since the oracle restates
OpenCV's integer / float32 arithmetic), 1e-6 absolute for standardised float outputs."""
import numpy as np
import pytest
import torch

from oracle import image_ops as ops
from tests.synth import gradient_image

pytestmark = pytest.mark.gpu


def run_kernel(ctx, srcs, params, slot_w, slot_h, output_type="uint8_t", channel_major=True, bgr_to_rgb=False,
               mean=None, stddev=None, pixel_stride=3):
    from aeon_b200 import kernels as K
    dt = K.DTYPE_BY_NAME[output_type]
    dev = torch.device("cuda", ctx.device)
    with torch.cuda.stream(ctx.torch_stream):
        tsrc = []
        for s in srcs:
            if s is None:
                tsrc.append(None)
                continue
            if pixel_stride == 4:
                s = np.concatenate([s, np.full(s.shape[:2] + (1,), 77, np.uint8)], -1)
            tsrc.append(torch.from_numpy(np.ascontiguousarray(s)).to(dev))
        shape = (len(srcs), 3, slot_h, slot_w) if channel_major else (len(srcs), slot_h, slot_w, 3)
        out = torch.full(shape, 99, dtype=K._TORCH_DTYPE[dt], device=dev)
        lay = K.make_layout(slot_w, slot_h, dt, channel_major, bgr_to_rgb, mean, stddev)
        K.image_batch(ctx, tsrc, params, out, lay)
        ctx.synchronize()
        return out.cpu().numpy()


def oracle(src, p, slot_w, slot_h, **kw):
    img = ops.transform_single_image(src, p)
    canvas = np.zeros((slot_h, slot_w, 3), np.uint8)
    canvas[:img.shape[0], :img.shape[1]] = img
    full = ops.load_image(canvas, **kw)
    if kw.get("mean") is not None and (img.shape[0] != slot_h or img.shape[1] != slot_w):
        # the reference standardises only the image region of a fixed-aspect canvas
        z = ops.load_image(np.zeros_like(canvas), kw.get("channel_major", True), kw.get("bgr_to_rgb", False),
                           kw.get("output_type", "uint8_t"))
        roi = ops.load_image(img, **kw)
        if kw.get("channel_major", True):
            z[:, :img.shape[0], :img.shape[1]] = roi
        else:
            z[:img.shape[0], :img.shape[1]] = roi
        full = z
    return full


def random_params(rng, w, h, ow, oh, photometric):
    cw = int(rng.integers(2, w + 1))
    ch = int(rng.integers(2, h + 1))
    kw = dict(cropbox=(int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch),
              output_size=(ow, oh), flip=bool(rng.integers(2)))
    if photometric:
        kw.update(contrast=float(np.float32(rng.uniform(0.6, 1.4))), brightness=float(np.float32(rng.uniform(0.6, 1.4))),
                  saturation=float(np.float32(rng.uniform(0.6, 1.4))), hue=int(rng.integers(-18, 19)),
                  lighting=[float(v) for v in rng.normal(0, 0.1, 3).astype(np.float32)], color_noise_std=0.1)
    return ops.ImageParams(**kw)


@pytest.mark.parametrize("pixel_stride", [3, 4])
def test_geometry_uint8_chw_bit_exact(ctx, pixel_stride):
    rng = np.random.default_rng(11)
    srcs, params = [], []
    for _ in range(24):
        h, w = (int(v) for v in rng.integers(256, 513, 2))
        srcs.append(gradient_image(rng, h, w))
        params.append(random_params(rng, w, h, 224, 224, False))
    got = run_kernel(ctx, srcs, params, 224, 224, pixel_stride=pixel_stride)
    for i in range(len(srcs)):
        want = oracle(srcs[i], params[i], 224, 224)
        assert np.array_equal(got[i], want), "record %d differs" % i


def test_full_photometric_float_normalised(ctx):
    rng = np.random.default_rng(12)
    mean = [123.7 / 255, 116.3 / 255, 103.5 / 255]
    std = [58.4 / 255, 57.1 / 255, 57.4 / 255]
    srcs, params = [], []
    for _ in range(24):
        h, w = (int(v) for v in rng.integers(256, 513, 2))
        srcs.append(gradient_image(rng, h, w))
        params.append(random_params(rng, w, h, 224, 224, True))
    got = run_kernel(ctx, srcs, params, 224, 224, "float", True, True, mean, std)
    got_u8 = run_kernel(ctx, srcs, params, 224, 224, "uint8_t", False, False)
    for i in range(len(srcs)):
        want_u8 = ops.transform_single_image(srcs[i], params[i])
        assert np.array_equal(got_u8[i], want_u8), "uint8 photometric output of record %d differs" % i
        want = oracle(srcs[i], params[i], 224, 224, channel_major=True, bgr_to_rgb=True, output_type="float",
                      mean=mean, stddev=std)
        assert np.abs(got[i] - want).max() <= 1e-6


def test_each_photometric_stage_alone(ctx):
    rng = np.random.default_rng(13)
    src = rng.integers(0, 256, (97, 131, 3), dtype=np.uint8)  # full-range noise exercises saturation
    base = dict(cropbox=(0, 0, 131, 97), output_size=(131, 97))
    cases = [dict(brightness=1.4), dict(saturation=0.6), dict(brightness=0.7, saturation=1.3),
             dict(hue=-18), dict(hue=17), dict(hue=-1), dict(contrast=0.6), dict(contrast=1.4),
             dict(lighting=[0.2, -0.1, 0.05], color_noise_std=0.1), dict(flip=True, hue=5)]
    params = [ops.ImageParams(**base, **c) for c in cases]
    got = run_kernel(ctx, [src] * len(cases), params, 131, 97, "uint8_t", False)
    for i, p in enumerate(params):
        assert np.array_equal(got[i], ops.transform_single_image(src, p)), cases[i]


def test_hsv_round_trip_all_inputs(ctx):
    """Every 8-bit BGR triple through hue shifts, 4096 x 4096 pixels in 16 bands."""
    v = np.arange(256, dtype=np.uint8)
    b, g, r = np.meshgrid(v, v, v, indexing="ij")
    img = np.stack([b, g, r], -1).reshape(4096, 4096, 3)
    for hue in (-7, 11):
        for band in (0, 5, 15):
            src = np.ascontiguousarray(img[band * 256:(band + 1) * 256, :1000])
            p = ops.ImageParams(cropbox=(0, 0, 1000, 256), output_size=(1000, 256), hue=hue)
            got = run_kernel(ctx, [src], [p], 1000, 256, "uint8_t", False)[0]
            assert np.array_equal(got, ops.transform_single_image(src, p))


@pytest.mark.parametrize("shape", [(1, 1), (2, 3), (7, 5), (16, 16), (17, 17), (33, 9)])
def test_tiny_and_odd_sizes(ctx, shape):
    rng = np.random.default_rng(14)
    h, w = shape
    src = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    params = [ops.ImageParams(cropbox=(0, 0, w, h), output_size=(ow, oh), flip=f, contrast=c)
              for (ow, oh, f, c) in [(w, h, False, 1.0), (13, 11, True, 1.0), (31, 17, False, 0.8), (5, 40, True, 1.3)]]
    for p in params:
        ow, oh = p.output_size
        got = run_kernel(ctx, [src], [p], ow, oh, "uint8_t", False)[0]
        assert np.array_equal(got, ops.transform_single_image(src, p))


def test_crop_at_borders_and_upscale(ctx):
    rng = np.random.default_rng(15)
    src = gradient_image(rng, 90, 120)
    boxes = [(0, 0, 40, 30), (80, 0, 40, 30), (0, 60, 40, 30), (80, 60, 40, 30), (0, 0, 120, 90), (119, 89, 1, 1)]
    params = [ops.ImageParams(cropbox=b, output_size=(224, 224), flip=bool(i & 1)) for i, b in enumerate(boxes)]
    got = run_kernel(ctx, [src] * len(boxes), params, 224, 224)
    for i, p in enumerate(params):
        assert np.array_equal(got[i], oracle(src, p, 224, 224)), boxes[i]


def test_expand_canvas_and_padding(ctx):
    rng = np.random.default_rng(16)
    src = gradient_image(rng, 75, 100)
    p1 = ops.ImageParams(expand_ratio=2.0, expand_offset=(37, 21), expand_size=(200, 150), cropbox=(10, 5, 160, 130),
                         output_size=(300, 300), flip=True)
    p2 = ops.ImageParams(cropbox=(0, 0, 100, 75), output_size=(100, 75), padding=4, padding_crop_offset=(1, 7))
    got1 = run_kernel(ctx, [src], [p1], 300, 300, "float", True)[0]
    assert np.array_equal(got1, oracle(src, p1, 300, 300, output_type="float"))
    got2 = run_kernel(ctx, [src], [p2], 100, 75, "uint8_t", False)[0]
    assert np.array_equal(got2, ops.transform_single_image(src, p2))


def test_fixed_aspect_slot_zero_fill_and_null_source(ctx):
    rng = np.random.default_rng(17)
    src = gradient_image(rng, 60, 90)
    p = ops.ImageParams(cropbox=(0, 0, 90, 60), output_size=(48, 32))
    got = run_kernel(ctx, [src, None], [p, p], 64, 64, "uint8_t", True)
    assert np.array_equal(got[0], oracle(src, p, 64, 64))
    assert not got[1].any()
    mean, std = [0.4, 0.5, 0.6], [0.2, 0.0, 0.3]
    gotf = run_kernel(ctx, [src], [p], 64, 64, "float", True, False, mean, std)[0]
    want = oracle(src, p, 64, 64, channel_major=True, output_type="float", mean=mean, stddev=std)
    assert np.abs(gotf - want).max() <= 1e-6
    assert not gotf[:, 32:, :].any() and not gotf[:, :, 48:].any()


@pytest.mark.parametrize("otype", ["int8_t", "int16_t", "uint16_t", "int32_t", "double"])
def test_output_types_and_hwc(ctx, otype):
    rng = np.random.default_rng(18)
    src = gradient_image(rng, 64, 64)
    p = ops.ImageParams(cropbox=(3, 5, 50, 40), output_size=(30, 20), flip=True)
    for cm in (True, False):
        got = run_kernel(ctx, [src], [p], 30, 20, otype, cm, True)[0]
        want = ops.load_image(ops.transform_single_image(src, p), cm, True, otype)
        assert np.array_equal(got, want.astype(got.dtype))


def test_nearest_interpolation(ctx):
    rng = np.random.default_rng(19)
    src = gradient_image(rng, 70, 55)
    p = ops.ImageParams(cropbox=(2, 3, 50, 60), output_size=(33, 47), interpolation_method="NEAREST")
    got = run_kernel(ctx, [src], [p], 33, 47, "uint8_t", False)[0]
    assert np.array_equal(got, ops.transform_single_image(src, p))


def test_reference_golden_train_vector(ctx, golden_dir):
    """aeon test/test_provider.cpp:96-179: crop (50,50,171x201) + flip + 224 LINEAR + RGB CHW float standardise."""
    import cv2
    import os
    enc = np.fromfile(os.path.join(golden_dir, "img_2112_70.jpg"), np.uint8)
    img = cv2.imdecode(enc, cv2.IMREAD_COLOR)
    p = ops.ImageParams(cropbox=(50, 50, 171, 201), output_size=(224, 224), flip=True)
    got = run_kernel(ctx, [img], [p], 224, 224, "float", True, True, [0.485, 0.456, 0.406], [0.229, 0.224, 0.225])[0]
    gold = np.fromfile(os.path.join(golden_dir, "augment_output_linear_train.bin"), np.float32).reshape(3, 224, 224)
    assert np.abs(got - gold).max() <= 1e-5


def test_invalid_descriptors_are_rejected(ctx):
    from aeon_b200._lib import AeonError
    rng = np.random.default_rng(20)
    src = gradient_image(rng, 32, 32)
    bad = ops.ImageParams(cropbox=(10, 10, 30, 30), output_size=(16, 16))
    with pytest.raises(AeonError, match="outside"):
        run_kernel(ctx, [src], [bad], 16, 16)
    big = ops.ImageParams(cropbox=(0, 0, 32, 32), output_size=(40, 16))
    with pytest.raises(AeonError, match="does not fit"):
        run_kernel(ctx, [src], [big], 16, 16)
