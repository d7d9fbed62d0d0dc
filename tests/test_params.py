"""The seeded augmentation draws of the C++ host code (std::minstd_rand0 + <random>) against the
python restatement of libstdc++'s algorithms, number for number (no GPU needed)."""
import ctypes as C
import json

import numpy as np
import pytest

from oracle import params as op


def draw(aug, seed, decode, sizes, ow, oh):
    from aeon_b200 import _lib as L
    lib = L.load()
    n = len(sizes)
    w = (C.c_int32 * n)(*[s[0] for s in sizes])
    h = (C.c_int32 * n)(*[s[1] for s in sizes])
    out = (C.c_double * (24 * n))()
    L.check(lib.aeonb_draw_params(json.dumps(aug).encode(), seed, decode, n, w, h, ow, oh, out))
    return np.array(out).reshape(n, 24)


AUGS = [
    {"type": "image", "crop_enable": True, "center": False, "do_area_scale": True, "scale": [0.08, 1.0],
     "horizontal_distortion": [0.75, 1.3333334], "flip_enable": True},
    {"type": "image", "crop_enable": True, "center": False, "do_area_scale": True, "scale": [0.08, 1.0],
     "horizontal_distortion": [0.75, 1.3333334], "flip_enable": True, "contrast": [0.6, 1.4], "brightness": [0.6, 1.4],
     "saturation": [0.6, 1.4], "hue": [-18, 18], "lighting": [0.0, 0.1]},
    {"type": "image", "scale": [0.5, 0.9], "center": False, "flip_enable": True, "horizontal_distortion": [0.8, 1.2]},
    {"type": "image", "scale": [0.875, 0.875], "center": True},
    {"type": "image", "crop_enable": False, "padding": 4, "flip_enable": True},
    {"type": "image", "crop_enable": False, "fixed_aspect_ratio": True},
    {"type": "image", "scale": [0.3, 0.8], "resize_short_size": 256, "center": False},
]


@pytest.mark.parametrize("aug", AUGS)
def test_draws_match_libstdcxx_restatement(aug):
    rng = np.random.default_rng(0)
    sizes = [(int(a), int(b)) for a, b in rng.integers(256, 513, (300, 2))]
    got = draw(aug, 1234, 128, sizes, 224, 224)
    f = op.ParamFactory(aug)
    eng = op.slot_engines(1234, 128)
    for i, (w, h) in enumerate(sizes):
        p = f.make_params(eng[i % 128], w, h, 224, 224)
        want = [*p.cropbox, *p.output_size, float(p.flip), p.angle, p.hue, float(p.contrast), float(p.brightness),
                float(p.saturation)] + [float(v) for v in (list(p.lighting) + [0, 0, 0])[:3]] + \
               [float(np.float32(p.color_noise_std)), *p.padding_crop_offset]
        assert np.array_equal(np.array(want, np.float64), got[i, :18]), i


def test_engine_constants():
    g = op.MinstdRand0(1)
    for _ in range(9999):
        g()
    assert g() == 1043618065   # the 10000th value of minstd_rand0 seeded with 1 (C++ standard, [rand.predef])


def test_crop_boxes_stay_inside_the_image():
    rng = np.random.default_rng(1)
    sizes = [(int(a), int(b)) for a, b in rng.integers(32, 2000, (2000, 2))]
    got = draw(AUGS[0], 77, 64, sizes, 224, 224)
    for (w, h), r in zip(sizes, got):
        x, y, cw, ch = r[:4]
        assert x >= 0 and y >= 0 and cw >= 1 and ch >= 1 and x + cw <= w and y + ch <= h


def test_invalid_augmentation_is_rejected():
    from aeon_b200._lib import AeonError
    with pytest.raises(AeonError, match="out of range"):
        draw({"type": "image", "scale": [0.9, 0.5]}, 1, 1, [(10, 10)], 4, 4)
    with pytest.raises(AeonError, match="missing 'type'"):
        draw({"scale": [0.5, 0.9]}, 1, 1, [(10, 10)], 4, 4)
    with pytest.raises(AeonError, match="batch_samplers"):
        draw({"type": "image", "crop_enable": True, "batch_samplers": [{}]}, 1, 1, [(10, 10)], 4, 4)


def test_ssd_draws_and_patch_sampling_match_restatement():
    """make_ssd_params (expand, patch samplers with IoU constraints) against oracle/ssd.py, value for value."""
    from aeon_b200 import _lib as L
    from oracle import ssd
    lib = L.load()
    samplers = [{"max_sample": 1, "max_trials": 1}] + [
        {"max_sample": 1, "max_trials": 50, "sampler": {"scale": [0.3, 1.0], "aspect_ratio": [0.5, 2.0]}, "sample_constraint": c}
        for c in ({"min_jaccard_overlap": 0.1}, {"min_jaccard_overlap": 0.5}, {"min_jaccard_overlap": 0.9},
                  {"max_jaccard_overlap": 1.0}, {"min_sample_coverage": 0.3, "max_object_coverage": 0.9})]
    aug = {"type": "image", "crop_enable": False, "flip_enable": True, "expand_ratio": [1.0, 4.0], "expand_probability": 0.5,
           "emit_constraint_type": "center", "batch_samplers": samplers}
    rng = np.random.default_rng(0)
    n, W, H = 200, 500, 375
    boxes, counts = [], []
    for _ in range(n):
        k = int(rng.integers(1, 9))
        counts.append(k)
        for _ in range(k):
            x0, y0 = int(rng.integers(0, W - 9)), int(rng.integers(0, H - 9))
            boxes.append((x0, y0, int(rng.integers(x0 + 8, W)), int(rng.integers(y0 + 8, H))))
    flat = np.array(boxes, np.float32).ravel()
    out = (C.c_double * (24 * n))()
    w = (C.c_int32 * n)(*[W] * n)
    h = (C.c_int32 * n)(*[H] * n)
    cnt = (C.c_int32 * n)(*counts)
    L.check(lib.aeonb_draw_ssd_params(json.dumps(aug).encode(), 1234, 32, n, w, h, 300, 300, cnt,
                                      flat.ctypes.data_as(C.POINTER(C.c_float)), out))
    got = np.array(out).reshape(n, 24)
    f = ssd.SsdFactory(aug)
    eng = op.slot_engines(1234, 32)
    at = 0
    for i in range(n):
        bb = [ssd.Box(*boxes[at + j]) for j in range(counts[i])]
        at += counts[i]
        p = f.make_ssd_params(eng[i % 32], W, H, 300, 300, bb)
        want = [*p.cropbox, *p.output_size, float(p.flip), p.angle, p.hue, float(p.contrast), float(p.brightness),
                float(p.saturation), 0, 0, 0, 0, *p.padding_crop_offset, float(np.float32(p.expand_ratio)),
                *p.expand_offset, *p.expand_size]
        assert np.array_equal(np.array(want, np.float64), got[i, :23]), i
    assert 60 < (got[:, 18] > 1).sum() < 140


def test_reference_validation_recipe_draws_the_centre_crop():
    """aeon test/test_provider.cpp:202-221 with the 480x360 fixture: resize_short 256 -> 341x256, scale 224/256,
    centred: the crop box the golden vector augment_output_linear_eval.bin was made with is (58, 16, 224, 224)."""
    aug = {"type": "image", "flip_enable": False, "center": True, "crop_enable": True, "scale": [224 / 256, 224 / 256],
           "resize_short_size": 256}
    got = draw(aug, 1, 1, [(480, 360)], 224, 224)[0]
    assert got[:6].tolist() == [58, 16, 224, 224, 224, 224]
