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
