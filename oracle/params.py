"""CPU oracle for aeon's seeded augmentation-parameter draws (TEST INFRASTRUCTURE ONLY).

Restates ``augment::image::param_factory::make_params`` (aeon src/augment_image.cpp:107-230),
the crop-box helpers it calls (src/image.cpp:214-273) and the per-slot engine seeding of
``batch_decoder`` (src/batch_decoder.cpp:47-54), together with the algorithms GNU libstdc++
uses for ``std::minstd_rand0`` and the ``<random>`` distributions the factory owns, so the
draws can be checked number for number against the shipped C++ code, which uses the real
``<random>`` classes.  aeon's only seeded end-to-end test is disabled
(test/test_loader.cpp:431), so the reference pins no seeded values: PARITY UNPINNED by the
reference for the drawn numbers; the draw ORDER and the arithmetic are what this restates.
Nothing in the shipped package imports this file.
"""
import math

import numpy as np

from .image_ops import ImageParams

f32 = np.float32
M = 2147483647

try:  # the C library's single-precision log, which std::log(float) resolves to
    import ctypes as _C
    _libm = _C.CDLL("libm.so.6")
    _libm.logf.restype = _C.c_float
    _libm.logf.argtypes = [_C.c_float]
    _logf = lambda v: f32(_libm.logf(float(v)))
except OSError:  # pragma: no cover
    _logf = lambda v: f32(math.log(float(v)))


class MinstdRand0:
    """x <- 16807 x mod (2^31 - 1); values in [1, 2^31 - 2]."""

    def __init__(self, seed=1):
        self.seed(seed)

    def seed(self, s):
        self.x = s % M or 1

    def __call__(self):
        self.x = (16807 * self.x) % M
        return self.x

    MIN = 1
    RANGE = 2147483646  # max - min + 1


def canonical_f32(g):
    """std::generate_canonical<float, 24>: one engine call, float division by float(range)."""
    s = f32(g() - g.MIN)
    r = s / f32(g.RANGE)
    return r if r < f32(1) else np.nextafter(f32(1), f32(0))


def canonical_f64(g):
    """std::generate_canonical<double, 53>: two engine calls."""
    s = float(g() - g.MIN)
    s += float(g() - g.MIN) * float(g.RANGE)
    r = s / (float(g.RANGE) * float(g.RANGE))
    return r if r < 1.0 else math.nextafter(1.0, 0.0)


def uniform_real_f32(g, a, b):
    a, b = f32(a), f32(b)
    return f32(f32(canonical_f32(g) * f32(b - a)) + a)


def uniform_int(g, a, b):
    """std::uniform_int_distribution<int> on an engine whose range exceeds the requested one."""
    urange = b - a
    urngrange = g.RANGE - 1
    uerange = urange + 1
    scaling = urngrange // uerange
    past = uerange * scaling
    while True:
        ret = g() - g.MIN
        if ret < past:
            break
    return a + ret // scaling


def bernoulli(g, p):
    return canonical_f64(g) < p


class NormalF32:
    """std::normal_distribution<float>: Marsaglia polar method keeping the second variate."""

    def __init__(self, mean, stddev):
        self.mean, self.stddev = f32(mean), f32(stddev)
        self.saved = None

    def __call__(self, g):
        if self.saved is not None:
            ret, self.saved = self.saved, None
        else:
            while True:
                x = f32(float(f32(2.0) * canonical_f32(g)) - 1.0)
                y = f32(float(f32(2.0) * canonical_f32(g)) - 1.0)
                r2 = f32(f32(x * x) + f32(y * y))
                if not (float(r2) > 1.0 or float(r2) == 0.0):
                    break
            lg = _logf(r2)
            mult = np.sqrt(f32(f32(f32(-2) * lg) / r2))
            self.saved = f32(x * mult)
            ret = f32(y * mult)
        return f32(f32(ret * self.stddev) + self.mean)


def slot_engines(seed, decode_size):
    master = MinstdRand0(seed)
    return [MinstdRand0(master()) for _ in range(decode_size)]


def cv_round(v):
    """OpenCV float->int conversion: nearest, ties to even."""
    return int(np.rint(f32(v)))


def unbiased_round(x):
    """aeon src/util.cpp:212-239 (half to even on the magnitude)."""
    x = float(f32(x))
    frac, whole = math.modf(x)
    if abs(frac) == 0.5:
        if int(whole) % 2 == 0:
            return int(whole)
        rc = int(abs(x) + 0.5)
    else:
        rc = int(math.floor(abs(x) + 0.5))
    return -rc if x < 0 else rc


class ParamFactory:
    """aeon param_factory for the keys that drive make_params (src/augment_image.hpp:141-246)."""

    def __init__(self, cfg=None):
        cfg = dict(cfg or {})
        g = cfg.get
        self.scale = tuple(g("scale", (1.0, 1.0)))
        self.angle = tuple(g("angle", (0, 0)))
        self.lighting = NormalF32(*g("lighting", (0.0, 0.0)))
        self.horizontal_distortion = tuple(g("horizontal_distortion", (1.0, 1.0)))
        self.contrast = tuple(g("contrast", (1.0, 1.0)))
        self.brightness = tuple(g("brightness", (1.0, 1.0)))
        self.saturation = tuple(g("saturation", (1.0, 1.0)))
        self.hue = tuple(g("hue", (0, 0)))
        self.flip_enable = g("flip_enable", False)
        self.center = g("center", True)
        self.do_area_scale = g("do_area_scale", False)
        self.crop_enable = g("crop_enable", True)
        self.resize_short_size = g("resize_short_size", 0)
        self.interpolation_method = g("interpolation_method", "LINEAR")
        self.fixed_scaling_factor = g("fixed_scaling_factor", -1)
        self.padding = g("padding", 0)
        self.crop_offset = (0.5, 0.5) if self.center else (0.0, 1.0)
        self.flip_p = 0.5 if self.flip_enable else 0.0
        self.pad_range = (0, self.padding * 2) if self.padding > 0 else (0, 0)

    def make_params(self, g, in_w, in_h, out_w, out_h):
        p = ImageParams(output_size=(out_w, out_h))
        # draw order of src/augment_image.cpp:119-124
        p.angle = uniform_int(g, *self.angle)
        p.flip = bernoulli(g, self.flip_p)
        p.hue = uniform_int(g, *self.hue)
        p.contrast = uniform_real_f32(g, *self.contrast)
        p.brightness = uniform_real_f32(g, *self.brightness)
        p.saturation = uniform_real_f32(g, *self.saturation)
        p.padding = self.padding
        p.resize_short_size = self.resize_short_size
        p.interpolation_method = self.interpolation_method
        fw, fh = f32(in_w), f32(in_h)
        if not self.crop_enable:
            ox = uniform_int(g, *self.pad_range)
            oy = uniform_int(g, *self.pad_range)
            p.padding_crop_offset = (ox, oy)
            p.cropbox = (0, 0, in_w, in_h)
            if self.fixed_scaling_factor > 0:
                s = f32(self.fixed_scaling_factor)
            else:
                s = f32(out_w) / fw
                if f32(fh * s) > out_h:
                    s = f32(out_h) / fh
            p.output_size = (unbiased_round(f32(fw * s)), unbiased_round(f32(fh * s)))
        elif self.do_area_scale:
            hd = np.sqrt(uniform_real_f32(g, *self.horizontal_distortion))
            ow, oh = hd, f32(f32(1) / hd)
            bound = min(f32(f32(fw / fh) / f32(ow * ow)), f32(f32(fh / fw) / f32(oh * oh)))
            smax = min(f32(self.scale[1]), bound)
            smin = min(f32(self.scale[0]), bound)
            area = np.sqrt(f32(f32(in_h * in_w) * uniform_real_f32(g, smin, smax)))
            ow, oh = f32(ow * area), f32(oh * area)
            cx = uniform_real_f32(g, *self.crop_offset)
            cy = uniform_real_f32(g, *self.crop_offset)
            x = int(f32(f32(fw - ow) * cx))
            y = int(f32(f32(fh - oh) * cy))
            p.cropbox = (x, y, cv_round(ow), cv_round(oh))
        else:
            s = uniform_real_f32(g, *self.scale)
            hd = uniform_real_f32(g, *self.horizontal_distortion)
            ow, oh = f32(f32(out_w) * hd), f32(out_h)
            if self.resize_short_size > 0:
                pct = f32(self.resize_short_size) / f32(min(in_h, in_w))
                fw = f32(int(math.floor(float(f32(f32(in_w) * pct)) + 0.5)))
                fh = f32(int(math.floor(float(f32(f32(in_h) * pct)) + 0.5)))
            sc = f32(fw / ow)
            cw, ch = f32(ow * sc), f32(oh * sc)
            if ch > fh:
                sc = f32(fh / ch)
                cw, ch = f32(cw * sc), f32(ch * sc)
            cw, ch = f32(cw * s), f32(ch * s)
            cx = uniform_real_f32(g, *self.crop_offset)
            cy = uniform_real_f32(g, *self.crop_offset)
            x = int(f32(f32(fw - cw) * cx))
            y = int(f32(f32(fh - ch) * cy))
            p.cropbox = (x, y, cv_round(cw), cv_round(ch))
        if self.lighting.stddev != 0:
            p.lighting = [self.lighting(g) for _ in range(3)]
            p.color_noise_std = float(self.lighting.stddev)
        return p
