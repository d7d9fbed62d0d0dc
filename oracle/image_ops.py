"""CPU oracle for aeon's per-record image ETL arithmetic (TEST INFRASTRUCTURE ONLY).

This module is a checker.  Nothing in the shipped package imports it; only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark do.

aeon delegates every pixel operation to OpenCV (un-vendored, version unpinned by
the reference's CMake: ``find_package(OpenCV REQUIRED)``).  The functions below
restate, in numpy integer / float32 arithmetic, what OpenCV 4.13 computes for the
exact call sequence aeon makes.  Each one names the aeon call site it follows
(paths are relative to the aeon source tree) and is pinned in the CPU test-suite
against the OpenCV binary itself (python ``cv2`` 4.13.0, exhaustively where the
domain is small) and against aeon's own golden vectors
(``test/test_data/augment_output_linear_{train,eval}.bin``).

Array conventions: images are ``uint8`` ``H x W x 3`` in BGR order, exactly as
``cv::imdecode`` hands them to aeon.
"""
import numpy as np

f32 = np.float32
f64 = np.float64

# ---------------------------------------------------------------------------------------------
# small helpers
# ---------------------------------------------------------------------------------------------


def _rne(x):
    """Round half to even (OpenCV ``cvRound`` / ``saturate_cast`` from floating point)."""
    return np.rint(x)


def _sat_u8(x):
    return np.clip(x, 0, 255).astype(np.uint8)


def _fnmadd32(a, b, c):
    """Single-rounding float32 ``c - a*b`` (what an FMA instruction returns)."""
    return (np.asarray(c, f64) - np.asarray(a, f64) * np.asarray(b, f64)).astype(f32)


# ---------------------------------------------------------------------------------------------
# geometry: cv::resize(INTER_LINEAR) on 8-bit data   (aeon: src/image.cpp:93-106 -> cv::resize)
# ---------------------------------------------------------------------------------------------

RESIZE_COEF_BITS = 11
RESIZE_COEF_ONE = 1 << RESIZE_COEF_BITS


def linear_taps(src_len, dst_len, clamp_weights):
    """Source index and 11-bit fixed-point tap pair for every destination index.

    ``clamp_weights`` is True for the horizontal axis, where OpenCV moves a tap that
    falls outside the row onto the border pixel and gives it the whole weight; on
    the vertical axis only the row index is clamped and the weights are kept.
    """
    scale = f64(src_len) / f64(dst_len)
    d = np.arange(dst_len, dtype=f64)
    f = ((d + 0.5) * scale - 0.5).astype(f32)
    s = np.floor(f).astype(np.int32)
    f = f - s.astype(f32)
    if clamp_weights:
        lo = s < 0
        f = np.where(lo, f32(0), f)
        s = np.where(lo, 0, s)
        hi = s >= src_len - 1
        f = np.where(hi, f32(0), f)
        s = np.where(hi, src_len - 1, s)
    w0 = np.clip(_rne((f32(1) - f) * f32(RESIZE_COEF_ONE)), -32768, 32767).astype(np.int32)
    w1 = np.clip(_rne(f * f32(RESIZE_COEF_ONE)), -32768, 32767).astype(np.int32)
    return s, w0, w1


def resize_linear_u8(src, out_w, out_h):
    """Bit-exact ``cv::resize(src, dst, Size(out_w,out_h), 0, 0, INTER_LINEAR)`` for uint8.

    aeon skips the call when the size is unchanged (src/image.cpp:97-100); the
    arithmetic below degenerates to a copy in that case, so no special case is needed.
    """
    h, w = src.shape[:2]
    sx, a0, a1 = linear_taps(w, out_w, True)
    sy, b0, b1 = linear_taps(h, out_h, False)
    sx1 = np.minimum(sx + 1, w - 1)
    y0 = np.clip(sy, 0, h - 1)
    y1 = np.clip(sy + 1, 0, h - 1)
    s = src.astype(np.int32)
    # horizontal pass keeps 11 fractional bits
    hor = s[:, sx, :] * a0[None, :, None] + s[:, sx1, :] * a1[None, :, None]
    r0 = hor[y0] >> 4
    r1 = hor[y1] >> 4
    out = (((b0[:, None, None] * r0) >> 16) + ((b1[:, None, None] * r1) >> 16) + 2) >> 2
    return _sat_u8(out)


def _area_table(src_len, dst_len, scale):
    """``computeResizeAreaTab``: (destination index, source index, float32 weight) in OpenCV's order."""
    tab = []
    for d in range(dst_len):
        f1 = d * scale
        f2 = f1 + scale
        cell = min(scale, src_len - f1)
        s1, s2 = int(np.ceil(f1)), int(np.floor(f2))
        s2 = min(s2, src_len - 1)
        s1 = min(s1, s2)
        if s1 - f1 > 1e-3:
            tab.append((d, s1 - 1, f32((s1 - f1) / cell)))
        for sidx in range(s1, s2):
            tab.append((d, sidx, f32(1.0 / cell)))
        if f2 - s2 > 1e-3:
            tab.append((d, s2, f32(min(min(f2 - s2, 1.0), cell) / cell)))
    return tab


def _area_linear_taps(src_len, dst_len, scale, inv_scale):
    """Tap positions of ``cv::resize`` when INTER_AREA enlarges (it then interpolates linearly from these)."""
    d = np.arange(dst_len, dtype=f64)
    s = np.floor(d * scale).astype(np.int64)
    f = ((d + 1) - (s + 1) * inv_scale).astype(f32)
    f = np.where(f <= 0, f32(0), f - np.floor(f)).astype(f32)
    lo = s < 0
    f = np.where(lo, f32(0), f)
    s = np.where(lo, 0, s)
    hi = s >= src_len - 1
    f = np.where(hi, f32(0), f)
    s = np.where(hi, src_len - 1, s)
    w0 = np.clip(_rne((f32(1) - f) * f32(RESIZE_COEF_ONE)), -32768, 32767).astype(np.int32)
    w1 = np.clip(_rne(f * f32(RESIZE_COEF_ONE)), -32768, 32767).astype(np.int32)
    return s, w0, w1


def resize_area_u8(src, out_w, out_h):
    """Bit-exact ``cv::resize(src, dst, Size(out_w,out_h), 0, 0, INTER_AREA)`` for uint8 (OpenCV 4.13).

    Three regimes: both axes shrink by whole factors -> box sums, 2x2 rounded as (sum + 2) >> 2, others as
    round-half-even(sum * float(1/area)); both axes shrink -> float32 weights, rows summed across first and then
    accumulated down, rounded half to even; otherwise -> the fixed-point linear interpolation with INTER_AREA's own
    tap positions.  The scale is 1/(dst/src) in float64, as OpenCV computes it."""
    h, w = src.shape[:2]
    inv_x, inv_y = f64(out_w) / f64(w), f64(out_h) / f64(h)
    scale_x, scale_y = 1.0 / inv_x, 1.0 / inv_y
    eps = np.finfo(np.float64).eps
    if scale_x >= 1 and scale_y >= 1:
        ix, iy = int(np.rint(scale_x)), int(np.rint(scale_y))
        if abs(scale_x - ix) < eps and abs(scale_y - iy) < eps:
            s = src[:out_h * iy, :out_w * ix].astype(np.int64).reshape(out_h, iy, out_w, ix, -1).sum(axis=(1, 3))
            if ix == 2 and iy == 2:
                return ((s + 2) >> 2).astype(np.uint8)
            return _sat_u8(_rne(s.astype(f32) * (f32(1.0) / f32(ix * iy))))
        xtab, ytab = _area_table(w, out_w, scale_x), _area_table(h, out_h, scale_y)
        srcf = src.astype(f32)
        out = np.zeros((out_h, out_w, src.shape[2]), np.uint8)
        dxs = np.array([t[0] for t in xtab])
        sxs = np.array([t[1] for t in xtab])
        als = np.array([t[2] for t in xtab], f32)
        acc, prev = None, ytab[0][0]
        for dy, sy, beta in ytab:
            buf = np.zeros((out_w, src.shape[2]), f32)
            row = srcf[sy]
            for k in range(len(xtab)):       # sequential: float32 sums in OpenCV's order
                buf[dxs[k]] = buf[dxs[k]] + row[sxs[k]] * als[k]
            if acc is None:
                acc = beta * buf
            elif dy != prev:
                out[prev] = _sat_u8(_rne(acc))
                acc = beta * buf
            else:
                acc = acc + beta * buf
            prev = dy
        out[prev] = _sat_u8(_rne(acc))
        return out
    sx, a0, a1 = _area_linear_taps(w, out_w, scale_x, inv_x)
    sy, b0, b1 = _area_linear_taps(h, out_h, scale_y, inv_y)
    sx1 = np.minimum(sx + 1, w - 1)
    y1 = np.minimum(sy + 1, h - 1)
    s = src.astype(np.int64)
    hor = s[:, sx, :] * a0[None, :, None] + s[:, sx1, :] * a1[None, :, None]
    out = (((b0[:, None, None] * (hor[sy] >> 4)) >> 16) + ((b1[:, None, None] * (hor[y1] >> 4)) >> 16) + 2) >> 2
    return _sat_u8(out)


def _cubic_taps(src_len, dst_len):
    """Tap indices (edge repeated) and 11-bit weights of ``cv::resize`` INTER_CUBIC: ``interpolateCubic`` with A = -0.75
    evaluated in float32 in OpenCV's order."""
    scale = 1.0 / (f64(dst_len) / f64(src_len))
    d = np.arange(dst_len, dtype=f64)
    f = ((d + 0.5) * scale - 0.5).astype(f32)
    s = np.floor(f).astype(np.int64)
    x = (f - s.astype(f32)).astype(f32)
    A, one = f32(-0.75), f32(1)
    x1, xm = x + one, one - x
    c0 = ((A * x1 - f32(5) * A) * x1 + f32(8) * A) * x1 - f32(4) * A
    c1 = ((A + f32(2)) * x - (A + f32(3))) * x * x + one
    c2 = ((A + f32(2)) * xm - (A + f32(3))) * xm * xm + one
    c3 = one - c0 - c1 - c2
    w = np.stack([np.clip(_rne(c * f32(RESIZE_COEF_ONE)), -32768, 32767).astype(np.int64) for c in (c0, c1, c2, c3)], 1)
    idx = np.clip(s[:, None] - 1 + np.arange(4)[None, :], 0, src_len - 1)
    return idx, w


CUBIC_VECTOR_BLOCK = 8   # int16 lanes of the 128-bit vector loop in OpenCV's vertical cubic pass


def resize_cubic_u8(src, out_w, out_h, vector_block=CUBIC_VECTOR_BLOCK):
    """``cv::resize(..., INTER_CUBIC)`` for uint8 as OpenCV's own code computes it: integer 4-tap horizontal pass; the
    vertical pass runs over the interleaved row (out_w * channels values), its first ``floor(n / 8) * 8`` values in
    float32 -- sum of value * (weight / 2^22), rounded half to even -- and the rest in integers as (sum + 2^21) >> 22.
    A cv2 built with Intel IPP hands 8-bit cubic resizes to IPP, which differs by one level in a few percent of the
    pixels: compare with ``cv2.ipp.setUseIPP(False)``."""
    h, w = src.shape[:2]
    ix, wx = _cubic_taps(w, out_w)
    iy, wy = _cubic_taps(h, out_h)
    s = src.astype(np.int64)
    hor = sum(s[:, ix[:, k], :] * wx[None, :, k, None] for k in range(4))
    rows = [hor[iy[:, k]].reshape(out_h, -1) for k in range(4)]              # out_h x (out_w * channels)
    fixed = (sum(rows[k] * wy[:, k, None] for k in range(4)) + (1 << 21)) >> 22
    scale = f32(1.0) / f32(RESIZE_COEF_ONE * RESIZE_COEF_ONE)
    b = [(wy[:, k].astype(f32) * scale).astype(f32)[:, None] for k in range(4)]
    t = rows[3].astype(f32) * b[3]
    for k in (2, 1, 0):
        t = (rows[k].astype(f32) * b[k]).astype(f32) + t
    n = fixed.shape[1]
    body = n - n % vector_block if vector_block else 0
    out = np.where(np.arange(n)[None, :] < body, _rne(t).astype(np.int64), fixed)
    return _sat_u8(out).reshape(out_h, out_w, src.shape[2])


def _lanczos4_taps(src_len, dst_len):
    """Tap indices (edge repeated) and 11-bit weights of ``cv::resize`` INTER_LANCZOS4 (``interpolateLanczos4``: weights
    from double-precision sines / cosines of the C library, normalised in float32)."""
    import math
    s45 = 0.70710678118654752440084436210485
    cs = [(1, 0), (-s45, -s45), (0, 1), (s45, -s45), (-1, 0), (s45, s45), (0, -1), (-s45, s45)]
    scale = 1.0 / (f64(dst_len) / f64(src_len))
    idx = np.zeros((dst_len, 8), np.int64)
    w = np.zeros((dst_len, 8), np.int64)
    for d in range(dst_len):
        x = f32((d + 0.5) * scale - 0.5)
        s = int(np.floor(x))
        x = f32(x - f32(s))
        if x < np.finfo(np.float32).eps:
            c = [f32(0)] * 8
            c[3] = f32(1)
        else:
            y0 = -(float(x) + 3) * math.pi * 0.25
            s0, c0 = math.sin(y0), math.cos(y0)
            c, total = [], f32(0)
            for i in range(8):
                y = -(float(x) + 3 - i) * math.pi * 0.25
                c.append(f32((cs[i][0] * s0 + cs[i][1] * c0) / (y * y)))
                total = f32(total + c[-1])
            total = f32(f32(1) / total)
            c = [f32(ci * total) for ci in c]
        w[d] = [int(np.clip(_rne(ci * f32(RESIZE_COEF_ONE)), -32768, 32767)) for ci in c]
        idx[d] = np.clip(s - 3 + np.arange(8), 0, src_len - 1)
    return idx, w


def resize_lanczos4_u8(src, out_w, out_h):
    """``cv::resize(..., INTER_LANCZOS4)`` for uint8: integer 8-tap passes, the vertical one rounded as (sum + 2^21) >> 22."""
    h, w = src.shape[:2]
    ix, wx = _lanczos4_taps(w, out_w)
    iy, wy = _lanczos4_taps(h, out_h)
    s = src.astype(np.int64)
    hor = sum(s[:, ix[:, k], :] * wx[None, :, k, None] for k in range(8))
    ver = sum(hor[iy[:, k]] * wy[:, k, None, None] for k in range(8))
    return _sat_u8((ver + (1 << 21)) >> 22)


def resize_nearest_u8(src, out_w, out_h):
    """``cv::resize(..., INTER_NEAREST)``: source index = min(floor(d * (1 / (dst/src))), src-1), the factor formed in
    float64 as the reciprocal of dst/src (forming src/dst directly differs in the last place for about one size
    pair in twenty, which moves a tap where d * src/dst is a whole number)."""
    h, w = src.shape[:2]
    ix = np.minimum(np.floor(np.arange(out_w) * (f64(1.0) / (f64(out_w) / f64(w)))).astype(np.int64), w - 1)
    iy = np.minimum(np.floor(np.arange(out_h) * (f64(1.0) / (f64(out_h) / f64(h)))).astype(np.int64), h - 1)
    return src[iy][:, ix]


def expand(src, offset_xy, out_size_wh):
    """aeon ``image::expand`` (src/image.cpp:276-303): zero canvas with the image pasted in."""
    h, w = src.shape[:2]
    ox, oy = offset_xy
    ow, oh = out_size_wh
    if w + ox > ow or h + oy > oh or ox * oy < 0 or w * h <= 0:
        raise ValueError("Invalid parameters to expand image")
    if (ow, oh) == (w, h):
        return src
    out = np.zeros((oh, ow) + src.shape[2:], src.dtype)
    out[oy:oy + h, ox:ox + w] = src
    return out


# ---------------------------------------------------------------------------------------------
# photometric: aeon photometric::cbsjitter (src/image.cpp:358-406)
# ---------------------------------------------------------------------------------------------

GRAY_BGR = (0.0820, 0.6094, 0.3086)  # src/image.cpp:367


def color_matrix(brightness, saturation):
    """3x3 float32 matrix ``b*(s*I + (1-s)*1*g^T)`` of src/image.cpp:367-371 (BGR order)."""
    b = f32(brightness)
    s = f32(saturation)
    g = np.array(GRAY_BGR, f32)
    oms = f32(f32(1) - s)
    gray = (f64(oms) * g.astype(f64)).astype(f32)          # (1-s)*ones*g^T, gemm accumulates in double
    sb = f32(f64(s) * f64(b))
    m = np.zeros((3, 3), f32)
    for i in range(3):
        for j in range(3):
            m[i, j] = f32(f32(sb if i == j else 0) + f32(gray[j] * b))
    return m


TRANSFORM_BITS = 10


def is_diagonal(m):
    """cv::transform's test: every off-diagonal entry is at most FLT_EPSILON in magnitude."""
    m = np.asarray(m, f32)
    off = np.abs(m[~np.eye(3, dtype=bool)])
    return bool(np.all(off.astype(f64) <= np.finfo(f32).eps))


def transform_u8(img, m):
    """``cv::transform`` of an 8-bit 3-channel image by a 3x3 float matrix.

    OpenCV evaluates the dense case in 10-bit fixed point: coefficients are
    ``round_half_even(m*1024)`` saturated to int16, the dot product is rounded with
    ``+512 >> 10`` and saturated to uint8 (src/image.cpp:372 -> cv::transform).
    """
    m = np.asarray(m, f32)
    if is_diagonal(m):
        # OpenCV routes a diagonal matrix (brightness alone) to a per-channel float scale instead
        d = np.array([m[0, 0], m[1, 1], m[2, 2]], f32)
        return _sat_u8(_rne(img.astype(f32) * d[None, None, :]))
    mi = np.clip(_rne(m * f32(1 << TRANSFORM_BITS)), -32768, 32767).astype(np.int32)
    s = img.astype(np.int32)
    out = np.empty(img.shape, np.int32)
    for k in range(3):
        out[..., k] = (s[..., 0] * mi[k, 0] + s[..., 1] * mi[k, 1] + s[..., 2] * mi[k, 2]
                       + (1 << (TRANSFORM_BITS - 1))) >> TRANSFORM_BITS
    return _sat_u8(out)


HSV_SHIFT = 12


def _hsv_tables():
    sdiv = np.zeros(256, np.int32)
    hdiv = np.zeros(256, np.int32)
    i = np.arange(1, 256, dtype=f64)
    sdiv[1:] = _rne((255 << HSV_SHIFT) / i).astype(np.int32)
    hdiv[1:] = _rne((180 << HSV_SHIFT) / (6.0 * i)).astype(np.int32)
    return sdiv, hdiv


_SDIV, _HDIV180 = _hsv_tables()


def bgr2hsv_u8(img):
    """8-bit ``cv::cvtColor(BGR2HSV)`` with H in [0,180): reciprocal tables, 12-bit fixed point."""
    b = img[..., 0].astype(np.int32)
    g = img[..., 1].astype(np.int32)
    r = img[..., 2].astype(np.int32)
    v = np.maximum(np.maximum(b, g), r)
    diff = v - np.minimum(np.minimum(b, g), r)
    half = 1 << (HSV_SHIFT - 1)
    s = (diff * _SDIV[v] + half) >> HSV_SHIFT
    h = np.where(v == r, g - b, np.where(v == g, b - r + 2 * diff, r - g + 4 * diff))
    h = (h * _HDIV180[diff] + half) >> HSV_SHIFT
    h = np.where(h < 0, h + 180, h)
    return np.stack([h, s, v], -1).astype(np.uint8)


_SECTOR = np.array([[1, 3, 0], [1, 0, 2], [3, 0, 1], [0, 2, 1], [0, 1, 3], [2, 1, 0]])


HSV_VECTOR_BLOCK = 32   # pixels per vector iteration of OpenCV's AVX2 HSV->BGR row kernel


def hsv2bgr_u8(hsv, vector_block=HSV_VECTOR_BLOCK):
    """8-bit ``cv::cvtColor(HSV2BGR)`` for H scaled by 180.

    Float32 sector interpolation; the two interpolated corners use a fused
    multiply-add.  OpenCV converts each row in vector blocks of ``vector_block``
    pixels whose final ``*255`` is TRUNCATED, and finishes the row (the last
    ``W mod vector_block`` pixels) in scalar code that ROUNDS half-to-even; both
    behaviours are reproduced because aeon's output inherits them.  H values of
    180..255 (which aeon's hue wrap produces for negative sums) land in sector
    ``floor(h/30) mod 6``.  Checked over all 2^24 inputs in both modes.
    """
    h = hsv[..., 0].astype(f32) * f32(6.0 / 180.0)
    s = hsv[..., 1].astype(f32) * f32(1.0 / 255.0)
    v = hsv[..., 2].astype(f32) * f32(1.0 / 255.0)
    sector = np.floor(h).astype(np.int32)
    f = h - sector.astype(f32)
    sector = sector % 6
    one = np.ones_like(s)
    tab = np.stack([v, v * (f32(1) - s), v * _fnmadd32(s, f, one), v * _fnmadd32(s, f32(1) - f, one)], 0)
    idx = _SECTOR[sector]
    out = np.stack([np.take_along_axis(tab, idx[..., k][None], 0)[0] for k in range(3)], -1)
    out = out * f32(255)
    width = hsv.shape[-2]
    body = (width // vector_block) * vector_block if vector_block else 0
    res = _rne(out)
    if body:
        res[..., :body, :] = np.trunc(out[..., :body, :])
    return _sat_u8(res.astype(np.int32))


def hue_shift_u8(img, hue):
    """src/image.cpp:376-394: BGR->HSV, ``H = uint8((H + hue) % 180)`` with C remainder, HSV->BGR."""
    hsv = bgr2hsv_u8(img)
    t = hsv[..., 0].astype(np.int32) + int(hue)
    rem = np.fmod(t, 180).astype(np.int32)            # C '%': sign follows the dividend
    hsv[..., 0] = (rem & 0xFF).astype(np.uint8)       # stored back through a uint8_t*
    return hsv2bgr_u8(hsv)


def channel_sums(img):
    return img.reshape(-1, img.shape[-1]).astype(np.int64).sum(0)


def contrast_u8(img, contrast):
    """src/image.cpp:396-405: ``float(x)*c + float((1-c)*mean_channel)`` -> round-half-even uint8."""
    c = f32(contrast)
    mean = channel_sums(img).astype(f64) / f64(img.shape[0] * img.shape[1])
    add = ((1.0 - f64(c)) * mean).astype(f32)
    return _sat_u8(_rne(img.astype(f32) * c + add))


def cbsjitter(img, contrast, brightness, saturation, hue):
    if img.shape[2] != 3 and (f32(brightness) != 1.0 or f32(saturation) != 1.0 or int(hue) != 0):
        # cv::transform with a 3x3 matrix and cv::cvtColor(BGR2HSV) reject a one-channel picture
        raise ValueError("brightness, saturation and hue need a 3-channel picture")
    if f32(brightness) != 1.0 or f32(saturation) != 1.0:
        img = transform_u8(img, color_matrix(brightness, saturation))
    if int(hue) != 0:
        img = hue_shift_u8(img, hue)
    if f32(contrast) != 1.0:
        img = contrast_u8(img, contrast)
    return img


# src/image.cpp:320-324
CPCA = np.array([[0.39731118, 0.70119634, -0.59200296],
                 [-0.81698062, -0.02354167, -0.57618440],
                 [0.41795513, -0.71257945, -0.56351045]], f32)
CSTD = np.array([19.72083305, 37.09388853, 121.78006099], f32)


def lighting_pixel(alphas):
    """The colour-noise pixel ``CPCA * (CSTD o alpha)`` of src/image.cpp:341 (float32, BGR order)."""
    t = (CSTD * np.asarray(alphas, f32)).astype(f32)
    return (CPCA.astype(f64) @ t.astype(f64)).astype(f32)


def lighting_terms(alphas, color_noise_std):
    """(scale, integer offsets) that ``(img + pixel) / (1 + std)`` applies to a uint8 image.

    The cv::MatExpr is evaluated as ``convertTo(uint8, alpha)`` followed by a saturating
    add of the scalar ``pixel*alpha``, which OpenCV rounds to integers for 8-bit data.
    No reference test fixes this choice (parity unpinned; the alternatives differ by 1 LSB).
    """
    alpha = 1.0 / (1.0 + f64(f32(color_noise_std)))
    pix = lighting_pixel(alphas).astype(f64) * alpha
    return f32(alpha), _rne(pix).astype(np.int32)


def lighting_u8(img, alphas, color_noise_std):
    if alphas is None or len(alphas) == 0:
        return img
    scale, offs = lighting_terms(alphas, color_noise_std)
    t = _sat_u8(_rne(img.astype(f32) * scale)).astype(np.int32)
    return _sat_u8(t + offs[None, None, :img.shape[2]])   # a one-channel picture takes the first element of the pixel


# ---------------------------------------------------------------------------------------------
# transformer / loader (aeon src/etl_image.cpp:146-202 and :246-341)
# ---------------------------------------------------------------------------------------------


class ImageParams:
    """Field-for-field stand-in for aeon's ``augment::image::params`` (src/augment_image.hpp:69-123)."""

    def __init__(self, **kw):
        self.expand_ratio = 1.0
        self.expand_offset = (0, 0)
        self.expand_size = (0, 0)
        self.cropbox = (0, 0, 0, 0)           # x, y, w, h
        self.output_size = (0, 0)             # w, h
        self.angle = 0
        self.flip = False
        self.padding = 0
        self.padding_crop_offset = (0, 0)
        self.resize_short_size = 0
        self.interpolation_method = "LINEAR"
        self.lighting = []
        self.color_noise_std = 0.0
        self.contrast = 1.0
        self.brightness = 1.0
        self.saturation = 1.0
        self.hue = 0
        self.emit_type = ""                   # emit_constraint_type: only make_ssd_params sets it
        self.emit_min_overlap = 0.0
        for k, v in kw.items():
            if not hasattr(self, k):
                raise AttributeError(k)
            setattr(self, k, v)


def resized_short_size(w, h, target):
    """src/image.cpp:108-116 (float percent, round half away from zero)."""
    pct = f32(target) / f32(min(h, w))
    rw = int(np.floor(f64(f32(w) * pct) + 0.5))
    rh = int(np.floor(f64(f32(h) * pct) + 0.5))
    return rw, rh


def _resize(img, size_wh, method):
    if (img.shape[1], img.shape[0]) == tuple(size_wh):
        return img
    m = method.upper()
    if m == "LINEAR":
        return resize_linear_u8(img, size_wh[0], size_wh[1])
    if m == "NEAREST":
        return resize_nearest_u8(img, size_wh[0], size_wh[1])
    if m == "AREA":
        return resize_area_u8(img, size_wh[0], size_wh[1])
    if m == "CUBIC":
        return resize_cubic_u8(img, size_wh[0], size_wh[1])
    if m == "LANCZOS4":
        return resize_lanczos4_u8(img, size_wh[0], size_wh[1])
    raise NotImplementedError("interpolation method %s has no oracle" % method)


def rotation_matrix(width, height, angle):
    """``cv::getRotationMatrix2D(Point2i(cols/2, rows/2), angle, 1.0)`` as aeon's ``image::rotate`` calls it
    (src/image.cpp:62-63): 2x3 float64, angle in degrees, counter-clockwise."""
    import math
    cx, cy = float(width // 2), float(height // 2)
    a = angle * (math.pi / 180.0)
    alpha, beta = math.cos(a), math.sin(a)
    return np.array([[alpha, beta, (1 - alpha) * cx - beta * cy], [-beta, alpha, beta * cx + (1 - alpha) * cy]], np.float64)


def invert_affine(m):
    """The inversion ``cv::warpAffine`` applies to the forward matrix (no WARP_INVERSE_MAP), same operation order."""
    M = np.array(m, np.float64).ravel().copy()
    D = M[0] * M[4] - M[1] * M[3]
    D = 1.0 / D if D != 0 else 0.0
    A11, A22 = M[4] * D, M[0] * D
    M[0] = A11
    M[1] *= -D
    M[3] *= -D
    M[4] = A22
    b1 = -M[0] * M[2] - M[1] * M[5]
    b2 = -M[3] * M[2] - M[4] * M[5]
    M[2], M[5] = b1, b2
    return M


def warp_affine_linear_u8(src, forward):
    """``cv::warpAffine(src, dst, M, src.size(), INTER_LINEAR, BORDER_CONSTANT, 0)`` for 8-bit images: source
    coordinates in 10-bit fixed point (rounded half to even from float64), reduced to 5 fractional bits, bilinear
    weights (32-fx)(32-fy)*32 ... summing to 2^15, result (sum + 2^14) >> 15; taps outside the picture are zero."""
    h, w = src.shape[:2]
    M = invert_affine(forward)
    ab = 1024.0
    xs = np.arange(w, dtype=np.float64)
    ys = np.arange(h, dtype=np.float64)
    adelta = np.rint(M[0] * xs * ab).astype(np.int64)
    bdelta = np.rint(M[3] * xs * ab).astype(np.int64)
    x0 = np.rint((M[1] * ys + M[2]) * ab).astype(np.int64) + 16
    y0 = np.rint((M[4] * ys + M[5]) * ab).astype(np.int64) + 16
    X = (x0[:, None] + adelta[None, :]) >> 5
    Y = (y0[:, None] + bdelta[None, :]) >> 5
    sx, sy, fx, fy = X >> 5, Y >> 5, X & 31, Y & 31
    s = src.astype(np.int64)

    def tap(yy, xx):
        ok = (xx >= 0) & (xx < w) & (yy >= 0) & (yy < h)
        return s[np.clip(yy, 0, h - 1), np.clip(xx, 0, w - 1)] * ok[..., None]

    acc = (tap(sy, sx) * ((32 - fx) * (32 - fy) * 32)[..., None] + tap(sy, sx + 1) * (fx * (32 - fy) * 32)[..., None] +
           tap(sy + 1, sx) * ((32 - fx) * fy * 32)[..., None] + tap(sy + 1, sx + 1) * (fx * fy * 32)[..., None])
    return np.clip((acc + (1 << 14)) >> 15, 0, 255).astype(np.uint8)


def warp_affine_nearest_u8(src, forward):
    """``cv::warpAffine(src, dst, M, src.size(), INTER_NEAREST, BORDER_CONSTANT, 0)``: the same 10-bit fixed-point source
    coordinates as the linear form, rounded to the nearest whole pixel (half of 2^10 added before the shift); a pixel
    whose source lies outside the picture is zero."""
    h, w = src.shape[:2]
    M = invert_affine(forward)
    ab = 1024.0
    xs = np.arange(w, dtype=np.float64)
    ys = np.arange(h, dtype=np.float64)
    adelta = np.rint(M[0] * xs * ab).astype(np.int64)
    bdelta = np.rint(M[3] * xs * ab).astype(np.int64)
    x0 = np.rint((M[1] * ys + M[2]) * ab).astype(np.int64) + 512
    y0 = np.rint((M[4] * ys + M[5]) * ab).astype(np.int64) + 512
    X = np.clip((x0[:, None] + adelta[None, :]) >> 10, -32768, 32767)
    Y = np.clip((y0[:, None] + bdelta[None, :]) >> 10, -32768, 32767)
    ok = (X >= 0) & (X < w) & (Y >= 0) & (Y < h)
    out = src[np.clip(Y, 0, h - 1), np.clip(X, 0, w - 1)]
    return (out * (ok if src.ndim == 2 else ok[..., None])).astype(np.uint8)


def rotate(img, angle, interpolate=True):
    """aeon ``image::rotate`` (src/image.cpp:53-75): linear interpolation by default, nearest with
    ``interpolate == false``; zero border."""
    if angle == 0:
        return img
    warp = warp_affine_linear_u8 if interpolate else warp_affine_nearest_u8
    return warp(img, rotation_matrix(img.shape[1], img.shape[0], angle))


def transform_pixel_mask(mask, p):
    """aeon ``pixel_mask::transformer::transform`` (src/etl_pixel_mask.cpp:62-92; ``depthmap::transformer`` is the
    same, src/etl_depthmap.cpp:62-92): rotation without interpolation, the crop box taken from the rotated mask itself,
    NEAREST resize to the output size, flip.  Nothing else of the parameters applies to a mask."""
    mask = rotate(mask, p.angle, interpolate=False)
    x, y, w, h = p.cropbox
    if x < 0 or y < 0 or w <= 0 or h <= 0 or x + w > mask.shape[1] or y + h > mask.shape[0]:
        raise ValueError("cropbox outside the mask")
    mask = _resize(mask[y:y + h, x:x + w], p.output_size, "NEAREST")
    if p.flip:
        mask = mask[:, ::-1]
    return np.ascontiguousarray(mask)


def transform_single_image(img, p):
    """aeon ``image::transformer::transform_single_image`` (src/etl_image.cpp:146-202)."""
    img = rotate(img, p.angle)
    if f32(p.expand_ratio) > 1.0:
        img = expand(img, p.expand_offset, p.expand_size)
    if p.resize_short_size != 0:
        img = _resize(img, resized_short_size(img.shape[1], img.shape[0], p.resize_short_size),
                      p.interpolation_method)
    x, y, w, h = p.cropbox
    if x < 0 or y < 0 or w <= 0 or h <= 0 or x + w > img.shape[1] or y + h > img.shape[0]:
        raise ValueError("cropbox outside the image")
    img = img[y:y + h, x:x + w]
    if p.padding != 0 and tuple(p.padding_crop_offset) != (p.padding, p.padding):
        pad = p.padding
        canvas = np.zeros((h + 2 * pad, w + 2 * pad, img.shape[2]), img.dtype)
        canvas[pad:pad + h, pad:pad + w] = img
        ox, oy = p.padding_crop_offset
        img = canvas[oy:oy + h, ox:ox + w]
    img = _resize(img, p.output_size, p.interpolation_method)
    img = cbsjitter(img, p.contrast, p.brightness, p.saturation, p.hue)
    img = lighting_u8(img, p.lighting, p.color_noise_std)
    if p.flip:
        img = img[:, ::-1]
    return np.ascontiguousarray(img)


_DTYPES = {"uint8_t": np.uint8, "int8_t": np.int8, "int16_t": np.int16, "uint16_t": np.uint16,
           "int32_t": np.int32, "uint32_t": np.int32, "float": np.float32, "double": np.float64,
           "char": np.int8}


def load_image(img, channel_major=True, bgr_to_rgb=False, output_type="uint8_t", mean=None, stddev=None):
    """aeon ``image::loader::load`` for one image without ``fixed_aspect_ratio``
    (src/etl_image.cpp:317-339): depth conversion, optional BGR->RGB, HWC->CHW split,
    then ``x*(1/255) - mean_c`` and ``*(1/std_c)`` in the output precision
    (src/image.cpp:129-174; a zero std leaves the channel unscaled).
    """
    dt = _DTYPES[output_type]
    if np.issubdtype(dt, np.integer) and dt != np.uint8:
        info = np.iinfo(dt)
        x = np.clip(img.astype(np.int64), info.min, info.max).astype(dt)
    else:
        x = img.astype(dt)
    if bgr_to_rgb:
        x = x[..., ::-1]
    if mean is not None and len(mean):
        x = x.copy()
        for c in range(x.shape[2]):
            t = x[..., c] * dt(1.0 / 255.0)
            t = t - dt(mean[c])
            if stddev[c]:
                t = t * dt(1.0 / stddev[c])
            x[..., c] = t
    if channel_major:
        x = np.transpose(x, (2, 0, 1))
    return np.ascontiguousarray(x)


def load_video(frames, max_frame_count):
    """aeon ``video::transformer`` trimming/padding + ``video::loader::load``
    (src/etl_video.cpp:49-107): uint8 planes at ``c*T*H*W + t*H*W``, no channel swap."""
    frames = list(frames[:max_frame_count])
    h, w = frames[0].shape[:2]
    while len(frames) < max_frame_count:
        frames.append(np.zeros((h, w, 3), np.uint8))
    return np.ascontiguousarray(np.stack(frames, 0).transpose(3, 0, 1, 2))
