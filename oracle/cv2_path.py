"""aeon's per-record image path replayed on the OpenCV binary (TEST INFRASTRUCTURE ONLY).

The reference cannot be compiled without OpenCV's C++ development files, but the
python ``cv2`` module exposes the same OpenCV entry points aeon calls.  This module
issues those calls in aeon's order so that

* the numpy restatement in ``image_ops`` can be pinned against what OpenCV returns, and
* the benchmark has a CPU baseline that spends its time in the same library code
  (libjpeg-turbo decode, SIMD resize/transform/cvtColor) as the reference would.

Nothing in the shipped package imports this file.
"""
import numpy as np
import cv2

from . import image_ops as ops

cv2.setNumThreads(1)  # aeon parallelises over records, not inside OpenCV calls

_INTERP = {"NEAREST": cv2.INTER_NEAREST, "LINEAR": cv2.INTER_LINEAR, "CUBIC": cv2.INTER_CUBIC,
           "AREA": cv2.INTER_AREA, "LANCZOS4": cv2.INTER_LANCZOS4}


def extract(encoded):
    """src/etl_image.cpp:83-99."""
    img = cv2.imdecode(np.frombuffer(encoded, np.uint8), cv2.IMREAD_COLOR)
    if img is None:
        raise RuntimeError("Decoding image failed due to invalid data in the image file.")
    return img


def cbsjitter(img, contrast, brightness, saturation, hue):
    """src/image.cpp:358-406."""
    if np.float32(brightness) != 1.0 or np.float32(saturation) != 1.0:
        img = cv2.transform(img, ops.color_matrix(brightness, saturation))
    if int(hue) != 0:
        hsv = cv2.cvtColor(img, cv2.COLOR_BGR2HSV)
        # uint8((H + hue) % 180) with C remainder, as a 256-entry table
        t = np.arange(256, dtype=np.int32) + int(hue)
        lut = (np.fmod(t, 180).astype(np.int32) & 0xFF).astype(np.uint8)
        hsv[..., 0] = cv2.LUT(np.ascontiguousarray(hsv[..., 0]), lut)
        img = cv2.cvtColor(hsv, cv2.COLOR_HSV2BGR)
    if np.float32(contrast) != 1.0:
        c = float(np.float32(contrast))
        mean = cv2.mean(img)
        add = np.array([(1.0 - c) * m for m in mean[:3]]).astype(np.float32)
        # convertTo(CV_32F, c); += scalar; convertTo(CV_8U).  The scalar add is done by numpy (same float32
        # addition) because the python binding of cv2.add with a scalar is far slower than the C++ call.
        dst = img.astype(np.float32) * np.float32(c) + add
        img = cv2.addWeighted(dst, 1.0, dst, 0.0, 0.0, dtype=cv2.CV_8U)  # saturating round-half-even cast
    return img


def lighting(img, alphas, color_noise_std):
    """src/image.cpp:336-346, two-step evaluation of the matrix expression."""
    if alphas is None or len(alphas) == 0:
        return img
    alpha = 1.0 / (1.0 + float(np.float32(color_noise_std)))
    pix = ops.lighting_pixel(alphas).astype(np.float64) * alpha
    t = cv2.convertScaleAbs(img, alpha=alpha)
    return cv2.add(t, (float(pix[0]), float(pix[1]), float(pix[2]), 0.0))


def transform_single_image(img, p):
    """src/etl_image.cpp:146-202 with OpenCV doing the pixel work."""
    if p.angle != 0:   # image::rotate, src/image.cpp:53-75
        rot = cv2.getRotationMatrix2D((img.shape[1] // 2, img.shape[0] // 2), p.angle, 1.0)
        img = cv2.warpAffine(img, rot, (img.shape[1], img.shape[0]), flags=cv2.INTER_LINEAR, borderMode=cv2.BORDER_CONSTANT,
                             borderValue=(0, 0, 0, 0))
    if np.float32(p.expand_ratio) > 1.0:
        img = ops.expand(img, p.expand_offset, p.expand_size)
    if p.resize_short_size != 0:
        img = cv2.resize(img, ops.resized_short_size(img.shape[1], img.shape[0], p.resize_short_size),
                         interpolation=_INTERP[p.interpolation_method.upper()])
    x, y, w, h = p.cropbox
    img = img[y:y + h, x:x + w]
    if p.padding != 0 and tuple(p.padding_crop_offset) != (p.padding, p.padding):
        padded = cv2.copyMakeBorder(img, p.padding, p.padding, p.padding, p.padding, cv2.BORDER_CONSTANT, value=0)
        ox, oy = p.padding_crop_offset
        img = padded[oy:oy + h, ox:ox + w]
    if (img.shape[1], img.shape[0]) != tuple(p.output_size):
        img = cv2.resize(img, tuple(p.output_size), interpolation=_INTERP[p.interpolation_method.upper()])
    img = cbsjitter(np.ascontiguousarray(img), p.contrast, p.brightness, p.saturation, p.hue)
    img = lighting(img, p.lighting, p.color_noise_std)
    if p.flip:
        img = cv2.flip(img, 1)
    return img


def load_image(img, channel_major=True, bgr_to_rgb=False, output_type="uint8_t", mean=None, stddev=None):
    """src/etl_image.cpp:317-339 + src/image.cpp:129-212 (split / convertTo / multiply / subtract)."""
    dt = ops._DTYPES[output_type]
    x = img.astype(dt)
    planes = list(cv2.split(x))
    if bgr_to_rgb:
        planes = planes[::-1]
    if mean is not None and len(mean):
        for c in range(len(planes)):
            t = cv2.multiply(planes[c], 1.0 / 255.0)
            t = t - dt(mean[c])  # cv::subtract with a scalar; numpy does the same subtraction far faster from python
            if stddev[c]:
                t = cv2.multiply(t, 1.0 / float(stddev[c]))
            planes[c] = t.reshape(planes[c].shape)
    if channel_major:
        return np.ascontiguousarray(np.stack(planes, 0))
    return np.ascontiguousarray(np.stack(planes, -1))
