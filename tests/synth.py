"""Seeded synthetic inputs shaped like the benchmark datasets (smooth gradients + uniform noise)."""
import numpy as np


def gradient_image(rng, h, w, noise=20):
    yy, xx = np.mgrid[0:h, 0:w]
    img = np.empty((h, w, 3), np.float64)
    for c in range(3):
        a, b = rng.uniform(-0.4, 0.4, 2)
        img[..., c] = rng.uniform(40, 215) + a * xx + b * yy
    img += rng.uniform(-noise, noise, img.shape)
    return np.clip(img, 0, 255).astype(np.uint8)


def jpeg_bytes(img, quality=90, extra=()):
    import cv2
    ok, enc = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, quality] + list(extra))
    assert ok
    return enc.tobytes()
