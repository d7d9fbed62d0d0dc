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


def with_exif_orientation(jpeg, orientation, big_endian=False):
    """Insert an APP1 Exif segment whose IFD0 holds only the orientation tag (0x0112) after the SOI marker."""
    import struct
    e = ">" if big_endian else "<"
    tiff = (b"MM\x00\x2a" if big_endian else b"II\x2a\x00") + struct.pack(e + "I", 8) + struct.pack(e + "H", 1) + \
        struct.pack(e + "HHIHH", 0x0112, 3, 1, orientation, 0) + struct.pack(e + "I", 0)
    payload = b"Exif\x00\x00" + tiff
    return jpeg[:2] + b"\xff\xe1" + struct.pack(">H", len(payload) + 2) + payload + jpeg[2:]
