"""Host PNG decoder against cv2.imdecode(IMREAD_COLOR): bit-exact for every colour type / bit depth / deflate strategy."""
import io

import numpy as np
import pytest


def decode(blob):
    from aeon_b200 import kernels as K
    return K.png_decode(blob)


def reference(blob):
    import cv2
    return cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_COLOR)


@pytest.mark.parametrize("size", [(1, 1), (7, 5), (32, 32), (100, 133), (375, 500)])
def test_opencv_written_files(size):
    import cv2
    h, w = size
    rng = np.random.default_rng(h * 991 + w)
    noise = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    smooth = (np.add.outer(np.arange(h), np.arange(w)) % 256).astype(np.uint8)
    blobs = [cv2.imencode(".png", noise, [cv2.IMWRITE_PNG_COMPRESSION, c])[1].tobytes() for c in (0, 1, 3, 6, 9)]
    blobs.append(cv2.imencode(".png", smooth)[1].tobytes())                                                 # grey
    blobs.append(cv2.imencode(".png", np.dstack([noise, smooth]))[1].tobytes())                             # alpha is dropped
    blobs.append(cv2.imencode(".png", rng.integers(0, 65536, (h, w), dtype=np.uint16))[1].tobytes())        # 16-bit grey
    blobs.append(cv2.imencode(".png", rng.integers(0, 65536, (h, w, 3), dtype=np.uint16))[1].tobytes())     # 16-bit colour
    for strategy in (cv2.IMWRITE_PNG_STRATEGY_FILTERED, cv2.IMWRITE_PNG_STRATEGY_HUFFMAN_ONLY, cv2.IMWRITE_PNG_STRATEGY_RLE,
                     cv2.IMWRITE_PNG_STRATEGY_FIXED):
        blobs.append(cv2.imencode(".png", np.dstack([smooth] * 3), [cv2.IMWRITE_PNG_STRATEGY, strategy])[1].tobytes())
    for i, blob in enumerate(blobs):
        assert np.array_equal(decode(blob), reference(blob)), (size, i)


def test_palette_and_low_bit_depths():
    Image = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(17)
    rgb = rng.integers(0, 256, (40, 53, 3), dtype=np.uint8)
    grey = rng.integers(0, 256, (40, 53), dtype=np.uint8)
    blobs = []
    for bits in (8, 4, 2, 1):
        b = io.BytesIO()
        Image.fromarray(rgb).convert("P", colors=1 << bits).save(b, format="PNG", bits=bits)
        blobs.append(b.getvalue())
    for mode in ("L", "1", "LA"):
        b = io.BytesIO()
        Image.fromarray(grey).convert(mode).save(b, format="PNG")
        blobs.append(b.getvalue())
    for i, blob in enumerate(blobs):
        assert np.array_equal(decode(blob), reference(blob)), i


def test_malformed_files():
    import cv2
    from aeon_b200 import _lib as L
    good = cv2.imencode(".png", np.zeros((20, 20, 3), np.uint8) + 7)[1].tobytes()
    idat = good.index(b"IDAT")
    for blob in (good[:40], good[:idat + 10] + good[idat + 14:], good[:idat + 4] + bytes(len(good) - idat - 4)):
        with pytest.raises(L.AeonError, match="Decoding image failed"):
            decode(blob)
