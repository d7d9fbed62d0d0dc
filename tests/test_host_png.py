"""Host PNG decoder against cv2.imdecode(IMREAD_COLOR): bit-exact for every colour type / bit depth / deflate strategy."""
import io

import numpy as np
import pytest


import struct
import zlib


def decode(blob, grey=False):
    from aeon_b200 import kernels as K
    return K.png_decode(blob, grey)


def reference(blob, grey=False):
    import cv2
    return cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_GRAYSCALE if grey else cv2.IMREAD_COLOR)


def write_png(samples, color_type, bit_depth, interlaced=False, palette=None, filters=(0, 1, 2, 3, 4)):
    """A PNG writer for the cases no library here emits (Adam7 interlacing, chosen row filters).  `samples`: H x W x C
    array of sample values (C = 1, 2, 3 or 4 by colour type; palette indices for type 3)."""
    h, w, ch = samples.shape

    def pack_row(row):      # row: n x C sample values -> bytes
        if bit_depth == 16:
            return row.astype(">u2").tobytes()
        if bit_depth == 8:
            return row.astype(np.uint8).tobytes()
        bits = np.zeros(((row.shape[0] * bit_depth + 7) // 8) * 8, np.uint8)
        flat = row[:, 0].astype(np.uint8)
        for k in range(bit_depth):
            bits[k:flat.size * bit_depth:bit_depth] = (flat >> (bit_depth - 1 - k)) & 1
        return np.packbits(bits).tobytes()

    bpp = max(1, ch * bit_depth // 8)

    def filtered(rows):     # list of bytes per row -> filter byte + filtered bytes, cycling through the filter types
        out, prev = bytearray(), None
        for y, cur in enumerate(rows):
            f = filters[y % len(filters)]
            cur = np.frombuffer(cur, np.uint8).astype(np.int32)
            up = np.zeros_like(cur) if prev is None else prev
            left = np.concatenate([np.zeros(bpp, np.int32), cur[:-bpp]]) if cur.size > bpp else np.zeros_like(cur)
            if cur.size <= bpp:
                left = np.zeros_like(cur)
            ul = np.concatenate([np.zeros(bpp, np.int32), up[:-bpp]]) if cur.size > bpp else np.zeros_like(cur)
            if f == 0:
                res = cur
            elif f == 1:
                res = cur - left
            elif f == 2:
                res = cur - up
            elif f == 3:
                res = cur - ((left + up) >> 1)
            else:
                p = left + up - ul
                pa, pb, pc = np.abs(p - left), np.abs(p - up), np.abs(p - ul)
                pred = np.where((pa <= pb) & (pa <= pc), left, np.where(pb <= pc, up, ul))
                res = cur - pred
            out.append(f)
            out += (res & 255).astype(np.uint8).tobytes()
            prev = cur
        return bytes(out)

    passes = [(0, 0, 8, 8), (4, 0, 8, 8), (0, 4, 4, 8), (2, 0, 4, 4), (0, 2, 2, 4), (1, 0, 2, 2), (0, 1, 1, 2)] if interlaced \
        else [(0, 0, 1, 1)]
    raw = b""
    for x0, y0, dx, dy in passes:
        sub = samples[y0::dy, x0::dx]
        if sub.shape[0] and sub.shape[1]:
            raw += filtered([pack_row(r) for r in sub])

    def chunk(tag, body):
        return struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body))

    blob = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, bit_depth, color_type, 0, 0, int(interlaced)))
    if palette is not None:
        blob += chunk(b"PLTE", np.asarray(palette, np.uint8).tobytes())
    z = zlib.compress(raw, 6)
    half = len(z) // 2
    return blob + chunk(b"IDAT", z[:half]) + chunk(b"IDAT", z[half:]) + chunk(b"IEND", b"")


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


@pytest.mark.parametrize("size", [(1, 1), (3, 2), (5, 9), (8, 8), (33, 47), (120, 67)])
def test_interlaced_files_and_every_row_filter(size):
    """Adam7 files (seven reduced images in one stream, empty passes for tiny pictures) for every colour type."""
    h, w = size
    rng = np.random.default_rng(h * 131 + w)
    cases = [(rng.integers(0, 256, (h, w, 3)), 2, 8, None), (rng.integers(0, 256, (h, w, 4)), 6, 8, None),
             (rng.integers(0, 256, (h, w, 1)), 0, 8, None), (rng.integers(0, 65536, (h, w, 3)), 2, 16, None),
             (rng.integers(0, 65536, (h, w, 2)), 4, 16, None), (rng.integers(0, 16, (h, w, 1)), 0, 4, None),
             (rng.integers(0, 2, (h, w, 1)), 0, 1, None),
             (rng.integers(0, 4, (h, w, 1)), 3, 2, rng.integers(0, 256, (4, 3))),
             (rng.integers(0, 200, (h, w, 1)), 3, 8, rng.integers(0, 256, (200, 3)))]
    for i, (samples, ctype, depth, palette) in enumerate(cases):
        for interlaced in (True, False):
            blob = write_png(samples, ctype, depth, interlaced, palette)
            want = reference(blob)
            assert want is not None and want.shape == (h, w, 3)
            assert np.array_equal(decode(blob), want), (size, i, interlaced)
            assert np.array_equal(decode(blob, grey=True), reference(blob, grey=True)), (size, i, interlaced, "grey")


def test_colour_files_read_as_one_channel():
    """IMREAD_GRAYSCALE / IMREAD_ANYDEPTH of a colour file: libpng's integer weights, truncated for 8-bit samples and
    rounded on the 16-bit values for 16-bit samples."""
    import cv2
    Image = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(23)
    rgb = rng.integers(0, 256, (61, 77, 3), dtype=np.uint8)
    blobs = [cv2.imencode(".png", rgb)[1].tobytes(),
             cv2.imencode(".png", np.dstack([rgb, rgb[..., 0]]))[1].tobytes(),
             cv2.imencode(".png", rng.integers(0, 65536, (61, 77, 3), dtype=np.uint16))[1].tobytes(),
             cv2.imencode(".png", rng.integers(0, 65536, (61, 77, 4), dtype=np.uint16))[1].tobytes(),
             cv2.imencode(".png", rgb[..., 1].copy())[1].tobytes()]
    for bits in (8, 4, 1):
        b = io.BytesIO()
        Image.fromarray(rgb).convert("P", colors=1 << bits).save(b, format="PNG", bits=bits)
        blobs.append(b.getvalue())
    for i, blob in enumerate(blobs):
        got = decode(blob, grey=True)
        assert np.array_equal(got, reference(blob, grey=True)), i
        if i not in (2, 3):   # 8-bit files: the pixelmask extractor's IMREAD_ANYDEPTH read gives the same picture
            assert np.array_equal(got, cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_ANYDEPTH)), i
