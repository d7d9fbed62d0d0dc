"""Host decoder for progressive JPEG (ITU-T T.81 annex G: spectral selection + successive approximation).

OpenCV writes the same quantised coefficients whether it codes them as one baseline scan or as libjpeg's ten
progressive scans, so decoding both files must give the same coefficient planes (over the blocks that hold
picture samples: baseline also codes the padding blocks of partial MCUs, a progressive AC scan does not)."""
import numpy as np
import pytest

from tests.synth import gradient_image


def planes(blob):
    from aeon_b200 import kernels as K
    return K.jpeg_entropy_decode(blob)


@pytest.mark.parametrize("size", [(64, 64), (37, 53), (200, 150), (8, 8), (1, 1), (375, 500)])
def test_progressive_and_baseline_files_hold_the_same_coefficients(size):
    import cv2
    h, w = size
    rng = np.random.default_rng(h * 1000 + w)
    for extra in ([], [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444],
                  [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422], [cv2.IMWRITE_JPEG_RST_INTERVAL, 5],
                  [cv2.IMWRITE_JPEG_OPTIMIZE, 1]):
        img = gradient_image(rng, h, w)
        q = int(rng.integers(40, 100))
        base = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, q] + extra)[1].tobytes()
        prog = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, q, cv2.IMWRITE_JPEG_PROGRESSIVE, 1] + extra)[1].tobytes()
        assert b"\xff\xc2" in prog and b"\xff\xc2" not in base[:600]
        ib, cb, qb = planes(base)
        ip, cp, qp = planes(prog)
        assert (ib.width, ib.height, ib.ncomp) == (ip.width, ip.height, ip.ncomp) == (w, h, 3)
        hmax, vmax = max(ib.hs[:3]), max(ib.vs[:3])
        for c in range(3):
            bw, bh = ib.blocks_w[c], ib.blocks_h[c]
            nbw, nbh = -(-(-(-w * ib.hs[c] // hmax)) // 8), -(-(-(-h * ib.vs[c] // vmax)) // 8)
            a = cb[c].reshape(bh, bw, 64)[:nbh, :nbw]
            b = cp[c].reshape(bh, bw, 64)[:nbh, :nbw]
            assert np.array_equal(a, b), (size, extra, c)
            assert np.array_equal(qb[c], qp[c])


def test_grey_progressive_and_truncated_stream():
    import cv2
    from aeon_b200 import _lib as L
    rng = np.random.default_rng(5)
    img = gradient_image(rng, 45, 30)[..., 0]
    base = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, 85])[1].tobytes()
    prog = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, 85, cv2.IMWRITE_JPEG_PROGRESSIVE, 1])[1].tobytes()
    ib, cb, _ = planes(base)
    ip, cp, _ = planes(prog)
    assert ip.ncomp == 1 and np.array_equal(cb[0], cp[0])   # one component: no padding blocks differ (both code ceil sizes)
    sos = prog.index(b"\xff\xda")
    with pytest.raises(L.AeonError, match="Decoding image failed"):
        planes(prog[:sos])                                   # headers only


def test_exif_orientation_tag_is_parsed():
    """aeonb_jpeg_parse reports the EXIF orientation (both byte orders); stored width/height stay those of the frame header."""
    from aeon_b200 import kernels as K
    from tests.synth import jpeg_bytes, with_exif_orientation
    rng = np.random.default_rng(6)
    blob = jpeg_bytes(gradient_image(rng, 24, 40), 90)
    assert K.jpeg_parse(blob).orientation == 1
    for o in range(1, 9):
        for big in (False, True):
            info = K.jpeg_parse(with_exif_orientation(blob, o, big))
            assert (info.orientation, info.width, info.height) == (o, 40, 24)
    assert K.jpeg_parse(with_exif_orientation(blob, 9)).orientation == 1          # out of range: ignored, as OpenCV does
    broken = blob[:2] + b"\xff\xe1\x00\x0cExif\x00\x00II\x2a\x00" + blob[2:]        # truncated TIFF header
    assert K.jpeg_parse(broken).orientation == 1


def test_truncated_scan_headers_are_rejected_not_read_past():
    """A scan header cut short (its length field says 2, or fewer selector bytes than components) is a decode error."""
    import cv2
    from aeon_b200._lib import AeonError
    img = gradient_image(np.random.default_rng(5), 24, 24)
    for extra in ([], [cv2.IMWRITE_JPEG_PROGRESSIVE, 1]):
        blob = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, 80] + extra)[1].tobytes()
        at = blob.index(b"\xff\xda")
        for cut in (blob[:at + 2] + b"\x00\x02", blob[:at + 2] + b"\x00\x03\x03", blob[:at + 2] + b"\x00\x08\x03\x01\x00\x02\x11\x03"):
            with pytest.raises(AeonError):
                planes(cut)
