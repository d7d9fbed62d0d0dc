"""Pins of the JPEG and spectrogram oracles against the OpenCV binary, and of the host entropy
decoder (product code, CPU only) against the oracle's entropy decoder."""
import os

import cv2
import numpy as np
import pytest

from oracle import jpeg as ojpeg
from oracle import specgram as ospec
from tests.synth import gradient_image, jpeg_bytes


def _cases():
    rng = np.random.default_rng(6)
    out = []
    for (h, w) in [(8, 8), (1, 1), (17, 16), (37, 53), (64, 80), (33, 47), (15, 130)]:
        for extra in ([], [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444],
                      [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422],
                      [cv2.IMWRITE_JPEG_RST_INTERVAL, 2]):
            out.append(jpeg_bytes(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), int(rng.integers(30, 100)), extra))
    out.append(jpeg_bytes(gradient_image(rng, 45, 30)[..., 0], 85))
    out.append(jpeg_bytes(gradient_image(rng, 120, 90), 90))
    return out


def test_jpeg_oracle_matches_opencv_bit_for_bit():
    for i, blob in enumerate(_cases()):
        ref = cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_COLOR)
        assert np.array_equal(ojpeg.decode(blob), ref), i


def test_jpeg_oracle_on_reference_fixture(golden_dir):
    blob = open(os.path.join(golden_dir, "img_2112_70.jpg"), "rb").read()
    assert np.array_equal(ojpeg.decode(blob), cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_COLOR))


def test_host_entropy_decoder_matches_oracle_coefficients(golden_dir):
    from aeon_b200 import kernels as K
    blobs = _cases() + [open(os.path.join(golden_dir, n), "rb").read() for n in ("img_2112_70.jpg", "flowers.jpg")]
    for i, blob in enumerate(blobs[:-1] + blobs[-1:]):
        if i == len(blobs) - 1:
            co = None  # flowers.jpg is large for the python decoder: check the restart-marker path against OpenCV on the GPU instead
        else:
            co = ojpeg.entropy_decode(blob)
        info, coefs, quants = K.jpeg_entropy_decode(blob)
        if co is None:
            assert (info.width, info.height) == (600, 800)
            continue
        assert (info.width, info.height, info.ncomp) == (co.width, co.height, co.ncomp)
        for c in range(info.ncomp):
            mine = coefs[c].reshape(info.blocks_h[c], info.blocks_w[c], 8, 8).transpose(0, 1, 3, 2)  # column-major blocks
            assert np.array_equal(mine, co.blocks[c]), (i, c)
            assert np.array_equal(quants[c].reshape(8, 8).T.ravel(), co.quant[c])


def test_corrupt_jpeg_is_reported_like_the_reference():
    import pytest
    from aeon_b200 import kernels as K
    from aeon_b200._lib import AeonError
    good = jpeg_bytes(gradient_image(np.random.default_rng(7), 32, 32), 90)
    for blob in (b"", b"abc", good[:10], b"\xff\xd8\xff\xd9"):
        with pytest.raises(AeonError, match="Decoding image failed due to invalid data in the image file."):
            K.jpeg_entropy_decode(blob)


def test_specgram_oracle_matches_opencv_dft_and_log():
    rng = np.random.default_rng(8)
    x = (rng.normal(0, 0.1, 16000) * 20000).astype(np.int16)
    win = ospec.create_window("hann", 320)
    spec = ospec.wav_to_specgram(x, 320, 160, 1599, win)
    idx = np.arange(spec.shape[0])[:, None] * 160 + np.arange(320)[None, :]
    fr = x[idx].astype(np.float32) * win[None, :]
    d = cv2.dft(np.stack([fr, np.zeros_like(fr)], -1), flags=cv2.DFT_ROWS)[:, :161]
    mag = cv2.magnitude(d[..., 0], d[..., 1])
    assert (np.abs(mag - spec) / np.abs(spec).max()).max() < 1e-5
    fb = ospec.create_filterbanks(64, 320, 16000)
    ceps = cv2.log(((mag * mag) / np.float32(320)) @ fb)
    mine = ospec.specgram_to_cepsgram(spec, fb)
    assert np.array_equal(np.isinf(ceps), np.isinf(mine)) and np.isinf(mine[0]).sum() == 3
    m = ~np.isinf(mine)
    assert np.abs(ceps[m] - mine[m]).max() < 2e-4
    assert ospec.filterbank_edges(64, 320, 16000)[:8] == [0, 0, 1, 1, 2, 3, 3, 4]


def test_mfcc_oracle_matches_opencv_dct():
    """cepsgram_to_mfcc (src/specgram.cpp:139-154) against cv2.dct(DCT_ROWS) on even and odd (zero-padded) widths."""
    import cv2
    rng = np.random.default_rng(88)
    for nf, nc in [(64, 40), (40, 13), (13, 13), (7, 3)]:
        x = rng.normal(0, 3, (50, nf)).astype(np.float32)
        pad = x if nf % 2 == 0 else np.concatenate([x, np.zeros((50, 1), np.float32)], 1)
        ref = cv2.dct(pad, flags=cv2.DCT_ROWS)[:, :nc]
        assert np.abs(ospec.cepsgram_to_mfcc(x, nc) - ref).max() <= 5e-6
    with pytest.raises(ValueError):
        ospec.cepsgram_to_mfcc(np.zeros((2, 4), np.float32), 5)
