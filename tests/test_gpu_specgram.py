"""Parity of the spectrogram kernel with the CPU oracle (1e-4 relative + 2e-4 absolute on log values;
-inf of empty mel filters must match exactly)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import specgram as ospec

pytestmark = pytest.mark.gpu


def synth_clip(rng, seconds, sr=16000):
    t = np.arange(int(seconds * sr)) / sr
    x = np.zeros_like(t)
    for _ in range(int(rng.integers(1, 6))):
        x += rng.uniform(0.05, 0.3) * np.sin(2 * np.pi * rng.uniform(80, 7000) * t + rng.uniform(0, 6.28))
    x += rng.normal(0, 0.05, len(t))
    return np.clip(x * 32767 / 2, -32768, 32767).astype(np.int16)


def run(ctx, clips, frame_length=320, frame_stride=160, max_time_steps=200, num_filters=64, sample_rate=16000, window=1,
        num_cepstra=0):
    from aeon_b200 import _lib as L
    dev = torch.device("cuda", ctx.device)
    n_out = num_cepstra if num_cepstra else num_filters if num_filters else frame_length // 2 + 1
    cfg = L.SpecgramConfig(frame_length, frame_stride, max_time_steps, num_filters, sample_rate, window, num_cepstra, 0)
    with torch.cuda.stream(ctx.torch_stream):
        out = torch.full((len(clips), max_time_steps, n_out), 7.0, dtype=torch.float32, device=dev)
        ts = [torch.from_numpy(c).to(dev) for c in clips]
        descs = (L.SpecgramDesc * len(clips))()
        for i, t in enumerate(ts):
            descs[i].samples, descs[i].n_samples = t.data_ptr(), t.numel()
            descs[i].dst = out[i].data_ptr()
        L.check(ctx.lib.aeonb_specgram_batch(ctx.handle, descs, len(clips), C.byref(cfg)))
        ctx.synchronize()
    return out.cpu().numpy()


def assert_close(got, want):
    inf_w = np.isinf(want)
    assert np.array_equal(np.isinf(got), inf_w)
    assert np.array_equal(got[inf_w], want[inf_w])
    g, w = got[~inf_w], want[~inf_w]
    assert np.all(np.abs(g - w) <= 1e-4 * np.abs(w) + 2e-4), float(np.abs(g - w).max())


def test_log_mel_benchmark_shape(ctx):
    rng = np.random.default_rng(31)
    clips = [synth_clip(rng, s) for s in (1.0, 1.99, 0.5, 1.3)]
    got = run(ctx, clips, max_time_steps=199)
    for i, c in enumerate(clips):
        assert_close(got[i], ospec.log_mel(c, max_time_steps=199))
    assert np.isinf(got[0][0]).sum() == 3  # the 64-filter bank at 16 kHz / 320 has three empty filters


def test_magnitude_output_other_lengths_and_windows(ctx):
    rng = np.random.default_rng(32)
    clip = synth_clip(rng, 0.7)
    for L_, win, name in [(256, 0, "none"), (512, 2, "hamming"), (640, 3, "blackman"), (64, 4, "bartlett"), (320, 1, "hann")]:
        got = run(ctx, [clip], frame_length=L_, frame_stride=L_ // 2, max_time_steps=50, num_filters=0, window=win)[0]
        want = ospec.log_mel(clip, L_, L_ // 2, 50, 0, 16000, name)
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 2e-5 * scale, (L_, name)


def test_short_and_empty_clips_zero_fill(ctx):
    rng = np.random.default_rng(33)
    clips = [synth_clip(rng, 0.01), synth_clip(rng, 0.02), synth_clip(rng, 0.0301)]
    got = run(ctx, clips, max_time_steps=8)
    assert not got[0].any()
    for i, c in enumerate(clips):
        assert_close(got[i], ospec.log_mel(c, max_time_steps=8))


def test_oversized_frame_length_is_an_error(ctx):
    from aeon_b200._lib import AeonError
    with pytest.raises(AeonError, match="frame_length"):
        run(ctx, [np.zeros(1000, np.int16)], frame_length=20000, frame_stride=160, num_filters=0)


def test_mfcc(ctx):
    """specgram::cepsgram_to_mfcc (src/specgram.cpp:139-154): DCT-II of the log-mel rows, even and odd filter counts.
    Tolerance: the log-mel bound (1e-4 relative + 2e-4) carried through a sum of num_filters terms: 1e-4 relative + 1e-3."""
    rng = np.random.default_rng(35)
    clips = [synth_clip(rng, s) for s in (0.9, 0.4)]
    for nf, nc, L_ in [(40, 13, 512), (23, 23, 512), (32, 1, 256)]:
        want = [ospec.log_mel(c, frame_length=L_, max_time_steps=60, num_filters=nf, num_cepstra=nc) for c in clips]
        assert all(np.isfinite(w).all() for w in want)      # a bank without empty filters
        got = run(ctx, clips, frame_length=L_, max_time_steps=60, num_filters=nf, num_cepstra=nc)
        assert got.shape == (2, 60, nc)
        for g, w in zip(got, want):
            assert np.all(np.abs(g - w) <= 1e-4 * np.abs(w) + 1e-3), float(np.abs(g - w).max())
    from aeon_b200 import _lib as L
    cfg = L.SpecgramConfig(512, 160, 60, 20, 16000, 1, 21, 0)   # more cepstra than filters: the reference's affirm
    d = (L.SpecgramDesc * 1)()
    t = torch.zeros(2000, dtype=torch.int16, device="cuda")
    o = torch.zeros(60 * 21, dtype=torch.float32, device="cuda")
    d[0].samples, d[0].n_samples, d[0].dst = t.data_ptr(), 2000, o.data_ptr()
    assert ctx.lib.aeonb_specgram_batch(ctx.handle, d, 1, C.byref(cfg)) == L.ERR_INVALID


def test_frame_lengths_without_a_factor_of_64(ctx):
    """400 samples (25 ms at 16 kHz), odd and long frames take the direct-sum kernel: same tolerances as the FFT kernel."""
    rng = np.random.default_rng(36)
    clip = synth_clip(rng, 0.9)
    for L_, win, name in [(400, 1, "hann"), (200, 0, "none"), (321, 2, "hamming"), (1000, 3, "blackman"), (7, 4, "bartlett"), (1024, 1, "hann")]:
        got = run(ctx, [clip], frame_length=L_, frame_stride=max(L_ // 2, 1), max_time_steps=40, num_filters=0, window=win)[0]
        want = ospec.log_mel(clip, L_, max(L_ // 2, 1), 40, 0, 16000, name)
        assert got.shape == want.shape == (40, L_ // 2 + 1)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max(), (L_, name)
    clips = [synth_clip(rng, s) for s in (1.0, 0.3)]
    got = run(ctx, clips, frame_length=400, frame_stride=160, max_time_steps=98, num_filters=40)
    for g, c in zip(got, clips):
        assert_close(g, ospec.log_mel(c, 400, 160, 98, 40))
    got = run(ctx, clips, frame_length=400, frame_stride=160, max_time_steps=98, num_filters=40, num_cepstra=13)
    for g, c in zip(got, clips):
        w = ospec.log_mel(c, 400, 160, 98, 40, num_cepstra=13)
        assert np.isfinite(w).all() and np.all(np.abs(g - w) <= 1e-4 * np.abs(w) + 1e-3)
