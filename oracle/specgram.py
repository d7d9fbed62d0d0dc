"""CPU oracle for aeon's spectrogram routines (TEST INFRASTRUCTURE ONLY).

Restates specgram::create_window, create_filterbanks, wav_to_specgram and
specgram_to_cepsgram (aeon src/specgram.cpp:26-189).  aeon's own test file for these
routines is empty and no provider calls them, so there is no reference vector to pin
against: PARITY UNPINNED by the reference; the CPU tests pin this module against the
OpenCV entry points the routines call (cv2.dft / cv2.magnitude / cv2.log) instead.
The transform itself is evaluated in float64 here; outputs are compared with a
relative tolerance of 1e-4 (OpenCV's own float32 DFT sits about 7e-5 from float64).
Nothing in the shipped package imports this file.
"""
import numpy as np

f32 = np.float32


def create_window(kind, n):
    """src/specgram.cpp:156-189; float32 argument to cos, double arithmetic around it, float32 result."""
    if kind == "none":
        return None
    i = np.arange(n)
    twopi_by_n = f32(2.0 * np.pi / float(f32(n - 1)))
    arg = (twopi_by_n * i.astype(f32)).astype(f32)
    c = np.cos(arg.astype(np.float64)).astype(f32).astype(np.float64)   # cosf result
    if kind == "hann":
        w = 0.5 - 0.5 * c
    elif kind == "hamming":
        w = 0.54 - 0.46 * c
    elif kind == "blackman":
        c2 = np.cos((f32(2) * twopi_by_n * i.astype(f32)).astype(f32).astype(np.float64)).astype(f32).astype(np.float64)
        w = 0.42 - 0.5 * c + 0.08 * c2
    elif kind == "bartlett":
        w = 1.0 - 2.0 * np.abs(i - n / 2.0) / n
    else:
        raise RuntimeError("Unsupported window function")
    return w.astype(f32)


def filterbank_edges(num_filters, fftsz, sample_freq_hz):
    hz_to_mel = lambda hz: 2595 * np.log10(1 + hz / 700.0)
    mel_to_hz = lambda mel: 700 * (10 ** (mel / 2595.0) - 1)
    lo, hi = hz_to_mel(0.0), hz_to_mel(sample_freq_hz / 2.0)
    delta = (hi - lo) / (num_filters + 1)
    scale_by = (1 + fftsz) / float(sample_freq_hz)
    return [int(np.floor(scale_by * mel_to_hz(lo + j * delta))) for j in range(num_filters + 2)]


def create_filterbanks(num_filters, fftsz, sample_freq_hz):
    """src/specgram.cpp:93-130 -> float32 matrix [fftsz/2+1, num_filters]."""
    bins = filterbank_edges(num_filters, fftsz, sample_freq_hz)
    nf = fftsz // 2 + 1
    fb = np.zeros((nf, num_filters), f32)
    for j in range(num_filters):
        for i in range(bins[j], min(bins[j + 1], nf)):
            fb[i, j] = (i - bins[j]) / (1.0 * (bins[j + 1] - bins[j]))
        for i in range(bins[j + 1], min(bins[j + 2], nf)):
            fb[i, j] = (bins[j + 2] - i) / (1.0 * (bins[j + 2] - bins[j + 1]))
    return fb


def frame_count(n_samples, frame_length, frame_stride, max_time_steps):
    if n_samples < frame_length:
        return 0
    return min((n_samples - frame_length) // frame_stride + 1, max_time_steps)


def wav_to_specgram(samples, frame_length, frame_stride, max_time_steps, window):
    """src/specgram.cpp:26-86 -> float32 magnitudes [frames, frame_length/2+1]."""
    n = frame_count(len(samples), frame_length, frame_stride, max_time_steps)
    idx = np.arange(n)[:, None] * frame_stride + np.arange(frame_length)[None, :]
    frames = samples[idx].astype(f32) if n else np.zeros((0, frame_length), f32)
    if window is not None:
        frames = frames * window[None, :]
    spec = np.fft.rfft(frames.astype(np.float64), axis=1)
    return np.abs(spec).astype(f32)


def specgram_to_cepsgram(spec, fbank):
    """src/specgram.cpp:132-137: log((mag*mag / (2*(cols-1))) x fbank); empty filters give -inf."""
    power = (spec.astype(np.float64) ** 2) / (2.0 * (spec.shape[1] - 1))
    with np.errstate(divide="ignore"):
        return np.log(power @ fbank.astype(np.float64)).astype(f32)


def cepsgram_to_mfcc(cepsgram, num_cepstra):
    """src/specgram.cpp:139-154: rows zero-padded to an even length N, ``cv::dct(..., DCT_ROWS)`` (orthonormal DCT-II:
    y[j] = s_j sum_k x[k] cos(pi (2k+1) j / (2N)), s_0 = sqrt(1/N), s_j = sqrt(2/N)), first ``num_cepstra`` columns."""
    if num_cepstra > cepsgram.shape[1]:
        raise ValueError("num_cepstra <= cepsgram.cols")
    x = cepsgram.astype(np.float64)
    if x.shape[1] % 2:
        x = np.concatenate([x, np.zeros((x.shape[0], 1))], 1)
    n = x.shape[1]
    k = np.arange(n)
    j = np.arange(num_cepstra)[:, None]
    basis = np.cos(np.pi * (2 * k + 1) * j / (2.0 * n)) * np.where(j == 0, np.sqrt(1.0 / n), np.sqrt(2.0 / n))
    return (x @ basis.T).astype(f32)


def log_mel(samples, frame_length=320, frame_stride=160, max_time_steps=1599, num_filters=64, sample_rate=16000,
            window="hann", num_cepstra=0):
    """Zero-padded [max_time_steps, n_out] float32 slab for one clip of int16 samples: magnitudes (num_filters == 0),
    log-mel energies, or with ``num_cepstra`` the MFCCs."""
    win = create_window(window, frame_length)
    spec = wav_to_specgram(np.asarray(samples), frame_length, frame_stride, max_time_steps, win)
    n_out = num_cepstra if num_cepstra else num_filters if num_filters else frame_length // 2 + 1
    out = np.zeros((max_time_steps, n_out), f32)
    if num_filters:
        ceps = specgram_to_cepsgram(spec, create_filterbanks(num_filters, frame_length, sample_rate))
        out[:spec.shape[0]] = cepsgram_to_mfcc(ceps, num_cepstra) if num_cepstra else ceps
    else:
        out[:spec.shape[0]] = spec
    return out
