"""End-to-end parity of the provider (header parsing and seeded draws on the host; entropy decoding, JPEG back end and
image kernel on the GPU) with the record-level oracle, through the C ABI, on the benchmark configurations at reduced
batch size and on every other stage the provider offers (tests/test_gpu_configs_full.py runs the stated batch sizes)."""
import os
import struct

import numpy as np
import pytest

from tests.pipeline_oracle import PipelineOracle
from tests.synth import gradient_image, jpeg_bytes

pytestmark = pytest.mark.gpu

AUG_C1 = {"type": "image", "crop_enable": True, "center": False, "do_area_scale": True, "scale": [0.08, 1.0],
          "horizontal_distortion": [0.75, 1.3333334], "flip_enable": True}
AUG_C2 = dict(AUG_C1, contrast=[0.6, 1.4], brightness=[0.6, 1.4], saturation=[0.6, 1.4], hue=[-18, 18],
              lighting=[0.0, 0.1], mean=[123.7 / 255, 116.3 / 255, 103.5 / 255], stddev=[58.4 / 255, 57.1 / 255, 57.4 / 255])


def image_records(seed, n):
    rng = np.random.default_rng(seed)
    recs = []
    for _ in range(n):
        h, w = (int(v) for v in rng.integers(256, 513, 2))
        recs.append((jpeg_bytes(gradient_image(rng, h, w), 90), struct.pack("<i", int(rng.integers(0, 1000)))))
    return recs


def make_provider(ctx, cfg):
    from aeon_b200.provider import Provider
    return Provider(ctx, cfg)


def test_config1_uint8_chw_two_batches_bit_exact(ctx):
    cfg = {"batch_size": 16, "random_seed": 1234, "decode_size": 32,
           "etl": [{"type": "image", "height": 224, "width": 224, "channels": 3, "channel_major": True, "output_type": "uint8_t"},
                   {"type": "label", "binary": True}],
           "augmentation": [AUG_C1]}
    prov, orc = make_provider(ctx, cfg), PipelineOracle(cfg)
    recs = image_records(41, 48)
    for b in range(3):  # three batches: the third reuses the slot engines of the first
        chunk = recs[16 * b:16 * (b + 1)]
        got = prov.run_host(chunk)
        want = orc.batch(chunk)
        assert np.array_equal(got["image"], want["image"])
        assert np.array_equal(got["label"].astype(np.int64), want["label"].astype(np.int64))
    st = prov.stats()
    # entropy kernel + JPEG back end + image kernel; the batch and one status word per stream come back
    assert st["launches"] == 3 and st["h2d_bytes"] > 0 and st["d2h_bytes"] == 16 * 3 * 224 * 224 + 16 * 4


def test_config2_photometric_float_device_and_host_outputs(ctx):
    cfg = {"batch_size": 16, "random_seed": 99,
           "etl": [{"type": "image", "height": 224, "width": 224, "output_type": "float", "bgr_to_rgb": True},
                   {"type": "label", "binary": True}],
           "augmentation": [AUG_C2]}
    recs = image_records(42, 16)
    want = PipelineOracle(cfg).batch(recs)
    got_h = make_provider(ctx, cfg).run_host(recs)
    got_d = make_provider(ctx, cfg).run_device(recs)
    for got in (got_h["image"], got_d["image"].cpu().numpy()):
        assert np.abs(got - want["image"]).max() <= 1e-6
    assert np.array_equal(got_d["label"].cpu().numpy().astype(np.int64), want["label"].astype(np.int64))


@pytest.mark.parametrize("stride", [3, 4])
def test_scratch_pixel_stride_does_not_change_results(ctx, stride):
    cfg = {"batch_size": 8, "random_seed": 5, "scratch_pixel_stride": stride,
           "etl": [{"type": "image", "height": 64, "width": 96, "channel_major": False}], "augmentation": [AUG_C2 | {"mean": [], "stddev": []}]}
    recs = [(r[0],) for r in image_records(43, 8)]
    got = make_provider(ctx, cfg).run_host(recs)
    assert np.array_equal(got["image"], PipelineOracle(cfg).batch(recs)["image"])


def test_batch_major_false_gives_transposed_buffers(ctx):
    cfg = {"batch_size": 8, "random_seed": 7, "batch_major": False,
           "etl": [{"type": "image", "height": 32, "width": 40}, {"type": "label", "binary": True}], "augmentation": [AUG_C1]}
    recs = image_records(44, 8)
    got = make_provider(ctx, cfg).run_host(recs)
    want = PipelineOracle(cfg).batch(recs)
    assert got["image"].shape == (3 * 32 * 40, 8)
    assert np.array_equal(got["image"], want["image"].reshape(8, -1).T)
    assert np.array_equal(got["label"].astype(np.int64), want["label"].reshape(8, -1).T.astype(np.int64))


def avi_frames(blob, tmp):
    import cv2
    path = os.path.join(tmp, "clip.avi")
    with open(path, "wb") as f:
        f.write(blob)
    cap = cv2.VideoCapture(path, cv2.CAP_OPENCV_MJPEG)
    frames = []
    while True:
        ok, fr = cap.read()
        if not ok:
            break
        frames.append(fr)
    return frames


def make_avi(rng, tmp, n_frames, w=171, h=128):
    import cv2
    path = os.path.join(tmp, "gen.avi")
    vw = cv2.VideoWriter(path, cv2.CAP_OPENCV_MJPEG, cv2.VideoWriter_fourcc(*"MJPG"), 25, (w, h))
    base = gradient_image(rng, h, w + 3 * n_frames)
    for t in range(n_frames):
        vw.write(np.ascontiguousarray(base[:, 3 * t:3 * t + w]))
    vw.release()
    return open(path, "rb").read()


def test_config4_video_clips(ctx, tmp_path):
    rng = np.random.default_rng(45)
    cfg = {"batch_size": 4, "random_seed": 11,
           "etl": [{"type": "video", "max_frame_count": 16, "frame": {"height": 112, "width": 112, "channels": 3}},
                   {"type": "label", "binary": True}],
           "augmentation": [{"type": "image", "frame": {"type": "image", "scale": [0.875, 0.875], "center": False, "flip_enable": True}}]}
    recs = [(make_avi(rng, str(tmp_path), nf), struct.pack("<i", i)) for i, nf in enumerate((16, 16, 9, 20))]
    got = make_provider(ctx, cfg).run_host(recs)
    want = PipelineOracle(cfg).batch(recs, lambda b: avi_frames(b, str(tmp_path)))
    assert got["video"].shape == (4, 3, 16, 112, 112)
    assert np.array_equal(got["video"], want["video"])
    assert not got["video"][2][:, 9:].any()  # a 9-frame clip is zero-padded to 16


def test_reference_avi_fixture_with_dropped_frame(ctx, golden_dir, tmp_path):
    """aeon test/test_util.cpp:144-184: bb8.avi has 6 index entries, one of length 0 (repeats the previous frame)."""
    blob = open(os.path.join(golden_dir, "bb8.avi"), "rb").read()
    cfg = {"batch_size": 1, "random_seed": 3,
           "etl": [{"type": "video", "max_frame_count": 8, "frame": {"height": 60, "width": 80}}],
           "augmentation": [{"type": "image", "frame": {"type": "image"}}]}
    got = make_provider(ctx, cfg).run_host([(blob,)])["video"][0]
    assert got[:, :6].any() and not got[:, 6:].any()
    frames = avi_frames(blob, str(tmp_path))
    # OpenCV's own reader skips the empty chunk; every decoded picture must appear, in order
    ours = [got[:, t].transpose(1, 2, 0) for t in range(6)]
    k = 0
    for f in frames:
        while k < 6 and not np.array_equal(ours[k], f):
            k += 1
        assert k < 6
    dup = [t for t in range(1, 6) if np.array_equal(ours[t], ours[t - 1])]
    assert len(dup) >= 1


SSD_SAMPLERS = [{"max_sample": 1, "max_trials": 1}] + [
    {"max_sample": 1, "max_trials": 50, "sampler": {"scale": [0.3, 1.0], "aspect_ratio": [0.5, 2.0]}, "sample_constraint": c}
    for c in ({"min_jaccard_overlap": 0.1}, {"min_jaccard_overlap": 0.3}, {"min_jaccard_overlap": 0.5},
              {"min_jaccard_overlap": 0.7}, {"min_jaccard_overlap": 0.9}, {"max_jaccard_overlap": 1.0})]


def ssd_records(seed, n, w=500, h=375):
    import json
    rng = np.random.default_rng(seed)
    names = ["class%02d" % i for i in range(20)]
    recs = []
    for _ in range(n):
        objs = []
        for _ in range(int(rng.integers(1, 9))):
            x0, y0 = int(rng.integers(0, w - 9)), int(rng.integers(0, h - 9))
            objs.append({"name": names[int(rng.integers(0, 20))], "difficult": bool(rng.integers(2)),
                         "bndbox": {"xmin": x0, "ymin": y0, "xmax": int(rng.integers(x0 + 8, w)), "ymax": int(rng.integers(y0 + 8, h))}})
        ann = {"object": objs, "size": {"width": w, "height": h, "depth": 3}}
        recs.append((json.dumps(ann).encode(), jpeg_bytes(gradient_image(rng, h, w), 90)))
    return names, recs


def test_config3_ssd_boxes_and_warped_image(ctx):
    names, recs = ssd_records(47, 16)
    cfg = {"batch_size": 16, "random_seed": 21,
           "etl": [{"type": "localization_ssd", "height": 300, "width": 300, "max_gt_boxes": 64, "class_names": names},
                   {"type": "image", "height": 300, "width": 300, "output_type": "float"}],
           "augmentation": [{"type": "image", "crop_enable": False, "flip_enable": True, "expand_ratio": [1.0, 4.0],
                             "expand_probability": 0.5, "emit_constraint_type": "center", "batch_samplers": SSD_SAMPLERS}]}
    got = make_provider(ctx, cfg).run_host(recs)
    want = PipelineOracle(cfg).batch(recs)
    assert sorted(got) == ["difficult_flag", "gt_box_count", "gt_boxes", "gt_class_count", "image", "image_shape"]
    for key in ("image_shape", "gt_box_count", "gt_class_count", "difficult_flag"):
        assert np.array_equal(got[key], want[key]), key
    assert np.array_equal(got["gt_boxes"], want["gt_boxes"])      # float32 box arithmetic restated op for op
    assert np.array_equal(got["image"], want["image"])            # unnormalised float output of uint8 pixels
    assert got["gt_box_count"].max() >= 1 and (want["image"][:, :, 0, 0] == 0).any()  # some crops start on the zero canvas


def test_errors_surface_with_reference_messages(ctx):
    from aeon_b200._lib import AeonError
    cfg = {"batch_size": 2, "random_seed": 1, "etl": [{"type": "image", "height": 32, "width": 32}], "augmentation": [AUG_C1]}
    prov = make_provider(ctx, cfg)
    good = image_records(46, 1)[0][0]
    with pytest.raises(AeonError, match="size 0"):
        prov.run_host([(good,), (b"",)])
    with pytest.raises(AeonError, match="Decoding image failed"):
        prov.run_host([(good,), (good[:2] + b"\x00" * 50,)])
    assert prov.run_host([(good,), (good,)])["image"].shape == (2, 3, 32, 32)  # still usable afterwards
    with pytest.raises(AeonError, match="not understood"):
        make_provider(ctx, dict(cfg, etl=[{"type": "image", "height": 32, "width": 32, "heigth": 3}]))
    with pytest.raises(AeonError, match="unsupported etl type"):
        make_provider(ctx, dict(cfg, etl=[{"type": "hologram"}]))


def test_config5_audio_log_mel_through_the_provider(ctx):
    from oracle import specgram as ospec
    from tests.test_gpu_specgram import assert_close, synth_clip
    rng = np.random.default_rng(48)
    clips = [synth_clip(rng, s) for s in (1.0, 2.5, 0.8, 1.7)]
    cfg = {"batch_size": 4, "random_seed": 1,
           "etl": [{"type": "audio", "frame_length": 320, "frame_stride": 160, "max_samples": 32000, "num_filters": 64,
                    "sample_rate": 16000, "window_type": "hann", "feature_type": "mfsc"},
                   {"type": "label", "binary": True}]}
    recs = [(c.tobytes(), struct.pack("<i", i)) for i, c in enumerate(clips)]
    got = make_provider(ctx, cfg).run_host(recs)
    steps = (32000 - 320) // 160 + 1
    assert got["audio"].shape == (4, steps, 64)
    for i, c in enumerate(clips):
        assert_close(got["audio"][i], ospec.log_mel(c[:32000], max_time_steps=steps))
    # a RIFF/WAVE container around the same samples gives the same features
    import io
    import wave
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(16000)
        w.writeframes(clips[0].tobytes())
    got2 = make_provider(ctx, cfg).run_host([(buf.getvalue(), recs[0][1])] + recs[1:])
    assert np.array_equal(got2["audio"][0], got["audio"][0])


def test_pipelined_calls_give_the_same_batches_as_blocking_calls(ctx):
    import torch
    cfg = {"batch_size": 16, "random_seed": 77,
           "etl": [{"type": "image", "height": 96, "width": 96, "output_type": "float", "bgr_to_rgb": True},
                   {"type": "label", "binary": True}],
           "augmentation": [AUG_C2]}
    recs = image_records(49, 64)
    blocking = make_provider(ctx, cfg)
    want = [{k: v.copy() for k, v in blocking.run_host(recs[16 * b:16 * b + 16]).items()} for b in range(4)]
    prov = make_provider(ctx, cfg)
    bufs = [{"image": torch.empty((16, 3, 96, 96), dtype=torch.float32).pin_memory().numpy(), "label": np.zeros((16, 1), np.int32)}
            for _ in range(2)]
    prev, got = None, []
    for b in range(4):
        t = prov.submit_host(recs[16 * b:16 * b + 16], bufs[b % 2])
        if prev is not None:
            prov.wait(prev)
            got.append({k: v.copy() for k, v in bufs[(b - 1) % 2].items()})
        prev = t
    prov.wait(prev)
    got.append({k: v.copy() for k, v in bufs[1].items()})
    for b in range(4):
        assert np.array_equal(got[b]["image"], want[b]["image"]) and np.array_equal(got[b]["label"], want[b]["label"])


def test_reference_golden_vectors_through_the_whole_gpu_path(ctx, golden_dir):
    """aeon test/test_provider.cpp:181-261 (validation recipe: resize_short 256, centre crop 224 drawn by make_params)
    and :96-179 (training recipe with the crop box forced by the test): encoded fixture -> host entropy decode ->
    JPEG back-end kernel -> image kernel(s) -> float CHW, against the reference's own golden vectors."""
    blob = open(os.path.join(golden_dir, "img_2112_70.jpg"), "rb").read()
    etl = [{"type": "image", "height": 224, "width": 224, "channels": 3, "output_type": "float", "channel_major": True,
            "bgr_to_rgb": True}]
    aug = {"type": "image", "flip_enable": False, "center": True, "crop_enable": True, "scale": [224 / 256, 224 / 256],
           "interpolation_method": "LINEAR", "mean": [0.485, 0.456, 0.406], "stddev": [0.229, 0.224, 0.225],
           "resize_short_size": 256}
    got = make_provider(ctx, {"batch_size": 1, "random_seed": 5, "etl": etl, "augmentation": [aug]}).run_host([(blob,)])["image"][0]
    gold = np.fromfile(os.path.join(golden_dir, "augment_output_linear_eval.bin"), np.float32).reshape(3, 224, 224)
    assert np.abs(got - gold).max() <= 1e-5          # the reference's own bound for this vector
    # resize_short on a batch of differently sized pictures, against the record-level oracle
    cfg = {"batch_size": 6, "random_seed": 9, "etl": [dict(etl[0], height=64, width=64)],
           "augmentation": [dict(aug, resize_short_size=96, scale=[0.5, 0.9], center=False, flip_enable=True)]}
    recs = [(r[0],) for r in image_records(50, 6)]
    got = make_provider(ctx, cfg).run_host(recs)["image"]
    want = PipelineOracle(cfg).batch(recs)["image"]
    assert np.abs(got - want).max() <= 1e-6


def test_region_decode_and_full_decode_give_identical_batches(ctx):
    cfg = {"batch_size": 16, "random_seed": 31,
           "etl": [{"type": "image", "height": 224, "width": 224, "output_type": "uint8_t"}], "augmentation": [AUG_C2 | {"mean": [], "stddev": []}]}
    recs = [(r[0],) for r in image_records(52, 16)]
    a = make_provider(ctx, dict(cfg, roi_decode=True, entropy_decode="host"))
    b = make_provider(ctx, dict(cfg, roi_decode=False, entropy_decode="host"))
    ga, gb = a.run_host(recs)["image"], b.run_host(recs)["image"]
    assert np.array_equal(ga, gb)
    assert a.stats()["h2d_bytes"] < 0.9 * b.stats()["h2d_bytes"]   # fewer coefficient bytes cross PCIe


def test_device_and_host_entropy_decoding_give_identical_batches(ctx):
    """"entropy_decode": "device" ships the compressed scans and Huffman-decodes on the GPU; "host" ships coefficients."""
    cfg = {"batch_size": 16, "random_seed": 33,
           "etl": [{"type": "image", "height": 224, "width": 224, "output_type": "uint8_t"}], "augmentation": [AUG_C2 | {"mean": [], "stddev": []}]}
    recs = [(r[0],) for r in image_records(53, 16)]
    for roi in (True, False):
        a = make_provider(ctx, dict(cfg, entropy_decode="device", roi_decode=roi))
        b = make_provider(ctx, dict(cfg, entropy_decode="host", roi_decode=roi))
        ga, gb = a.run_host(recs)["image"], b.run_host(recs)["image"]
        assert np.array_equal(ga, gb)
        assert a.stats()["h2d_bytes"] < 0.5 * b.stats()["h2d_bytes"]   # compressed bytes instead of coefficients
        assert a.stats()["launches"] == b.stats()["launches"] + 1


def test_device_entropy_decoding_reports_malformed_streams(ctx):
    cfg = {"batch_size": 2, "random_seed": 34, "entropy_decode": "device",
           "etl": [{"type": "image", "height": 64, "width": 64, "output_type": "uint8_t"}], "augmentation": [{"type": "image"}]}
    good = image_records(54, 1)[0][0]
    sos = good.index(b"\xff\xda")
    broken = good[:sos + 14 + 100] + b"\xff\xd9"      # scan cut short: the decoder runs out of blocks
    p = make_provider(ctx, cfg)
    with pytest.raises(Exception, match="Decoding image failed"):
        p.run_host([(good,), (broken,)])
    out = p.run_host([(good,), (good,)])["image"]      # the provider stays usable
    assert np.array_equal(out[0], out[1])


def test_rotation_angle_through_the_provider_bit_exact(ctx):
    """'angle' (image::rotate before every other step, src/etl_image.cpp:150-151): with the random-area crop, and
    with resize_short + linear-scale crop (the reference sizes an area-scale crop box for the unresized picture)."""
    etl = [{"type": "image", "height": 96, "width": 96, "output_type": "uint8_t"}]
    recs = [(r[0],) for r in image_records(57, 8)]
    linear = {"type": "image", "crop_enable": True, "scale": [0.5, 0.9], "flip_enable": True, "resize_short_size": 128,
              "interpolation_method": "LINEAR"}
    for aug in (dict(AUG_C1, angle=[-20, 20]), dict(linear, angle=[-20, 20])):
        cfg = {"batch_size": 8, "random_seed": 41, "etl": etl, "augmentation": [aug]}
        got = make_provider(ctx, cfg).run_host(recs)["image"]
        want = PipelineOracle(cfg).batch(recs)["image"]
        assert np.array_equal(got, want)


def test_video_frames_with_rotation_and_resize_short(ctx, tmp_path):
    """Every frame of a clip goes through transform_single_image with the clip's parameters (src/etl_video.cpp:56-74),
    so 'angle' and 'resize_short_size' apply per frame, a short clip is still zero-padded."""
    rng = np.random.default_rng(46)
    frame_aug = {"type": "image", "crop_enable": True, "scale": [0.6, 0.9], "flip_enable": True, "angle": [-15, 15],
                 "resize_short_size": 96, "interpolation_method": "LINEAR"}
    cfg = {"batch_size": 3, "random_seed": 12,
           "etl": [{"type": "video", "max_frame_count": 8, "frame": {"height": 64, "width": 64, "channels": 3}}],
           "augmentation": [{"type": "image", "frame": frame_aug}]}
    recs = [(make_avi(rng, str(tmp_path), nf),) for nf in (8, 5, 10)]
    got = make_provider(ctx, cfg).run_host(recs)["video"]
    want = PipelineOracle(cfg).batch(recs, lambda b: avi_frames(b, str(tmp_path)))["video"]
    assert np.array_equal(got, want)
    assert not got[1][:, 5:].any()


def test_progressive_and_baseline_records_in_one_batch(ctx):
    """A progressive file takes the host Huffman decoder (its scans revisit the same coefficients), a baseline one
    the GPU decoder; both end in the same kernels and the batch equals the oracle's."""
    import cv2
    rng = np.random.default_rng(58)
    recs = []
    for i in range(8):
        img = gradient_image(rng, int(rng.integers(200, 400)), int(rng.integers(200, 400)))
        recs.append((jpeg_bytes(img, 90, [cv2.IMWRITE_JPEG_PROGRESSIVE, 1] if i % 2 else []),))
    cfg = {"batch_size": 8, "random_seed": 43, "etl": [{"type": "image", "height": 96, "width": 96, "output_type": "uint8_t"}],
           "augmentation": [AUG_C1]}
    got = make_provider(ctx, cfg).run_host(recs)["image"]
    want = PipelineOracle(cfg).batch(recs)["image"]
    assert np.array_equal(got, want)


def test_exif_orientation_through_the_provider(ctx):
    """cv::imdecode turns the picture by its EXIF orientation before aeon sees it: sizes for make_params, crop, rotation."""
    from tests.synth import with_exif_orientation
    rng = np.random.default_rng(59)
    recs = []
    for o in (1, 2, 3, 4, 5, 6, 7, 8):
        img = gradient_image(rng, int(rng.integers(200, 300)), int(rng.integers(300, 400)))
        recs.append((with_exif_orientation(jpeg_bytes(img, 90), o),))
    etl = [{"type": "image", "height": 96, "width": 96, "output_type": "uint8_t"}]
    for aug in (AUG_C1, dict(AUG_C1, angle=[-20, 20])):
        cfg = {"batch_size": 8, "random_seed": 44, "etl": etl, "augmentation": [aug]}
        got = make_provider(ctx, cfg).run_host(recs)["image"]
        want = PipelineOracle(cfg).batch(recs)["image"]
        assert np.array_equal(got, want)


def test_png_records_lossless_geometry_like_the_reference_tests(ctx):
    """aeon's geometry tests feed PNG-coded "indexed" pictures (pixel value = position, test/test_image.cpp:462-493,
    564-595): with a crop of exactly the output size nothing is resampled, so every output pixel must be the source
    pixel at the drawn crop offset, flipped when the draw says so; and the batch must equal the oracle's."""
    import cv2
    h, w = 200, 256
    yy, xx = np.mgrid[0:h, 0:w]
    indexed = np.dstack([xx, yy, (xx + yy) % 256]).astype(np.uint8)
    blob = cv2.imencode(".png", indexed)[1].tobytes()
    cfg = {"batch_size": 4, "random_seed": 71, "etl": [{"type": "image", "height": 100, "width": 128, "output_type": "uint8_t",
                                                         "channel_major": False}],
           "augmentation": [{"type": "image", "crop_enable": True, "scale": [0.5, 0.5], "center": False, "flip_enable": True}]}
    recs = [(blob,)] * 4
    got = make_provider(ctx, cfg).run_host(recs)["image"]
    want = PipelineOracle(cfg).batch(recs)["image"]
    assert np.array_equal(got, want)
    for img in got:                                           # 100 x 128 x 3, values are source coordinates
        x0 = int(min(img[0, 0, 0], img[0, -1, 0]))
        y0 = int(img[0, 0, 1])
        window = indexed[y0:y0 + 100, x0:x0 + 128]
        assert np.array_equal(img, window) or np.array_equal(img, window[:, ::-1])


def test_png_and_jpeg_records_in_one_batch(ctx):
    import cv2
    rng = np.random.default_rng(72)
    recs = []
    for i in range(8):
        img = gradient_image(rng, int(rng.integers(200, 400)), int(rng.integers(200, 400)))
        recs.append((cv2.imencode(".png", img)[1].tobytes() if i % 2 else jpeg_bytes(img, 90),))
    cfg = {"batch_size": 8, "random_seed": 45, "etl": [{"type": "image", "height": 96, "width": 96, "output_type": "float"}],
           "augmentation": [dict(AUG_C2, angle=[-10, 10])]}
    got = make_provider(ctx, cfg).run_host(recs)["image"]
    want = PipelineOracle(cfg).batch(recs)["image"]
    assert np.abs(got - want).max() <= 1e-6


def test_one_channel_output_from_grey_png_and_from_jpeg_luma(ctx):
    """"channels": 1 makes aeon call cv::imdecode(..., GRAYSCALE) (src/etl_image.cpp:63-99): a grey PNG as it is (the MNIST
    shape), a colour JPEG as its luma plane; geometry, contrast, lighting and standardisation act on the one channel."""
    import cv2
    rng = np.random.default_rng(73)
    digits = [cv2.imencode(".png", rng.integers(0, 256, (28, 28), dtype=np.uint8))[1].tobytes() for _ in range(8)]
    cfg = {"batch_size": 8, "random_seed": 46, "etl": [{"type": "image", "height": 28, "width": 28, "channels": 1, "output_type": "uint8_t"}],
           "augmentation": [{"type": "image", "flip_enable": True, "crop_enable": False}]}
    got = make_provider(ctx, cfg).run_host([(b,) for b in digits])["image"]
    assert got.shape == (8, 1, 28, 28)
    assert np.array_equal(got, PipelineOracle(cfg).batch([(b,) for b in digits])["image"])
    photos = [(jpeg_bytes(gradient_image(rng, int(rng.integers(200, 400)), int(rng.integers(200, 400))), 90),) for _ in range(8)]
    for channel_major in (True, False):
        cfg = {"batch_size": 8, "random_seed": 47,
               "etl": [{"type": "image", "height": 64, "width": 80, "channels": 1, "output_type": "float", "channel_major": channel_major}],
               "augmentation": [dict(AUG_C1, contrast=[0.6, 1.4], lighting=[0.0, 0.1], angle=[-10, 10], mean=[0.45], stddev=[0.22])]}
        got = make_provider(ctx, cfg).run_host(photos)["image"]
        want = PipelineOracle(cfg).batch(photos)["image"]
        assert got.shape == ((8, 1, 64, 80) if channel_major else (8, 64, 80, 1))
        assert np.abs(got - want).max() <= 1e-6
    bad = dict(cfg, augmentation=[dict(AUG_C1, brightness=[0.5, 0.6])])
    with pytest.raises(Exception, match="3-channel"):
        make_provider(ctx, bad).run_host(photos)


@pytest.mark.parametrize("method", ["AREA", "CUBIC", "LANCZOS4"])
def test_area_cubic_and_lanczos_interpolation_through_the_provider(ctx, tmp_path, method):
    """interpolation_method "AREA" / "CUBIC" / "LANCZOS4" (cv::resize): crops that shrink, grow and mix, resize_short, video frames."""
    recs = [(r[0],) for r in image_records(60, 8)]
    etl = [{"type": "image", "height": 96, "width": 96, "output_type": "uint8_t"}]
    configs = [dict(AUG_C1, interpolation_method=method),                                        # mostly shrinking
               dict(AUG_C1, interpolation_method=method, scale=[0.02, 0.08]),                    # small crops: enlarging
               {"type": "image", "crop_enable": True, "scale": [0.5, 0.9], "flip_enable": True, "resize_short_size": 128,
                "interpolation_method": method, "angle": [-10, 10]}]
    for aug in configs:
        cfg = {"batch_size": 8, "random_seed": 48, "etl": etl, "augmentation": [aug]}
        got = make_provider(ctx, cfg).run_host(recs)["image"]
        want = PipelineOracle(cfg).batch(recs)["image"]
        assert np.array_equal(got, want)
    rng = np.random.default_rng(61)
    frame_aug = {"type": "image", "crop_enable": True, "scale": [0.6, 0.9], "flip_enable": True, "interpolation_method": method}
    cfg = {"batch_size": 2, "random_seed": 13,
           "etl": [{"type": "video", "max_frame_count": 6, "frame": {"height": 48, "width": 64, "channels": 3}}],
           "augmentation": [{"type": "image", "frame": frame_aug}]}
    clips = [(make_avi(rng, str(tmp_path), nf),) for nf in (6, 4)]
    got = make_provider(ctx, cfg).run_host(clips)["video"]
    want = PipelineOracle(cfg).batch(clips, lambda b: avi_frames(b, str(tmp_path)))["video"]
    assert np.array_equal(got, want)


def test_crop_disabled_branch_fixed_aspect_ratio_scaling_factor_and_padding(ctx):
    """make_params with crop_enable false (src/augment_image.cpp:132-152): the picture is scaled to fit (or by
    fixed_scaling_factor) and written top-left into a zero slot (fixed_aspect_ratio, src/etl_image.cpp:264-315); with
    'padding' a window of the picture's size is cut from the picture framed in black (src/image.cpp:77-91)."""
    rng = np.random.default_rng(74)
    recs = [(jpeg_bytes(gradient_image(rng, int(rng.integers(120, 260)), int(rng.integers(120, 260))), 90),) for _ in range(8)]
    etl = [{"type": "image", "height": 128, "width": 160, "output_type": "uint8_t"}]
    for aug in ({"type": "image", "crop_enable": False, "fixed_aspect_ratio": True, "flip_enable": True},
                {"type": "image", "crop_enable": False, "fixed_aspect_ratio": True, "fixed_scaling_factor": 0.4}):
        cfg = {"batch_size": 8, "random_seed": 49, "etl": etl, "augmentation": [aug]}
        got = make_provider(ctx, cfg).run_host(recs)["image"]
        want = PipelineOracle(cfg).batch(recs)["image"]
        assert np.array_equal(got, want)
        assert (got == 0).all(axis=1).any()                       # part of every slot is the zero fill
    same = [(jpeg_bytes(gradient_image(rng, 96, 96), 90),) for _ in range(8)]
    cfg = {"batch_size": 8, "random_seed": 50, "etl": [{"type": "image", "height": 96, "width": 96, "output_type": "uint8_t"}],
           "augmentation": [{"type": "image", "crop_enable": False, "padding": 8, "flip_enable": True}]}
    got = make_provider(ctx, cfg).run_host(same)["image"]
    assert np.array_equal(got, PipelineOracle(cfg).batch(same)["image"])


def mask_png(rng, h, w, colour=False, interlaced=False):
    """A class-index mask with large flat regions, PNG coded (what segmentation data sets ship)."""
    import cv2
    from tests.test_host_png import write_png
    yy, xx = np.mgrid[0:h, 0:w]
    m = ((yy // int(rng.integers(9, 40)) + xx // int(rng.integers(9, 40))) % 21).astype(np.uint8)
    if colour:
        m = np.dstack([m * 12, 255 - m * 7, m * 3]).astype(np.uint8)
        return cv2.imencode(".png", m)[1].tobytes()
    if interlaced:
        return write_png(m[..., None], 0, 8, interlaced=True)
    return cv2.imencode(".png", m)[1].tobytes()


def test_image_and_pixelmask_share_the_geometry(ctx):
    """provider type image,pixelmask (src/provider.cpp:353-394, doc/source/provider_pixelmask.rst): the mask follows the
    image's rotation, crop box and flip, without interpolation and without the photometric steps; int32 and uint8
    outputs; PNG masks (grey, colour read as one channel, interlaced) and a JPEG mask (its luma plane)."""
    rng = np.random.default_rng(71)
    recs = []
    for i in range(8):
        h, w = int(rng.integers(200, 320)), int(rng.integers(200, 320))
        img = jpeg_bytes(gradient_image(rng, h, w), 90)
        if i == 6:
            mask = jpeg_bytes(gradient_image(rng, h, w), 95)
        else:
            mask = mask_png(rng, h, w, colour=(i == 5), interlaced=(i == 4))
        recs.append((img, mask))
    for out_type, aug in (("int32_t", dict(AUG_C2, angle=[-25, 25])), ("uint8_t", AUG_C1),
                          ("float", {"type": "image", "crop_enable": True, "scale": [0.6, 0.9], "flip_enable": True, "angle": [5, 40]})):
        aug = {k: v for k, v in aug.items() if k not in ("mean", "stddev")}
        cfg = {"batch_size": 8, "random_seed": 77,
               "etl": [{"type": "image", "height": 96, "width": 112, "output_type": "uint8_t"},
                       {"type": "pixelmask", "height": 96, "width": 112, "channels": 1, "output_type": out_type}],
               "augmentation": [aug]}
        got = make_provider(ctx, cfg).run_host(recs)
        want = PipelineOracle(cfg).batch(recs)
        assert got["pixelmask"].shape == (8, 1, 96, 112) and got["pixelmask"].dtype == want["pixelmask"].dtype
        assert np.array_equal(got["image"], want["image"])
        assert np.array_equal(got["pixelmask"], want["pixelmask"])


def test_pixelmask_alone_and_its_errors(ctx):
    """A pixelmask stage on its own draws the parameters itself; the configuration needs one channel; an empty record and
    a crop box that leaves the mask are errors (src/provider.cpp:372-377; cv::Mat refuses the window)."""
    from aeon_b200._lib import AeonError
    rng = np.random.default_rng(72)
    recs = [(mask_png(rng, 120 + 7 * i, 150 + 3 * i),) for i in range(4)]
    cfg = {"batch_size": 4, "random_seed": 5, "etl": [{"type": "pixelmask", "height": 64, "width": 64, "channels": 1}],
           "augmentation": [{"type": "image", "crop_enable": True, "scale": [0.5, 0.8], "flip_enable": True}]}
    got = make_provider(ctx, cfg).run_host(recs)["pixelmask"]
    assert np.array_equal(got, PipelineOracle(cfg).batch(recs)["pixelmask"])
    with pytest.raises(AeonError, match="channels"):
        make_provider(ctx, dict(cfg, etl=[{"type": "pixelmask", "height": 64, "width": 64}]))
    with pytest.raises(AeonError, match="received pixelmask with size 0"):
        make_provider(ctx, cfg).run_host([(b"",)] * 4)
    two = dict(cfg, etl=[{"type": "image", "height": 64, "width": 64}, cfg["etl"][0]])
    small = [(jpeg_bytes(gradient_image(rng, 300, 300), 90), mask_png(rng, 40, 40)) for _ in range(4)]
    with pytest.raises(AeonError, match="crop box"):
        make_provider(ctx, two).run_host(small)


def test_outputs_too_large_for_eight_bands(ctx):
    """A 1000 x 800 output (detection-sized) does not fit eight on-chip bands: it runs as more, independent bands, which
    covers everything but the contrast step (that one needs the whole-image mean inside one cluster)."""
    from aeon_b200._lib import AeonError
    etl = [{"type": "image", "height": 800, "width": 1000, "output_type": "uint8_t", "channel_major": False}]
    recs = [(r[0],) for r in image_records(63, 4)]
    aug = {"type": "image", "crop_enable": True, "scale": [0.6, 0.9], "flip_enable": True, "brightness": [0.7, 1.3],
           "saturation": [0.7, 1.3], "hue": [-10, 10], "lighting": [0.0, 0.1]}
    cfg = {"batch_size": 4, "random_seed": 21, "etl": etl, "augmentation": [aug]}
    got = make_provider(ctx, cfg).run_host(recs)["image"]
    assert np.array_equal(got, PipelineOracle(cfg).batch(recs)["image"])
    cfg = {"batch_size": 4, "random_seed": 21, "etl": etl, "augmentation": [dict(aug, contrast=[0.6, 0.8])]}
    with pytest.raises(AeonError, match="contrast"):
        make_provider(ctx, cfg).run_host(recs)


def test_image_and_boundingbox_stage(ctx):
    """provider type image,boundingbox (src/provider.cpp:399-441): the record's boxes go through the same crop, flip and
    rescale as the picture (boundingbox::transformer::transform_box) and fill the first max_bbox_count rows of four floats
    of a buffer declared as {max_bbox_count, 16} elements; a rotated record is an error."""
    import json
    from aeon_b200._lib import AeonError
    rng = np.random.default_rng(91)
    names = ["cat", "dog"]
    recs = []
    for i in range(6):
        h, w = int(rng.integers(150, 260)), int(rng.integers(200, 320))
        objs = []
        for _ in range(int(rng.integers(0, 7))):
            x0, y0 = int(rng.integers(0, w - 50)), int(rng.integers(0, h - 50))
            objs.append({"bndbox": {"xmin": x0, "ymin": y0, "xmax": x0 + int(rng.integers(5, 49)), "ymax": y0 + int(rng.integers(5, 49))},
                         "name": names[int(rng.integers(2))]})
        recs.append((jpeg_bytes(gradient_image(rng, h, w), 90),
                     json.dumps({"object": objs, "size": {"width": w, "height": h, "depth": 3}}).encode()))
    for out_type in ("float", "uint8_t"):
        cfg = {"batch_size": 6, "random_seed": 31,
               "etl": [{"type": "image", "height": 96, "width": 128},
                       {"type": "boundingbox", "height": 96, "width": 128, "max_bbox_count": 4, "class_names": names, "output_type": out_type}],
               "augmentation": [{"type": "image", "crop_enable": True, "scale": [0.5, 0.9], "flip_enable": True, "center": False}]}
        got = make_provider(ctx, cfg).run_host(recs)
        want = PipelineOracle(cfg).batch(recs)
        assert got["boundingbox"].shape == (6, 4, 16) and got["boundingbox"].dtype == want["boundingbox"].dtype
        assert np.array_equal(got["image"], want["image"])
        assert np.array_equal(got["boundingbox"].view(np.uint8), want["boundingbox"].view(np.uint8))
        assert got["boundingbox"].view(np.uint8).any()
    cfg["augmentation"][0]["angle"] = [5, 10]
    with pytest.raises(AeonError, match="angle"):
        make_provider(ctx, cfg).run_host(recs)


def test_blob_stage_copies_bytes_next_to_an_image(ctx):
    """provider::blob (aeon src/provider.cpp:445-470): the element's bytes land unchanged in a buffer of output_count elements."""
    from aeon_b200._lib import AeonError
    cfg = {"batch_size": 4, "random_seed": 3,
           "etl": [{"type": "image", "height": 32, "width": 32}, {"type": "blob", "output_count": 5, "output_type": "float"}],
           "augmentation": [AUG_C1]}
    rng = np.random.default_rng(50)
    vecs = [rng.normal(size=5).astype(np.float32) for _ in range(4)]
    recs = [(image_records(51 + i, 1)[0][0], v.tobytes()) for i, v in enumerate(vecs)]
    got = make_provider(ctx, cfg).run_host(recs)
    assert got["blob"].shape == (4, 5) and got["blob"].dtype == np.float32
    assert np.array_equal(got["blob"], np.stack(vecs))
    assert np.array_equal(got["image"], PipelineOracle({**cfg, "etl": cfg["etl"][:1]}).batch([(r[0],) for r in recs])["image"])
    with pytest.raises(AeonError, match="does not fit"):
        make_provider(ctx, cfg).run_host([(recs[0][0], b"x" * 21)] + recs[1:])
    with pytest.raises(AeonError, match="received blob with size 0"):
        make_provider(ctx, cfg).run_host([(recs[0][0], b"")] + recs[1:])


def test_seven_batches_in_flight_match_blocking_calls(ctx):
    """The caller plans batch t+1 while the provider's driver thread stages and launches batch t: submitting seven batches
    before waiting for any must give what seven blocking calls give (same draws in the same record order, no buffer of a
    batch reused before its kernels and copies have finished)."""
    import torch
    cfg = {"batch_size": 16, "random_seed": 5, "decode_size": 32,
           "etl": [{"type": "image", "height": 64, "width": 80, "output_type": "float", "bgr_to_rgb": True},
                   {"type": "label", "binary": True}],
           "augmentation": [AUG_C2]}
    recs = image_records(61, 7 * 16)
    blocking = make_provider(ctx, cfg)
    want = [{k: v.copy() for k, v in blocking.run_host(recs[16 * b:16 * b + 16]).items()} for b in range(7)]
    for to_device in (False, True):
        prov = make_provider(ctx, cfg)
        if to_device:
            bufs = [{"image": torch.full((16, 3, 64, 80), -1.0, dtype=torch.float32, device="cuda:%d" % ctx.device),
                     "label": torch.full((16, 1), -1, dtype=torch.int32, device="cuda:%d" % ctx.device)} for _ in range(7)]
            tickets = [prov.submit_device(recs[16 * b:16 * b + 16], bufs[b]) for b in range(7)]
        else:
            bufs = [{"image": torch.full((16, 3, 64, 80), -1.0, dtype=torch.float32).pin_memory().numpy(),
                     "label": np.full((16, 1), -1, np.int32)} for _ in range(7)]
            tickets = [prov.submit_host(recs[16 * b:16 * b + 16], bufs[b]) for b in range(7)]
        for b in (3, 0, 1, 2, 6, 5, 4):  # any order
            prov.wait(tickets[b])
        for b in range(7):
            img = bufs[b]["image"].cpu().numpy() if to_device else bufs[b]["image"]
            lbl = bufs[b]["label"].cpu().numpy() if to_device else bufs[b]["label"]
            assert np.array_equal(img, want[b]["image"]) and np.array_equal(lbl, want[b]["label"]), (to_device, b)


def test_errors_of_pipelined_batches(ctx):
    """What the calling thread finds while planning (an empty record) fails the submission itself and uses up no ticket; what
    the driver thread or the GPU finds (a scan that ends early) is reported when that batch is waited for; the batches
    around it are delivered and the provider stays usable."""
    import torch
    from aeon_b200._lib import AeonError
    cfg = {"batch_size": 2, "random_seed": 34, "etl": [{"type": "image", "height": 64, "width": 64, "output_type": "uint8_t"}],
           "augmentation": [{"type": "image"}]}
    good = image_records(62, 1)[0][0]
    sos = good.index(b"\xff\xda")
    broken = good[:sos + 14 + 100] + b"\xff\xd9"
    prov = make_provider(ctx, cfg)
    want = prov.run_host([(good,), (good,)])["image"].copy()
    bufs = [{"image": torch.zeros((2, 3, 64, 64), dtype=torch.uint8).pin_memory().numpy()} for _ in range(3)]
    t0 = prov.submit_host([(good,), (good,)], bufs[0])
    with pytest.raises(AeonError, match="size 0"):
        prov.submit_host([(good,), (b"",)], bufs[1])
    t1 = prov.submit_host([(good,), (broken,)], bufs[1])
    t2 = prov.submit_host([(good,), (good,)], bufs[2])
    assert (t1, t2) == (t0 + 1, t0 + 2)
    prov.wait(t0)
    with pytest.raises(AeonError, match="Decoding image failed"):
        prov.wait(t1)
    prov.wait(t2)
    assert np.array_equal(bufs[0]["image"], want) and np.array_equal(bufs[2]["image"], want)
    assert np.array_equal(prov.run_host([(good,), (good,)])["image"], want)
