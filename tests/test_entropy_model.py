"""The bookkeeping of the block-parallel entropy kernel, as a model on the CPU (tests/entropy_model.py): what the kernel
counts must be what the stream holds, every piece of the storing pass must start at the right block in a known state."""
import os

import cv2
import numpy as np
import pytest

from tests.entropy_model import simulate
from tests.synth import gradient_image


def test_stream_whose_last_segment_ends_just_before_a_checkpoint(golden_dir):
    blob = open(os.path.join(golden_dir, "entropy_stream_507_segments.jpg"), "rb").read()
    r = simulate(blob)
    assert (r["segment"], r["segments"]) == (176, 507) and r["counted"] == r["total_blocks"] == 6144 and not r["problems"]
    # with a checkpoint allowed past the segment's end, the last segment takes an older run's count: three blocks missing
    old = simulate(blob, checkpoint_past_end=True)
    assert old["counted"] == 6141 and ("segment count", 506, 8, 11) in old["problems"]


@pytest.mark.parametrize("seed", range(3))
def test_random_streams_in_every_sampling_mode_and_block_size(seed):
    rng = np.random.default_rng(100 + seed)
    modes = [cv2.IMWRITE_JPEG_SAMPLING_FACTOR_420, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422, None]
    for k in range(12):
        h, w = int(rng.integers(40, 520)), int(rng.integers(40, 520))
        noise = int(rng.integers(1, 40))
        img = np.clip(gradient_image(rng, h, w).astype(np.int16) + rng.integers(-noise, noise + 1, (h, w, 3)), 0, 255).astype(np.uint8)
        quality = int(rng.choice([60, 75, 90, 95, 100]))
        mode = modes[k % 4]
        if mode is None:
            ok, enc = cv2.imencode(".jpg", cv2.cvtColor(img, cv2.COLOR_BGR2GRAY), [cv2.IMWRITE_JPEG_QUALITY, quality])
        else:
            ok, enc = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, quality, cv2.IMWRITE_JPEG_SAMPLING_FACTOR, mode])
        assert ok
        r = simulate(enc.tobytes(), threads=int(rng.choice([512, 256, 128])))
        assert r["counted"] == r["total_blocks"] and not r["problems"], (seed, k, r)
