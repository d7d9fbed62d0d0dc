"""The DataLoader surface (aeon test/test_dataloader.py, test/test_loader.cpp): length, iteration modes,
reset, wrap-around, broken records, node sharding, and batch contents against the record-level oracle."""
import os

import numpy as np
import pytest

from tests.pipeline_oracle import PipelineOracle
from tests.synth import gradient_image, jpeg_bytes

pytestmark = pytest.mark.gpu

AUG = {"type": "image", "crop_enable": True, "center": False, "do_area_scale": True, "scale": [0.3, 1.0],
       "horizontal_distortion": [0.75, 1.3333334], "flip_enable": True, "contrast": [0.8, 1.2], "hue": [-5, 5]}


@pytest.fixture(scope="module")
def dataset(tmp_path_factory):
    root = tmp_path_factory.mktemp("ds")
    rng = np.random.default_rng(51)
    lines = ["@FILE\tASCII_INT"]
    recs = []
    for i in range(20):
        blob = jpeg_bytes(gradient_image(rng, int(rng.integers(40, 90)), int(rng.integers(40, 90))), 90)
        with open(root / ("img_%02d.jpg" % i), "wb") as f:
            f.write(blob)
        lines.append("img_%02d.jpg\t%d" % (i, 100 + i))
        recs.append((blob, np.int32(100 + i).tobytes()))
    (root / "manifest.tsv").write_text("\n".join(lines) + "\n# a comment line\n")
    return root, recs


def config(root, **kw):
    cfg = {"manifest_filename": str(root / "manifest.tsv"), "manifest_root": str(root), "batch_size": 8, "random_seed": 1234,
           "cpu_list": "0", "iteration_mode": "ONCE",
           "etl": [{"type": "image", "height": 32, "width": 32, "channels": 3, "channel_major": True, "output_type": "uint8_t"},
                   {"type": "label", "binary": True}],
           "augmentation": [AUG]}
    cfg.update(kw)
    return cfg


def test_once_mode_wraps_the_last_batch_and_matches_the_oracle(ctx, dataset):
    from aeon_b200 import DataLoader
    root, recs = dataset
    cfg = config(root)
    dl = DataLoader(config=cfg)
    assert len(dl) == 20 and dl.ndata == 20 and dl.batch_size == 8
    assert dl.axes_info["image"] == {"channels": 3, "height": 32, "width": 32}
    orc = PipelineOracle(dict(cfg, decode_size=8))
    stream = recs + recs            # the record stream wraps to the start of the data set
    seen = 0
    for b, batch in enumerate(dl):
        d = dict(batch)
        assert [n for n, _ in batch] == ["image", "label"]
        want = orc.batch(stream[8 * b:8 * b + 8])
        assert np.array_equal(d["image"], want["image"])
        assert d["label"].ravel().tolist() == [100 + (8 * b + i) % 20 for i in range(8)]
        seen += 1
    assert seen == 3
    with pytest.raises(StopIteration):
        next(dl)
    dl.reset()
    assert dict(next(dl))["label"].ravel().tolist() == list(range(100, 108))
    dl.close()


def test_count_and_infinite_modes(ctx, dataset):
    from aeon_b200 import DataLoader
    root, _ = dataset
    dl = DataLoader(config=config(root, iteration_mode="COUNT", iteration_mode_count=5))
    assert sum(1 for _ in dl) == 5
    dl.close()
    dl = DataLoader(config=config(root, iteration_mode="INFINITE"))
    labels = [dict(next(dl))["label"].ravel()[0] for _ in range(7)]
    assert labels == [100 + (8 * b) % 20 for b in range(7)]
    dl.close()


def test_device_output_and_batch_major_false(ctx, dataset):
    import torch
    from aeon_b200 import DataLoader
    root, recs = dataset
    # batches are views of loader-owned buffers: the loaders must outlive them (as in aeon)
    dl_host = DataLoader(config=config(root))
    dl_dev = DataLoader(config=config(root, device_output=True))
    dl_tr = DataLoader(config=config(root, batch_major=False))
    host, dev, tr = dict(next(dl_host)), dict(next(dl_dev)), dict(next(dl_tr))
    assert dev["image"].is_cuda and torch.equal(dev["image"].cpu(), torch.from_numpy(host["image"].copy()))
    assert tr["image"].shape == (3 * 32 * 32, 8) and np.array_equal(tr["image"], host["image"].reshape(8, -1).T)
    for d in (dl_host, dl_dev, dl_tr):
        d.close()


def test_node_sharding_gives_interleaved_batches(ctx, dataset):
    from aeon_b200 import DataLoader
    root, _ = dataset
    got = []
    for node in range(2):
        dl = DataLoader(config=config(root, batch_size=4, node_id=node, node_count=2))
        assert dl.ndata == 10
        got.append([dict(b)["label"].ravel().tolist() for b in dl][:2])
        dl.close()
    assert got[0][0] == [100, 101, 102, 103] and got[1][0] == [104, 105, 106, 107] and got[0][1] == [108, 109, 110, 111]


def test_errors(ctx, dataset, tmp_path):
    from aeon_b200 import DataLoader
    root, _ = dataset
    with pytest.raises(RuntimeError, match="doesn't exist"):
        DataLoader(config=config(root, manifest_filename=str(tmp_path / "none.tsv")))
    with pytest.raises(RuntimeError, match="not understood"):
        DataLoader(config=config(root, batch_sise=4))
    with pytest.raises(RuntimeError, match="iteration_mode"):
        DataLoader(config=config(root, iteration_mode="TWICE"))
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "a.jpg").write_bytes(b"this is not a jpeg")
    (bad / "manifest.tsv").write_text("@FILE\tASCII_INT\na.jpg\t1\n")
    dl = DataLoader(config=config(bad, batch_size=1))
    with pytest.raises(RuntimeError, match="Decoding image failed"):
        next(dl)
    (bad / "empty.tsv").write_text("@FILE\tASCII_INT\n")
    with pytest.raises(RuntimeError, match="manifest file is empty"):
        DataLoader(config=config(bad, manifest_filename=str(bad / "empty.tsv")))


def test_segmentation_and_detection_manifests_through_the_loader(ctx, tmp_path):
    """image,pixelmask and image,localization_rcnn data sets (doc/source/provider_pixelmask.rst, provider_localization_rcnn):
    two files per manifest line; every buffer of a batch equals the record-level oracle's."""
    import cv2
    import json
    from aeon_b200 import DataLoader
    from tests.test_gpu_rcnn import compare_rcnn
    rng = np.random.default_rng(52)
    names = ["car", "person", "dog"]
    lines_m, lines_d, recs_m, recs_d = ["@FILE\tFILE"], ["@FILE\tFILE"], [], []
    for i in range(6):
        h, w = int(rng.integers(120, 200)), int(rng.integers(150, 260))
        img = jpeg_bytes(gradient_image(rng, h, w), 90)
        yy, xx = np.mgrid[0:h, 0:w]
        mask = cv2.imencode(".png", ((yy // 17 + xx // 23) % 5).astype(np.uint8))[1].tobytes()
        objs = []
        for _ in range(int(rng.integers(1, 5))):
            x0, y0 = int(rng.integers(0, w - 40)), int(rng.integers(0, h - 40))
            objs.append({"bndbox": {"xmin": x0, "ymin": y0, "xmax": x0 + int(rng.integers(20, 39)), "ymax": y0 + int(rng.integers(20, 39))},
                         "name": names[int(rng.integers(3))], "difficult": bool(rng.integers(2))})
        ann = json.dumps({"object": objs, "size": {"width": w, "height": h, "depth": 3}}).encode()
        for name, blob in (("i%d.jpg" % i, img), ("m%d.png" % i, mask), ("a%d.json" % i, ann)):
            (tmp_path / name).write_bytes(blob)
        lines_m.append("i%d.jpg\tm%d.png" % (i, i))
        lines_d.append("i%d.jpg\ta%d.json" % (i, i))
        recs_m.append((img, mask))
        recs_d.append((img, ann))
    (tmp_path / "seg.tsv").write_text("\n".join(lines_m) + "\n")
    (tmp_path / "det.tsv").write_text("\n".join(lines_d) + "\n")
    base = {"manifest_root": str(tmp_path), "batch_size": 3, "random_seed": 7, "cpu_list": "0", "iteration_mode": "ONCE"}
    seg = dict(base, manifest_filename=str(tmp_path / "seg.tsv"),
               etl=[{"type": "image", "height": 64, "width": 80}, {"type": "pixelmask", "height": 64, "width": 80, "channels": 1}],
               augmentation=[{"type": "image", "crop_enable": True, "scale": [0.5, 0.9], "flip_enable": True, "angle": [-10, 10]}])
    dl = DataLoader(config=seg)
    orc = PipelineOracle(dict(seg, decode_size=9))   # one worker thread: 8 slots rounded up to whole batches (src/loader.cpp:159-164)
    for b, batch in enumerate(dl):
        d, want = dict(batch), orc.batch(recs_m[3 * b:3 * b + 3])
        assert [n for n, _ in batch] == ["image", "pixelmask"]
        assert np.array_equal(d["image"], want["image"]) and np.array_equal(d["pixelmask"], want["pixelmask"])
    dl.close()
    det = dict(base, manifest_filename=str(tmp_path / "det.tsv"),
               etl=[{"type": "image", "height": 320, "width": 400},
                    {"type": "localization_rcnn", "height": 320, "width": 400, "class_names": names, "debug_deterministic": True,
                     "rois_per_image": 64}],
               augmentation=[{"type": "image", "crop_enable": False, "fixed_aspect_ratio": True, "flip_enable": True}])
    dl = DataLoader(config=det)
    oracle_cfg = dict(det, decode_size=9, etl=[det["etl"][0], {k: v for k, v in det["etl"][1].items() if k != "debug_deterministic"}])
    orc = PipelineOracle(oracle_cfg)
    for b, batch in enumerate(dl):
        d, want = dict(batch), orc.batch(recs_d[3 * b:3 * b + 3])
        assert len(batch) == 11 and batch[0][0] == "image" and batch[1][0] == "bbtargets"
        assert np.array_equal(d["image"], want["image"])
        compare_rcnn(d, want)
    dl.close()
