"""localization_rcnn anchor labelling on the GPU against the oracle: labels and best-box indices bit-exact."""
import json

import numpy as np
import pytest

from oracle import rcnn as orcnn
from tests.test_oracle_rcnn import golden, run_golden

pytestmark = pytest.mark.gpu


def oracle_labels(anchors, gt, im_size, neg=0.3, pos=0.7):
    """Labels / best box over all anchors as transformer::transform leaves them (src/etl_localization_rcnn.cpp:118-208)."""
    from oracle import ssd as ossd
    labels = np.full(len(anchors), -1, np.int8)
    best = np.zeros(len(anchors), np.int16)
    inside = np.nonzero((anchors[:, 0] >= 0) & (anchors[:, 1] >= 0) & (anchors[:, 2] < im_size[0]) & (anchors[:, 3] < im_size[1]))[0]
    if len(gt):
        boxes = [ossd.Box(*row) for row in gt]
        lab, arg = orcnn.label_anchors(orcnn.bbox_overlaps(anchors[inside], boxes), neg, pos)
        labels[inside], best[inside] = lab, arg
    return labels, best


def test_reference_annotation_labels_and_sampling(ctx):
    """The reference's loader test record (test/test_localization_rcnn.cpp:595-1213) through the GPU pass: labels equal the
    oracle's, and deterministic sampling on them gives the reference's foreground / background indices."""
    from aeon_b200 import kernels as K
    g = golden()
    cfg, anchors, r = run_golden(g)
    gt = np.array([[b.xmin, b.ymin, b.xmax, b.ymax] for b in r.gt_boxes], np.float32)
    table = K.rcnn_anchors(K.rcnn_config(1000, 1000))
    assert np.array_equal(table, anchors)
    labels, best = K.rcnn_label_batch(ctx, table, [gt, gt[:0], gt[:1]], [r.im_size] * 3)
    assert np.array_equal(labels[0], r.labels.astype(np.int8))
    assert (labels[1] == -1).all() and (best[1] == 0).all()
    assert orcnn.sample_anchors(labels[0]) == g["fg_idx"] + g["bg_idx"]
    want_l, want_b = oracle_labels(anchors, gt, r.im_size)
    assert np.array_equal(labels[0], want_l) and np.array_equal(best[0], want_b)
    want_l, want_b = oracle_labels(anchors, gt[:1], r.im_size)
    assert np.array_equal(labels[2], want_l) and np.array_equal(best[2], want_b)


def test_random_boxes_thresholds_and_a_box_nobody_overlaps(ctx):
    from aeon_b200 import kernels as K
    rng = np.random.default_rng(81)
    kw = {"width": 600, "height": 450}
    anchors = K.rcnn_anchors(K.rcnn_config(**kw))
    gts, sizes = [], []
    for i in range(12):
        w, h = int(rng.integers(300, 601)), int(rng.integers(250, 451))
        k = int(rng.integers(1, 65)) if i else 300
        x0, y0 = rng.uniform(0, w - 20, k), rng.uniform(0, h - 20, k)
        bw, bh = rng.uniform(8, w / 1.5, k), rng.uniform(8, h / 1.5, k)
        g = np.stack([x0, y0, np.minimum(x0 + bw, w - 1), np.minimum(y0 + bh, h - 1)], 1).astype(np.float32)
        if i == 3:
            g[0] = (5000, 5000, 5100, 5100)      # outside every anchor: its best overlap is 0, which every anchor "equals"
        if i == 4:
            g = np.round(g)                      # whole-pixel boxes: exact ties between anchors
        gts.append(g)
        sizes.append((w, h))
    for neg, pos in ((0.3, 0.7), (0.1, 0.5), (0.0, 1.0)):
        labels, best = K.rcnn_label_batch(ctx, anchors, gts, sizes, neg, pos)
        for i, (g, s) in enumerate(zip(gts, sizes)):
            want_l, want_b = oracle_labels(anchors, g, s, neg, pos)
            assert np.array_equal(labels[i], want_l), (i, neg, pos)
            assert np.array_equal(best[i], want_b), (i, neg, pos)
    labels3, _ = K.rcnn_label_batch(ctx, anchors, [gts[3]], [sizes[3]])
    inside = (anchors[:, 0] >= 0) & (anchors[:, 1] >= 0) & (anchors[:, 2] < sizes[3][0]) & (anchors[:, 3] < sizes[3][1])
    assert (labels3[0][inside] == 1).all() and (labels3[0][~inside] == -1).all()


def test_anchor_table_beyond_the_16_bit_index_list(ctx):
    """More than 65 535 anchors (a 2000 x 1500 configuration): the kernel's plain strided walk."""
    from aeon_b200 import kernels as K
    rng = np.random.default_rng(82)
    anchors = K.rcnn_anchors(K.rcnn_config(2000, 1500))
    assert len(anchors) == 9 * 125 * 93
    gts = []
    for k in (5, 40):
        x0, y0 = rng.uniform(0, 1500, k), rng.uniform(0, 1100, k)
        gts.append(np.stack([x0, y0, x0 + rng.uniform(30, 400, k), y0 + rng.uniform(30, 400, k)], 1).astype(np.float32))
    labels, best = K.rcnn_label_batch(ctx, anchors, gts, [(1900, 1500), (2000, 1400)])
    for i, s in enumerate([(1900, 1500), (2000, 1400)]):
        want_l, want_b = oracle_labels(anchors, gts[i], s)
        assert np.array_equal(labels[i], want_l) and np.array_equal(best[i], want_b)


def test_bad_arguments(ctx):
    from aeon_b200 import _lib as L
    d = (L.RcnnDesc * 1)()
    assert ctx.lib.aeonb_rcnn_label_batch(ctx.handle, None, 10, d, 1, 0.3, 0.7) == L.ERR_INVALID
    assert ctx.lib.aeonb_rcnn_label_batch(ctx.handle, None, 10, d, 0, 0.3, 0.7) == 0


RCNN_NAMES = ["bbtargets", "bbtargets_mask", "labels_flat", "labels_mask", "image_shape", "gt_boxes", "gt_box_count",
              "gt_class_count", "image_scale", "difficult_flag"]


def compare_rcnn(got, want):
    for k in RCNN_NAMES:
        assert got[k].shape == want[k].shape and got[k].dtype == want[k].dtype, k
        if k == "bbtargets":     # the two log terms go through libm on either side: 1e-6 relative; the rest is exact
            assert np.array_equal(got[k] != 0, want[k] != 0)
            assert np.all(np.abs(got[k] - want[k]) <= 1e-6 * np.abs(want[k]) + 1e-7)
        else:
            assert np.array_equal(got[k], want[k]), k


def test_provider_like_the_reference_test(ctx):
    """TEST(localization_rcnn, provider), test/test_localization_rcnn.cpp:1373-1450: image + localization_rcnn,
    fixed_aspect_ratio with a fixed scaling factor; the picture fills 800 x 600 of the 1000 x 1000 slot.  The ten buffers
    in deterministic sampling mode equal the oracle's, and without a flip the reference's known foreground anchors."""
    import cv2
    from aeon_b200.provider import Provider
    from tests.pipeline_oracle import PipelineOracle
    g = golden()
    img = np.empty((375, 500, 3), np.uint8)
    img[:] = (50, 100, 200)
    png = cv2.imencode(".png", img)[1].tobytes()
    ann = g["annotation"].encode()
    for flip in (True, False):
        cfg = {"batch_size": 4, "random_seed": 3,
               "etl": [{"type": "image", "height": 1000, "width": 1000, "channel_major": False},
                       {"type": "localization_rcnn", "height": 1000, "width": 1000, "max_gt_boxes": 64,
                        "class_names": g["class_names"], "debug_deterministic": True}],
               "augmentation": [{"type": "image", "fixed_aspect_ratio": True, "fixed_scaling_factor": 1.6, "crop_enable": False,
                                 "flip_enable": flip}]}
        recs = [(png, ann)] * 4
        prov = Provider(ctx, cfg)
        assert len(prov.outputs) == 11
        got = prov.run_host(recs)
        image = got["image"]
        assert image.shape == (4, 1000, 1000, 3)
        assert (image[:, :600, :800] == np.array([50, 100, 200], np.uint8)).all()
        assert not image[:, 600:].any() and not image[:, :, 800:].any()
        oracle_cfg = dict(cfg, etl=[cfg["etl"][0], {k: v for k, v in cfg["etl"][1].items() if k != "debug_deterministic"}])
        want = PipelineOracle(oracle_cfg).batch(recs)
        compare_rcnn(got, want)
        if not flip:
            A = 34596
            fg = np.nonzero(got["labels_flat"][0].ravel()[A:])[0].tolist()
            assert fg == g["fg_idx"]
            assert sorted(np.nonzero(got["labels_mask"][0].ravel())[0].tolist()) == sorted(g["labels_mask_idx"])


def test_provider_random_sampling_is_a_valid_sample(ctx):
    """Without debug_deterministic the sample is random (the reference draws it from an engine seeded by std::random_device):
    check what every valid sample has in common -- sizes, labels of the chosen anchors, masks consistent with each other."""
    import cv2
    from aeon_b200.provider import Provider
    g = golden()
    png = cv2.imencode(".png", np.zeros((375, 500, 3), np.uint8))[1].tobytes()
    cfg = {"batch_size": 2, "random_seed": 9,
           "etl": [{"type": "image", "height": 1000, "width": 1000},
                   {"type": "localization_rcnn", "height": 1000, "width": 1000, "class_names": g["class_names"]}],
           "augmentation": [{"type": "image", "fixed_aspect_ratio": True, "fixed_scaling_factor": 1.6, "crop_enable": False}]}
    got = Provider(ctx, cfg).run_host([(png, g["annotation"].encode())] * 2)
    _, anchors, r = run_golden(g)
    A = len(anchors)
    picks = []
    for i in range(2):
        mask = got["labels_mask"][i].ravel()
        chosen = np.nonzero(mask[:A])[0]
        assert np.array_equal(mask[:A], mask[A:]) and len(chosen) == 256
        assert (r.labels[chosen] >= 0).all()
        fg = chosen[r.labels[chosen] == 1]
        assert len(fg) == min(128, int((r.labels == 1).sum()))
        assert np.array_equal(np.nonzero(got["labels_flat"][i].ravel()[A:])[0], fg)
        bm = got["bbtargets_mask"][i].reshape(4, A)
        assert np.array_equal(np.nonzero(bm[0])[0], fg) and (bm == bm[0]).all()
        assert np.array_equal(np.nonzero(np.abs(got["bbtargets"][i].reshape(4, A)).sum(0))[0].tolist(),
                              [c for c in chosen if np.abs(r.targets[c]).sum() != 0])
        picks.append(chosen.tolist())
    assert picks[0] != picks[1]      # two draws from one engine


def test_provider_with_random_crops_thresholds_and_small_samples(ctx):
    """Cropping enabled (boxes are cut, shifted and rescaled by the crop box before the anchors see them), other overlap
    thresholds, fewer rois than foreground anchors, a record whose boxes all fall outside the crop."""
    import cv2
    from aeon_b200.provider import Provider
    from tests.pipeline_oracle import PipelineOracle
    rng = np.random.default_rng(83)
    names = ["a", "b", "c"]
    recs = []
    for i in range(6):
        h, w = int(rng.integers(200, 300)), int(rng.integers(260, 400))
        png = cv2.imencode(".png", rng.integers(0, 256, (h, w, 3), dtype=np.uint8))[1].tobytes()
        objs = []
        for _ in range(int(rng.integers(1, 9))):
            x0, y0 = int(rng.integers(0, w - 60)), int(rng.integers(0, h - 60))
            if i == 5:
                x0, y0 = 0, 0          # a sliver in the corner: usually outside the crop
            objs.append({"bndbox": {"xmin": x0, "ymin": y0, "xmax": x0 + int(rng.integers(3 if i == 5 else 20, 6 if i == 5 else 59)),
                                    "ymax": y0 + int(rng.integers(3 if i == 5 else 20, 6 if i == 5 else 59))},
                         "name": names[int(rng.integers(3))], "difficult": bool(rng.integers(2))})
        recs.append((png, json.dumps({"object": objs, "size": {"width": w, "height": h, "depth": 3}}).encode()))
    for rc in ({"rois_per_image": 16, "foreground_fraction": 0.25}, {"negative_overlap": 0.2, "positive_overlap": 0.5},
               {"scaling_factor": 0.125, "base_size": 8, "ratios": [0.5, 1, 2, 3], "scales": [4, 8]}):
        etl_r = dict({"type": "localization_rcnn", "height": 240, "width": 320, "class_names": names, "debug_deterministic": True}, **rc)
        cfg = {"batch_size": 6, "random_seed": 17,
               "etl": [{"type": "image", "height": 240, "width": 320}, etl_r],
               "augmentation": [{"type": "image", "crop_enable": True, "scale": [0.5, 0.8], "flip_enable": True, "center": False}]}
        got = Provider(ctx, cfg).run_host(recs)
        oracle_cfg = dict(cfg, etl=[cfg["etl"][0], {k: v for k, v in etl_r.items() if k != "debug_deterministic"}])
        want = PipelineOracle(oracle_cfg).batch(recs)
        assert np.array_equal(got["image"], want["image"])
        compare_rcnn(got, want)
