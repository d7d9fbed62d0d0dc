"""The localization_rcnn oracle against the reference's own known answers (read from its test file into
tests/golden/rcnn_loader_006637.json by tests/golden/make_rcnn_golden.py)."""
import json
import os

import numpy as np
import pytest

from oracle import params as oparams
from oracle import rcnn as orcnn
from oracle import ssd as ossd

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "rcnn_loader_006637.json")


def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def test_base_anchors_match_the_published_table():
    """test/test_localization_rcnn.cpp:101-140: the nine anchors of base size 16, ratios 0.5/1/2, scales 8/16/32 (the
    Matlab table minus one)."""
    want = np.array([[-83, -39, 100, 56], [-175, -87, 192, 104], [-359, -183, 376, 200], [-55, -55, 72, 72],
                     [-119, -119, 136, 136], [-247, -247, 264, 264], [-35, -79, 52, 96], [-79, -167, 96, 184],
                     [-167, -343, 184, 360]], np.float32) - 1
    assert np.array_equal(orcnn.base_anchors(), want)
    cfg = {"width": 1000, "height": 1000}
    anchors = orcnn.generate_anchors(cfg)
    assert anchors.shape == (34596, 4)                      # 9 * 62 * 62
    assert np.array_equal(anchors[:3], want[0] + np.array([[0, 0, 0, 0], [16, 0, 16, 0], [32, 0, 32, 0]], np.float32))
    assert np.array_equal(anchors[62], want[0] + np.array([0, 16, 0, 16], np.float32))
    assert np.array_equal(anchors[62 * 62], want[1])


def run_golden(g):
    cfg = dict(g["config"], class_names=g["class_names"])
    fixed = cfg.pop("fixed_scaling_factor")
    w, h, boxes = ossd.parse_annotation(g["annotation"].encode(), g["class_names"])
    factory = oparams.ParamFactory({"type": "image", "flip_enable": False, "crop_enable": False, "fixed_aspect_ratio": True,
                                    "fixed_scaling_factor": fixed})
    p = factory.make_params(oparams.MinstdRand0(1), w, h, cfg["width"], cfg["height"])
    anchors = orcnn.generate_anchors(cfg)
    return cfg, anchors, orcnn.transform(cfg, anchors, boxes, p, fixed_scaling_factor=fixed)


def test_reference_loader_known_answers():
    """TEST(localization_rcnn, loader), test/test_localization_rcnn.cpp:595-1213: sampled anchors in deterministic mode,
    every buffer of the loader; targets to the reference's 1e-5."""
    g = golden()
    cfg, anchors, r = run_golden(g)
    A = len(anchors)
    assert A == 34596 and r.im_size == (800, 600) and np.float32(r.image_scale) == np.float32(1.6)
    assert r.anchor_index == g["fg_idx"] + g["bg_idx"]
    out = orcnn.load(cfg, A, r)
    fg = set(g["fg_idx"])
    flat = out["labels_flat"].ravel()
    want_flat = np.concatenate([np.ones(A, np.int32), np.zeros(A, np.int32)])
    for i in fg:
        want_flat[i], want_flat[i + A] = 0, 1
    assert np.array_equal(flat, want_flat)
    want_mask = np.zeros(2 * A, np.int32)
    want_mask[g["labels_mask_idx"]] = 1
    assert np.array_equal(out["labels_mask"].ravel(), want_mask)
    want_t = np.zeros(4 * A, np.float32)
    for k, v in g["bbox_targets"]:
        want_t[k] = v
    assert np.abs(out["bbtargets"] - want_t).max() <= 1e-5
    assert np.array_equal(out["bbtargets"] != 0, want_t != 0) or np.abs(out["bbtargets"][(out["bbtargets"] != 0) != (want_t != 0)]).max() < 1e-5
    want_bm = np.zeros(4 * A, np.float32)
    want_bm[g["bbox_mask_index"]] = 1
    assert np.array_equal(out["bbtargets_mask"], want_bm)
    assert out["image_shape"].ravel().tolist() == [800, 600] and int(out["gt_box_count"][0, 0]) == 6
    _, _, boxes = ossd.parse_annotation(g["annotation"].encode(), g["class_names"])
    s = np.float32(1.6)
    for i, b in enumerate(boxes):
        want = [b.xmin * s, b.ymin * s, (b.xmax + np.float32(1)) * s - np.float32(1), (b.ymax + np.float32(1)) * s - np.float32(1)]
        assert out["gt_boxes"][i].tolist() == [float(np.float32(v)) for v in want]
        assert out["gt_class_count"][i, 0] == b.label and out["difficult_flag"][i, 0] == int(b.difficult)
    assert not out["gt_boxes"][6:].any()


def test_no_ground_truth_boxes_leaves_every_anchor_unlabelled():
    """TEST(localization_rcnn, loader_zero_gt_boxes), test/test_localization_rcnn.cpp:1215-1317: nothing is sampled."""
    g = golden()
    ann = json.loads(g["annotation"])
    ann["object"] = []
    g["annotation"] = json.dumps(ann)
    cfg, anchors, r = run_golden(g)
    assert r.anchor_index == [] and (r.labels == -1).all()
    out = orcnn.load(cfg, len(anchors), r)
    assert not out["bbtargets"].any() and not out["labels_mask"].any() and int(out["gt_box_count"][0, 0]) == 0
    assert out["labels_flat"].ravel()[:len(anchors)].all() and not out["labels_flat"].ravel()[len(anchors):].any()


def test_host_anchor_table_equals_the_oracle():
    """aeonb_rcnn_anchors (host C++) against the numpy restatement, default and odd configurations."""
    from aeon_b200 import kernels as K
    for kw in ({"width": 1000, "height": 1000}, {"width": 600, "height": 400, "base_size": 8, "scaling_factor": 1.0 / 8.0},
               {"width": 300, "height": 333, "ratios": (0.33, 1, 3, 1.7), "scales": (2, 4.5)},
               {"width": 100, "height": 50, "scaling_factor": 0.1, "base_size": 10}):
        got = K.rcnn_anchors(K.rcnn_config(**kw))
        want = orcnn.generate_anchors(kw)
        assert got.shape == want.shape and np.array_equal(got, want), kw


def test_host_anchor_table_rejects_bad_configurations():
    from aeon_b200 import _lib as L, kernels as K
    import ctypes as C
    lib = L.load()
    out = np.zeros((16, 4), np.float32)
    for kw in ({"width": 0, "height": 100}, {"width": 100, "height": 100, "scaling_factor": 0.0},
               {"width": 100, "height": 100, "base_size": 0}):
        cfg = K.rcnn_config(**kw)
        assert lib.aeonb_rcnn_anchor_count(C.byref(cfg)) == 0 or kw.get("base_size") == 0
        assert lib.aeonb_rcnn_anchors(C.byref(cfg), out.ctypes.data) == L.ERR_INVALID
    cfg = K.rcnn_config(100, 100)
    cfg.n_ratios = 9
    assert lib.aeonb_rcnn_anchors(C.byref(cfg), out.ctypes.data) == L.ERR_INVALID
    assert lib.aeonb_rcnn_anchors(None, out.ctypes.data) == L.ERR_INVALID
