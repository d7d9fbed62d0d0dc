"""Pins of the SSD / boundingbox box arithmetic against the known answers the reference's own tests hold
(tests/golden/bbox_known_answers.json, extracted from aeon test/test_bbox.cpp:283-637,761-912,
test/test_localization_ssd.cpp:158-271 and test/test_augmentation.cpp:246-317 by tests/golden/make_bbox_golden.py).

Both the CPU oracle (oracle/ssd.py) and the C++ host code of the library (through the C ABI, no GPU needed) must
reproduce every one of them."""
import ctypes as C
import json
import math
import os

import numpy as np
import pytest

from oracle import params as op
from oracle import ssd

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "bbox_known_answers.json")))
EPS = 1e-5   # nervana::epsilon, the tolerance of the reference's EXPECT_NEAR lines


def lib():
    from aeon_b200 import _lib as L
    return L, L.load()


class BoxParams(C.Structure):
    _fields_ = [("crop", C.c_int32 * 4), ("out", C.c_int32 * 2), ("flip", C.c_int32), ("expand_ratio", C.c_float),
                ("expand_off", C.c_int32 * 2), ("expand_size", C.c_int32 * 2), ("emit_type", C.c_int32),
                ("emit_min_overlap", C.c_float)]


def rect(b):
    """boundingbox::box::rect() (src/box.hpp:53-57)."""
    r = lambda v: int(math.floor(abs(float(v)) + 0.5)) * (1 if v >= 0 else -1)
    return [r(b[0]), r(b[1]), r(np.float32(b[2]) - np.float32(b[0]) + np.float32(1)), r(np.float32(b[3]) - np.float32(b[1]) + np.float32(1))]


def oracle_params(p):
    q = op.ImageParams(cropbox=tuple(p["cropbox"]), output_size=tuple(p["output_size"]), flip=p["flip"])
    q.expand_ratio, q.expand_offset, q.expand_size = p["expand_ratio"], tuple(p["expand_offset"]), tuple(p["expand_size"])
    q.emit_type, q.emit_min_overlap = "", np.float32(0)
    return q


def host_transform(p, boxes):
    L, l = lib()
    bp = BoxParams()
    bp.crop[:] = p["cropbox"]
    bp.out[:] = p["output_size"]
    bp.flip = int(p["flip"])
    bp.expand_ratio = p["expand_ratio"]
    bp.expand_off[:] = p["expand_offset"]
    bp.expand_size[:] = p["expand_size"]
    n = len(boxes)
    src = np.array(boxes, np.float32).ravel()
    out = np.zeros(4 * n, np.float32)
    kept = (C.c_int32 * n)()
    n_out = C.c_int32()
    L.check(l.aeonb_transform_boxes(C.byref(bp), src.ctypes.data, n, out.ctypes.data, kept, C.byref(n_out)))
    return out.reshape(n, 4)[:n_out.value]


@pytest.mark.parametrize("case", GOLD["boundingbox_transform"], ids=lambda c: c["name"])
def test_boundingbox_transform_known_answers(case):
    p = case["params"]
    got_o = ssd.transform_boxes([ssd.Box(*b) for b in case["boxes"]], oracle_params(p))
    assert [rect((b.xmin, b.ymin, b.xmax, b.ymax)) for b in got_o] == case["expected_rects"]
    got_h = host_transform(p, case["boxes"])
    assert [rect(b) for b in got_h] == case["expected_rects"]
    # the two restatements agree to the bit, not only after rounding to a cv::Rect
    assert np.array_equal(got_h, np.array([[b.xmin, b.ymin, b.xmax, b.ymax] for b in got_o], np.float32).reshape(-1, 4))


def host_overlap(normalized, a, b):
    L, l = lib()
    fa, fb, out = (C.c_float * 4)(*a), (C.c_float * 4)(*b), (C.c_float * 6)()
    L.check(l.aeonb_box_overlap(int(normalized), fa, fb, out))
    return list(out)


def oracle_overlap(normalized, a, b):
    if normalized:
        x, y = ssd.NBox(*a), ssd.NBox(*b)
        i = x.intersect(y)
        return [i.xmin, i.ymin, i.xmax, i.ymax, x.jaccard_overlap(y), x.coverage(y)]
    x, y = ssd.Box(*a), ssd.Box(*b)
    i = ssd.box_intersect(x, y)
    return [i.xmin, i.ymin, i.xmax, i.ymax, ssd.box_jaccard(x, y), ssd.box_coverage(x, y)]


def float_eq(a, b):
    """gtest's EXPECT_FLOAT_EQ: within 4 units in the last place of float32."""
    a, b = np.float32(a), np.float32(b)
    return a == b or abs(float(a) - float(b)) <= 4 * float(np.spacing(max(abs(a), abs(b))))


@pytest.mark.parametrize("normalized,key", [(False, "bbox_intersect"), (True, "nbox_intersect")])
def test_intersect_known_answers(normalized, key):
    for c in GOLD[key]:
        for a, b in ((c["a"], c["b"]), (c["b"], c["a"])):
            for got in (host_overlap(normalized, a, b), oracle_overlap(normalized, a, b)):
                assert all(float_eq(g, w) for g, w in zip(got[:4], c["expected"])), (c, got)


@pytest.mark.parametrize("normalized,key", [(False, "bbox_jaccard"), (True, "nbox_jaccard")])
def test_jaccard_known_answers(normalized, key):
    for c in GOLD[key]:
        for a, b in ((c["a"], c["b"]), (c["b"], c["a"])):
            for got in (host_overlap(normalized, a, b), oracle_overlap(normalized, a, b)):
                assert float_eq(got[4], c["expected"]), (c, got)


@pytest.mark.parametrize("normalized,key", [(False, "bbox_coverage"), (True, "nbox_coverage")])
def test_coverage_known_answers(normalized, key):
    for c in GOLD[key]:
        for got in (host_overlap(normalized, c["a"], c["b"]), oracle_overlap(normalized, c["a"], c["b"])):
            assert abs(float(got[5]) - c["expected"]) <= EPS, (c, got)


def test_localization_ssd_transform_known_answers():
    """aeon test/test_localization_ssd.cpp:158-201: flip + rescale by 3 of three boxes, crop box = whole picture."""
    t = GOLD["localization_ssd"]["transform"]
    p = dict(cropbox=[0, 0, *t["input_size"]], output_size=t["output_size"], flip=t["flip"], expand_ratio=1.0,
             expand_offset=[0, 0], expand_size=t["input_size"])
    want = np.array(t["expected_boxes"], np.float32)
    got_o = ssd.transform_boxes([ssd.Box(*b) for b in t["boxes"]], oracle_params(p))
    assert np.array_equal(np.array([[b.xmin, b.ymin, b.xmax, b.ymax] for b in got_o], np.float32), want)
    assert np.array_equal(host_transform(p, t["boxes"]), want)


def test_localization_ssd_loader_known_answers():
    """aeon test/test_localization_ssd.cpp:203-271: normalised boxes, classes, difficult flags, zero rows after them."""
    g = GOLD["localization_ssd"]["loader"]
    W, H, M = g["width"], g["height"], g["max_gt_boxes"]
    f32 = np.float32
    want = np.zeros((M, 4), f32)
    for i, b in enumerate(g["gt_boxes"]):   # boundingbox::box::normalize (src/boundingbox.cpp:150-163)
        b = [f32(v) for v in b]
        want[i] = [b[0] / f32(W), b[1] / f32(H), (b[2] + f32(1)) / f32(W), (b[3] + f32(1)) / f32(H)]
    labels = [a["label"] for a in g["attrs"]]
    diff = [int(a["difficult"]) for a in g["attrs"]]
    gt = [ssd.Box(*b, label=l, difficult=bool(d)) for b, l, d in zip(g["gt_boxes"], labels, diff)]
    shape, boxes, count, classes, difficult = ssd.load_buffers(gt, W, H, M)
    L, l = lib()
    n = len(gt)
    src = np.array(g["gt_boxes"], f32).ravel()
    h_shape, h_boxes = np.zeros(2, np.int32), np.full((M, 4), 9, f32)
    h_count, h_cls, h_diff = np.zeros(1, np.int32), np.full(M, 9, np.int32), np.full(M, 9, np.int32)
    a_lab, a_diff = np.array(labels, np.int32), np.array(diff, np.int32)
    L.check(l.aeonb_ssd_load_boxes(src.ctypes.data, a_lab.ctypes.data, a_diff.ctypes.data,
                                   n, W, H, M, h_shape.ctypes.data, h_boxes.ctypes.data, h_count.ctypes.data,
                                   h_cls.ctypes.data, h_diff.ctypes.data))
    for s, b, c, k, d in ((shape.ravel(), boxes, count.ravel(), classes.ravel(), difficult.ravel()),
                          (h_shape, h_boxes, h_count, h_cls, h_diff)):
        assert s.tolist() == [W, H] and int(c[0]) == n
        assert all(float_eq(x, y) for x, y in zip(b.ravel(), want.ravel()))
        assert k[:n].tolist() == labels and d[:n].tolist() == diff
        assert not k[n:].any() and not d[n:].any() and not b[n:].any()


@pytest.mark.parametrize("name", ["make_ssd_params_default", "make_ssd_params_transformations"])
def test_make_ssd_params_known_answers(name):
    """aeon test/test_augmentation.cpp:246-317.  The reference's factory draws from a random-device seeded engine, so
    what it asserts holds for every seed: checked here over many seeds for the oracle and the host code."""
    g = GOLD["make_ssd_params"][name]
    exp = g["expected"]
    (iw, ih), (ow, oh) = g["input_size"], g["output_size"]
    L, l = lib()
    n = 64
    boxes = np.array(g["boxes"] * n, np.float32).ravel()
    cnt = (C.c_int32 * n)(*[len(g["boxes"])] * n)
    out = (C.c_double * (24 * n))()
    L.check(l.aeonb_draw_ssd_params(json.dumps(g["augmentation"]).encode(), 4321, n, n, (C.c_int32 * n)(*[iw] * n),
                                    (C.c_int32 * n)(*[ih] * n), ow, oh, cnt,
                                    boxes.ctypes.data_as(C.POINTER(C.c_float)) if len(boxes) else None, out))
    host = np.array(out).reshape(n, 24)
    f = ssd.SsdFactory(g["augmentation"])
    eng = op.slot_engines(4321, n)
    rows = []
    for i in range(n):
        p = f.make_ssd_params(eng[i], iw, ih, ow, oh, [ssd.Box(*b) for b in g["boxes"]])
        rows.append([*p.cropbox, *p.output_size, float(p.flip), p.angle, p.hue, float(p.contrast), float(p.brightness),
                     float(p.saturation), 0, 0, 0, 0, *p.padding_crop_offset, float(np.float32(p.expand_ratio)),
                     *p.expand_offset, *p.expand_size])
    orc = np.array(rows, np.float64)
    assert np.array_equal(orc, host[:, :23])
    for r in (orc, host):
        for row in r:
            if "cropbox" in exp:
                assert row[0:4].tolist() == exp["cropbox"]
            if "cropbox.width" in exp:
                assert row[2] == exp["cropbox.width"] and row[3] == exp["cropbox.height"]
            assert row[4:6].tolist() == exp["output_size"]
            assert bool(row[6]) == exp["flip"] and row[7] == exp["angle"] and row[8] == exp["hue"]
            assert row[9] == exp["contrast"] and row[10] == exp["brightness"] and row[11] == exp["saturation"]
            assert row[18] == exp["expand_ratio"] and row[21:23].tolist() == exp["expand_size"]
            if "expand_offset" in exp:
                assert row[19:21].tolist() == exp["expand_offset"]
            if "expand_offset.width_max" in exp:
                assert row[19] <= exp["expand_offset.width_max"] and row[20] <= exp["expand_offset.height_max"]
