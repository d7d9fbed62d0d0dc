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


def test_bad_arguments(ctx):
    from aeon_b200 import _lib as L
    d = (L.RcnnDesc * 1)()
    assert ctx.lib.aeonb_rcnn_label_batch(ctx.handle, None, 10, d, 1, 0.3, 0.7) == L.ERR_INVALID
    assert ctx.lib.aeonb_rcnn_label_batch(ctx.handle, None, 10, d, 0, 0.3, 0.7) == 0
