"""CPU oracle (test infrastructure only) for aeon's localization_rcnn ETL: anchor generation, anchor labelling
against the ground-truth boxes, regression targets, anchor sampling and the ten output buffers.

Restates src/etl_localization_rcnn.cpp in numpy float32, operation by operation; every function cites the lines it
follows.  Pinned against the reference's own known answers (test/test_localization_rcnn.cpp:101-140 for the anchors,
:595-1213 for the sampled indices and targets of test/test_data/006637.json).
"""
import math

import numpy as np

from . import params as P
from . import ssd as S

f32 = np.float32


def _c_round(v):
    """C ``round`` on a float: half away from zero."""
    v = float(v)
    return f32(math.floor(abs(v) + 0.5) * (1 if v >= 0 else -1))


def _center(lo, hi):
    """box::xcenter / ycenter (src/box.hpp:92-93): lo + (hi - lo) / 2. with the division and sum in double."""
    return f32(float(lo) + float(f32(hi - lo)) / 2.0)


def _mkanchors(ws, hs, xc, yc):
    """anchor::mkanchors (src/etl_localization_rcnn.cpp:508-522): the 0.5 * (w - 1) terms are formed in double."""
    out = []
    for w, h in zip(ws, hs):
        dw, dh = 0.5 * float(f32(w - f32(1))), 0.5 * float(f32(h - f32(1)))
        out.append((f32(float(xc) - dw), f32(float(yc) - dh), f32(float(xc) + dw), f32(float(yc) + dh)))
    return out


def _ratio_enum(anchor, ratios):
    """anchor::ratio_enum (:524-545): size is truncated to an int, widths and heights are rounded."""
    x0, y0, x1, y1 = anchor
    w, h = f32(f32(x1 - x0) + f32(1)), f32(f32(y1 - y0) + f32(1))
    size = int(f32(w * h))
    ws = [_c_round(f32(math.sqrt(float(f32(f32(size) / f32(r)))))) for r in ratios]
    hs = [_c_round(f32(wi * f32(r))) for wi, r in zip(ws, ratios)]
    return _mkanchors(ws, hs, _center(x0, x1), _center(y0, y1))


def _scale_enum(anchor, scales):
    """anchor::scale_enum (:547-557)."""
    x0, y0, x1, y1 = anchor
    w, h = f32(f32(x1 - x0) + f32(1)), f32(f32(y1 - y0) + f32(1))
    return _mkanchors([f32(w * f32(s)) for s in scales], [f32(h * f32(s)) for s in scales], _center(x0, x1), _center(y0, y1))


def base_anchors(base_size=16, ratios=(0.5, 1, 2), scales=(8, 16, 32)):
    """anchor::generate_anchors (:489-506): ratios outermost, scales inner."""
    out = []
    for ra in _ratio_enum((f32(0), f32(0), f32(base_size - 1), f32(base_size - 1)), ratios):
        out += _scale_enum(ra, scales)
    return np.array(out, f32)


def generate_anchors(cfg):
    """anchor::generate (:434-472): every base anchor shifted over the conv grid; anchor-major, then y, then x.
    The shifts ``i * 1. / scaling_factor`` are formed in double from a float i and a float factor."""
    sf = f32(cfg.get("scaling_factor", 1.0 / 16.0))
    nx = int(math.floor(float(f32(f32(cfg["width"]) * sf))))
    ny = int(math.floor(float(f32(f32(cfg["height"]) * sf))))
    sx = np.array([f32(float(i) * 1.0 / float(sf)) for i in range(nx)], f32)
    sy = np.array([f32(float(i) * 1.0 / float(sf)) for i in range(ny)], f32)
    base = base_anchors(cfg.get("base_size", 16), cfg.get("ratios", (0.5, 1, 2)), cfg.get("scales", (8, 16, 32)))
    gx, gy = np.meshgrid(sx, sy)                    # y-major
    shifts = np.stack([gx.ravel(), gy.ravel(), gx.ravel(), gy.ravel()], 1).astype(f32)
    return (shifts[None, :, :] + base[:, None, :]).astype(f32).reshape(-1, 4)


def bbox_overlaps(anchors, gt):
    """transformer::bbox_overlaps (:302-338): intersection over union with the "+ 1" pixel convention, float32; zero where
    the boxes do not meet."""
    n, k = len(anchors), len(gt)
    out = np.zeros((n, k), f32)
    if n == 0 or k == 0:
        return out
    a = anchors.astype(f32)
    aw = (a[:, 2] - a[:, 0]) + f32(1)
    ah = (a[:, 3] - a[:, 1]) + f32(1)
    for j, g in enumerate(gt):
        area = f32(g.width() * g.height())
        iw = (np.minimum(a[:, 2], g.xmax) - np.maximum(a[:, 0], g.xmin)) + f32(1)
        ih = (np.minimum(a[:, 3], g.ymax) - np.maximum(a[:, 1], g.ymin)) + f32(1)
        ok = (iw > 0) & (ih > 0)
        inter = iw * ih
        ua = (aw * ah + area) - inter
        with np.errstate(divide="ignore", invalid="ignore"):
            out[:, j] = np.where(ok, inter / ua, f32(0))
    return out


def label_anchors(overlaps, negative_overlap=0.3, positive_overlap=0.7):
    """The labelling rules of transformer::transform (:127-193) on the anchors inside the picture: background below the
    negative threshold, foreground for every anchor that equals a ground-truth box's best overlap (ties included; a box
    nobody overlaps has a best overlap of 0 and so marks every anchor that misses it), foreground at or above the
    positive threshold; the rest stays -1.  Also the index of the best box per anchor (first one on ties, 0 when none)."""
    n, k = overlaps.shape
    labels = np.full(n, -1, np.int32)
    row_max = overlaps.max(axis=1) if k else np.zeros(n, f32)
    col_max = overlaps.max(axis=0) if n else np.zeros(k, f32)
    row_max, col_max = np.maximum(row_max, f32(0)), np.maximum(col_max, f32(0))
    labels[row_max < f32(negative_overlap)] = 0
    if k:
        labels[(overlaps == col_max[None, :]).any(axis=1)] = 1
    labels[row_max >= f32(positive_overlap)] = 1
    argmax = np.where(row_max > 0, overlaps.argmax(axis=1), 0) if k else np.zeros(n, np.int64)
    return labels, argmax


def compute_targets(gt_rows, anchors):
    """transformer::compute_targets (:265-300): (dx, dy, dw, dh) of each anchor towards its box, float32."""
    out = np.zeros((len(anchors), 4), f32)
    for i, (g, a) in enumerate(zip(gt_rows, anchors)):
        aw, ah = f32(f32(a[2] - a[0]) + f32(1)), f32(f32(a[3] - a[1]) + f32(1))
        out[i, 0] = f32(f32(_center(g.xmin, g.xmax) - _center(a[0], a[2])) / aw)
        out[i, 1] = f32(f32(_center(g.ymin, g.ymax) - _center(a[1], a[3])) / ah)
        out[i, 2] = f32(np.log(f32(g.width() / aw)))
        out[i, 3] = f32(np.log(f32(g.height() / ah)))
    return out


def sample_anchors(labels, rois_per_image=256, foreground_fraction=0.5, shuffle=None):
    """transformer::sample_anchors (:218-263).  ``shuffle`` permutes a list in place; None is the reference's
    debug_deterministic mode (index order).  The reference shuffles with a thread-local engine seeded from
    std::random_device, so only the deterministic mode has a defined answer."""
    num_fg = int(f32(f32(foreground_fraction) * f32(rois_per_image)))
    fg = [i for i, v in enumerate(labels) if v >= 1]
    bg = [i for i, v in enumerate(labels) if v == 0]
    if shuffle is not None:
        shuffle(fg)
        shuffle(bg)
    fg = fg[:num_fg]
    bg = bg[:rois_per_image - len(fg)]
    return fg + bg


class RcnnResult:
    pass


def transform(cfg, anchors, boxes, p, fixed_scaling_factor=-1.0, shuffle=None):
    """transformer::transform (:97-216).  cfg: the localization_rcnn etl block; boxes: oracle.ssd.Box list; p: the
    record's augmentation parameters."""
    cw, ch = p.cropbox[2], p.cropbox[3]
    if fixed_scaling_factor > 0:
        scale = f32(fixed_scaling_factor)
    else:                                                    # image::calculate_scale (src/image.cpp:214-222)
        scale = f32(f32(cfg["width"]) / f32(cw))
        if f32(f32(ch) * scale) > cfg["height"]:
            scale = f32(f32(cfg["height"]) / f32(ch))
    r = RcnnResult()
    r.image_scale = scale
    r.im_size = (P.unbiased_round(f32(f32(cw) * scale)), P.unbiased_round(f32(f32(ch) * scale)))
    total = len(anchors)
    inside = np.nonzero((anchors[:, 0] >= 0) & (anchors[:, 1] >= 0) & (anchors[:, 2] < r.im_size[0]) &
                        (anchors[:, 3] < r.im_size[1]))[0]
    r.gt_boxes = S.transform_boxes([b.copy() for b in boxes], p)
    r.labels = np.full(total, -1, np.int32)
    r.targets = np.zeros((total, 4), f32)
    if r.gt_boxes:           # without boxes no target list is built and no label is carried over (:181-208)
        ov = bbox_overlaps(anchors[inside], r.gt_boxes)
        labels, argmax = label_anchors(ov, cfg.get("negative_overlap", 0.3), cfg.get("positive_overlap", 0.7))
        r.labels[inside] = labels
        r.targets[inside] = compute_targets([r.gt_boxes[j] for j in argmax], anchors[inside])
    r.anchor_index = sample_anchors(r.labels, cfg.get("rois_per_image", 256), cfg.get("foreground_fraction", 0.5), shuffle)
    return r


def load(cfg, total_anchors, r):
    """loader::load (:340-432): the ten buffers, in the provider's order (src/provider.cpp:229-252)."""
    A, M = total_anchors, cfg.get("max_gt_boxes", 64)
    bbtargets, bbmask = np.zeros(4 * A, f32), np.zeros(4 * A, f32)
    labels_flat = np.concatenate([np.ones(A, np.int32), np.zeros(A, np.int32)])
    labels_mask = np.zeros(2 * A, np.int32)
    for i in r.anchor_index:
        if r.labels[i] == 1:
            labels_flat[i], labels_flat[i + A] = 0, 1
            bbmask[i::A] = 1
        labels_mask[i] = labels_mask[i + A] = 1
        bbtargets[i::A] = r.targets[i]
    n = min(M, len(r.gt_boxes))
    gt = np.zeros((M, 4), f32)
    cls, diff = np.zeros(M, np.int32), np.zeros(M, np.int32)
    for i, b in enumerate(r.gt_boxes[:n]):
        gt[i] = (b.xmin, b.ymin, b.xmax, b.ymax)
        cls[i], diff[i] = b.label, int(b.difficult)
    return {"bbtargets": bbtargets, "bbtargets_mask": bbmask, "labels_flat": labels_flat.reshape(1, 2 * A),
            "labels_mask": labels_mask.reshape(2 * A, 1), "image_shape": np.array([[r.im_size[0]], [r.im_size[1]]], np.int32),
            "gt_boxes": gt, "gt_box_count": np.array([[n]], np.int32), "gt_class_count": cls.reshape(M, 1),
            "image_scale": np.array([[r.image_scale]], f32), "difficult_flag": diff.reshape(M, 1)}
