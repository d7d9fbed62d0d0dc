"""CPU oracle for aeon's SSD localisation path (TEST INFRASTRUCTURE ONLY).

Restates, in float32 arithmetic, ``param_factory::make_ssd_params`` and the patch samplers
(aeon src/augment_image.cpp:232-586), the box classes (src/box.hpp, src/boundingbox.cpp:78-163,
src/normalized_box.cpp:47-107), ``boundingbox::transformer::transform_box``
(src/etl_boundingbox.cpp:146-261) and ``localization::ssd::loader::load``
(src/etl_localization_ssd.cpp:116-149).  Pinned (tests/test_oracle_ssd.py) against the known answers the
reference's own tests hold: box crop / expand / rescale / flip and their combinations, intersect /
jaccard / coverage of both box kinds (test/test_bbox.cpp:283-637,761-912), the SSD transform and
loader buffers (test/test_localization_ssd.cpp:158-271) and make_ssd_params
(test/test_augmentation.cpp:246-317).  What the reference does not pin is the SEEDED patch sampling
(its sampler tests check properties of a random-device seeded engine): those values are compared
between this file and the C++ host code only.  Nothing in the shipped package imports this file.
"""
import json
import math

import numpy as np

from . import params as P

f32 = np.float32
EPS = f32(0.00001)


class Box:
    """Pixel box with inclusive max corner."""

    def __init__(self, xmin, ymin, xmax, ymax, label=0, difficult=False):
        self.xmin, self.ymin, self.xmax, self.ymax = f32(xmin), f32(ymin), f32(xmax), f32(ymax)
        self.label, self.difficult = label, difficult

    def width(self):
        return f32(f32(self.xmax - self.xmin) + f32(1))

    def height(self):
        return f32(f32(self.ymax - self.ymin) + f32(1))

    def size(self):
        if self.xmax < self.xmin or self.ymax < self.ymin:
            return f32(0)
        return f32(self.width() * self.height())

    def copy(self):
        return Box(self.xmin, self.ymin, self.xmax, self.ymax, self.label, self.difficult)


class NBox:
    """Normalised box with exclusive max corner; must lie in [0,1] up to 1e-5."""

    def __init__(self, xmin=0, ymin=0, xmax=0, ymax=0, check=True):
        self.xmin, self.ymin, self.xmax, self.ymax = f32(xmin), f32(ymin), f32(xmax), f32(ymax)
        if check:
            for v in (self.xmin, self.xmax, self.ymin, self.ymax):
                if not (v >= f32(0) - EPS and v <= f32(1) + EPS):
                    raise ValueError("bounding box is not properly normalized")

    def size(self):
        if self.xmax < self.xmin or self.ymax < self.ymin:
            return f32(0)
        return f32(f32(self.xmax - self.xmin) * f32(self.ymax - self.ymin))

    def intersect(self, o):
        if o.xmin > self.xmax or o.xmax < self.xmin or o.ymin > self.ymax or o.ymax < self.ymin:
            return NBox()
        return NBox(max(self.xmin, o.xmin), max(self.ymin, o.ymin), min(self.xmax, o.xmax), min(self.ymax, o.ymax))

    def jaccard_overlap(self, o):
        inter = self.intersect(o).size()
        if inter == 0:
            return f32(0)
        return f32(inter / f32(f32(self.size() + o.size()) - inter))

    def coverage(self, o):
        inter = self.intersect(o).size()
        return f32(inter / self.size()) if inter > 0 else f32(0)


def c_round(v):
    """std::round: half away from zero."""
    v = float(v)
    return int(math.floor(abs(v) + 0.5)) * (1 if v >= 0 else -1)


class Sampler:
    def __init__(self, cfg):
        cfg = cfg or {}
        self.scale = tuple(cfg.get("scale", (1.0, 1.0)))
        self.aspect = tuple(cfg.get("aspect_ratio", (1.0, 1.0)))

    def sample_patch(self, g):
        scale = P.uniform_real_f32(g, *self.scale)
        s2 = float(scale) ** 2.0
        lo = max(f32(self.aspect[0]), f32(s2))
        hi = min(f32(self.aspect[1]), f32(1.0 / s2))
        ar = P.uniform_real_f32(g, lo, hi)
        bw = f32(scale * np.sqrt(ar))
        bh = f32(scale / np.sqrt(ar))
        w_off = P.uniform_real_f32(g, 0.0, f32(f32(1) - bw))
        h_off = P.uniform_real_f32(g, 0.0, f32(f32(1) - bh))
        return NBox(w_off, h_off, f32(w_off + bw), f32(h_off + bh))


class Constraint:
    KEYS = ("min_jaccard_overlap", "max_jaccard_overlap", "min_sample_coverage", "max_sample_coverage",
            "min_object_coverage", "max_object_coverage")

    def __init__(self, cfg):
        cfg = cfg or {}
        for k in self.KEYS:
            setattr(self, k, f32(cfg[k]) if k in cfg else None)

    def satisfies(self, sampled, objects):
        has_j = self.min_jaccard_overlap is not None or self.max_jaccard_overlap is not None
        has_s = self.min_sample_coverage is not None or self.max_sample_coverage is not None
        has_o = self.min_object_coverage is not None or self.max_object_coverage is not None
        if not (has_j or has_s or has_o):
            return True
        found = False
        for ob in objects:
            if has_j:
                v = sampled.jaccard_overlap(ob)
                if self.min_jaccard_overlap is not None and v < self.min_jaccard_overlap:
                    continue
                if self.max_jaccard_overlap is not None and v > self.max_jaccard_overlap:
                    continue
                found = True
            if has_s:
                v = sampled.coverage(ob)
                if self.min_sample_coverage is not None and v < self.min_sample_coverage:
                    continue
                if self.max_sample_coverage is not None and v > self.max_sample_coverage:
                    continue
                found = True
            if has_o:
                v = ob.coverage(sampled)
                if self.min_object_coverage is not None and v < self.min_object_coverage:
                    continue
                if self.max_object_coverage is not None and v > self.max_object_coverage:
                    continue
                found = True
            if found:
                return True
        return found


class BatchSampler:
    def __init__(self, cfg):
        cfg = cfg or {}
        self.max_sample = cfg.get("max_sample", -1)
        self.max_trials = cfg.get("max_trials", 100)
        self.sampler = Sampler(cfg.get("sampler"))
        self.constraint = Constraint(cfg.get("sample_constraint"))

    def sample_patches(self, g, objects, out):
        found = 0
        for _ in range(self.max_trials):
            if self.max_sample != -1 and found >= self.max_sample:
                break
            s = self.sampler.sample_patch(g)
            if self.constraint.satisfies(s, objects):
                found += 1
                out.append(s)


class SsdFactory(P.ParamFactory):
    def __init__(self, cfg):
        super().__init__(cfg)
        cfg = cfg or {}
        self.expand_ratio = tuple(cfg.get("expand_ratio", (1.0, 1.0)))
        self.expand_probability = f32(cfg.get("expand_probability", 0.0))
        self.emit_type = cfg.get("emit_constraint_type", "").lower()
        self.emit_min_overlap = f32(cfg.get("emit_constraint_min_overlap", 0.0))
        self.batch_samplers = [BatchSampler(c) for c in cfg.get("batch_samplers", [])]

    def make_ssd_params(self, g, in_w, in_h, out_w, out_h, boxes):
        p = self.make_params(g, in_w, in_h, out_w, out_h)
        p.output_size = (out_w, out_h)
        p.emit_type, p.emit_min_overlap = self.emit_type, self.emit_min_overlap
        ratio = P.uniform_real_f32(g, *self.expand_ratio)
        enabled = P.uniform_real_f32(g, 0.0, 1.0) < self.expand_probability
        if enabled:
            ew, eh = f32(ratio * f32(in_w)), f32(ratio * f32(in_h))
            p.expand_ratio = float(ratio)
            p.expand_size = (int(math.floor(ew)), int(math.floor(eh)))
            w_off = f32(P.uniform_real_f32(g, 0.0, 1.0) * f32(ew - f32(in_w)))
            h_off = f32(P.uniform_real_f32(g, 0.0, 1.0) * f32(eh - f32(in_h)))
            p.expand_offset = (int(math.floor(w_off)), int(math.floor(h_off)))
        else:
            p.expand_ratio, p.expand_offset, p.expand_size = 1.0, (0, 0), (in_w, in_h)
        W, H = p.expand_size
        objs = []
        for b in boxes:
            e = expand_box(b, p)
            objs.append(NBox(f32(e.xmin / f32(W)), f32(e.ymin / f32(H)), f32(f32(e.xmax + f32(1)) / f32(W)),
                             f32(f32(e.ymax + f32(1)) / f32(H))))
        if not self.crop_enable:
            samples = []
            for bs in self.batch_samplers:
                bs.sample_patches(g, objs, samples)
            patch = samples[P.uniform_int(g, 0, len(samples) - 1)] if samples else NBox(0, 0, 1, 1)
            bx = Box(f32(patch.xmin * f32(W)), f32(patch.ymin * f32(H)), f32(f32(patch.xmax * f32(W)) - f32(1)),
                     f32(f32(patch.ymax * f32(H)) - f32(1)))
            p.cropbox = (c_round(bx.xmin), c_round(bx.ymin), c_round(bx.width()), c_round(bx.height()))
        return p


def expand_box(b, p):
    if f32(p.expand_ratio) <= 1.0:
        return b.copy()
    ox, oy = p.expand_offset
    W, H = p.expand_size
    if b.xmax + f32(ox) > W or b.ymax + f32(oy) > H:
        raise ValueError("Invalid parameters to expand boundingbox")
    return Box(f32(b.xmin + f32(ox)), f32(b.ymin + f32(oy)), f32(b.xmax + f32(ox)), f32(b.ymax + f32(oy)), b.label, b.difficult)


def box_intersect(a, b):
    """boundingbox::box::intersect (src/boundingbox.cpp:134-148); no intersection gives the default box (0, 0, -1, -1)."""
    if b.xmin > a.xmax or b.xmax < a.xmin or b.ymin > a.ymax or b.ymax < a.ymin:
        return Box(0, 0, -1, -1)
    return Box(max(a.xmin, b.xmin), max(a.ymin, b.ymin), min(a.xmax, b.xmax), min(a.ymax, b.ymax))


def box_jaccard(a, b):
    """boundingbox::box::jaccard_overlap (src/boundingbox.cpp:105-116)."""
    inter = box_intersect(a, b).size()
    if inter == 0:
        return f32(0)
    return f32(inter / f32(f32(a.size() + b.size()) - inter))


def box_coverage(a, b):
    """boundingbox::box::coverage (src/boundingbox.cpp:118-132)."""
    s = box_intersect(a, b).size()
    return f32(s / a.size()) if s > 0 else f32(0)


def transform_boxes(boxes, p):
    cx, cy, cw, ch = p.cropbox
    xs = f32(f32(p.output_size[0]) / f32(cw))
    ys = f32(f32(p.output_size[1]) / f32(ch))
    out = []
    for b in boxes:
        b = expand_box(b, p)
        if p.emit_type in ("center", "min_overlap"):
            cb = Box(cx, cy, cx + cw - 1, cy + ch - 1)
            if p.emit_type == "center":
                xc = f32(float(b.xmin) + float(f32(b.xmax - b.xmin)) / 2.0)
                yc = f32(float(b.ymin) + float(f32(b.ymax - b.ymin)) / 2.0)
                keep = cb.xmin <= xc <= cb.xmax and cb.ymin <= yc <= cb.ymax
            else:
                keep = box_coverage(b, cb) >= p.emit_min_overlap
            if not keep:
                continue
        if b.xmax < cx or b.xmin >= cx + cw or b.ymax < cy or b.ymin >= cy + ch:
            continue
        b.xmin = f32(0) if b.xmin < cx else f32(b.xmin - f32(cx))
        b.ymin = f32(0) if b.ymin < cy else f32(b.ymin - f32(cy))
        b.xmax = f32(cw - 1) if b.xmax >= cx + cw else f32(b.xmax - f32(cx))
        b.ymax = f32(ch - 1) if b.ymax >= cy + ch else f32(b.ymax - f32(cy))
        if p.flip:
            xmax = b.xmax
            b.xmax = f32(f32(f32(cw) - b.xmin) - f32(1))
            b.xmin = f32(f32(f32(cw) - xmax) - f32(1))
        b.xmin = f32(b.xmin * xs)
        b.ymin = f32(b.ymin * ys)
        b.xmax = f32(f32(f32(b.xmax + f32(1)) * xs) - f32(1))
        b.ymax = f32(f32(f32(b.ymax + f32(1)) * ys) - f32(1))
        out.append(b)
    return out


def parse_annotation(blob, class_names):
    j = json.loads(blob)
    boxes = []
    for o in j["object"]:
        bb = o["bndbox"]
        boxes.append(Box(bb["xmin"], bb["ymin"], bb["xmax"], bb["ymax"], class_names.index(o["name"]),
                         bool(o.get("difficult", False))))
    return j["size"]["width"], j["size"]["height"], boxes


def load_buffers(gt, out_w, out_h, max_gt_boxes):
    """The five SSD buffers of one record (src/etl_localization_ssd.cpp:116-149)."""
    im_shape = np.array([[out_w], [out_h]], np.int32)
    boxes = np.zeros((max_gt_boxes, 4), f32)
    classes = np.zeros((max_gt_boxes, 1), np.int32)
    difficult = np.zeros((max_gt_boxes, 1), np.int32)
    n = min(max_gt_boxes, len(gt))
    for i in range(n):
        b = gt[i]
        boxes[i] = [f32(b.xmin / f32(out_w)), f32(b.ymin / f32(out_h)), f32(f32(b.xmax + f32(1)) / f32(out_w)),
                    f32(f32(b.ymax + f32(1)) / f32(out_h))]
        classes[i, 0] = b.label
        difficult[i, 0] = int(b.difficult)
    return im_shape, boxes, np.array([[n]], np.int32), classes, difficult
