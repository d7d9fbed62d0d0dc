"""Writes tests/golden/bbox_known_answers.json from the aeon tree: the known answers the reference's own tests hold
for the box arithmetic of the SSD / boundingbox path --

* test/test_bbox.cpp:283-637   boundingbox crop / expand / rescale / flip / crop_flip / expand_crop_flip_resize
                               (inputs, augmentation parameters, expected cv::Rect of every surviving box),
* test/test_bbox.cpp:761-912   intersect / jaccard_overlap / coverage of pixel boxes and of normalised boxes,
* test/test_localization_ssd.cpp:158-271   localization_ssd transform (flip + rescale) and loader buffers,
* test/test_augmentation.cpp:246-317       make_ssd_params without and with expansion + batch sampler.

The tests are C++ code, not tables, so this script reads the literals out of the test text (cv::Rect / bbox / nbox /
Point2f constructors, EXPECT_EQ lines) and, where the test computes its expectation in a loop, evaluates the same
loop on the extracted literals.  Nothing here calls into the repository's own box code.

Usage: python tests/golden/make_bbox_golden.py /path/to/aeon
"""
import json
import math
import os
import re
import sys

NUM = r"-?\d+(?:\.\d*)?(?:e-?\d+)?f?"


def test_body(src, suite, name):
    a = src.index("TEST(%s, %s)" % (suite, name))
    a = src.index("{", a)
    depth, i = 0, a
    while True:
        if src[i] == "{":
            depth += 1
        elif src[i] == "}":
            depth -= 1
            if depth == 0:
                return src[a + 1:i]
        i += 1


def split_args(text):
    """Top-level comma split of an argument list."""
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def call_args(text, start):
    """Arguments of the call whose '(' is at text[start]; returns (args, index after ')')."""
    depth, i = 0, start
    while True:
        if text[i] == "(":
            depth += 1
        elif text[i] == ")":
            depth -= 1
            if depth == 0:
                return split_args(text[start + 1:i]), i + 1
        i += 1


def c_eval(expr, env=None):
    """A C arithmetic expression over literals and the given variables, evaluated in double."""
    e = re.sub(r"(?<![\d.])0(\d+)(?![\d.])", lambda m: str(int(m.group(1), 8)), expr)  # C octal literals (00, 06)
    e = re.sub(r"(\d)\.(?=\D|$)", r"\1.0", e)
    e = re.sub(r"(\d)f\b", r"\1", e)
    e = e.replace("static_cast<float>", "float")
    return float(eval(e, {"__builtins__": {}, "float": float}, dict(env or {})))


def c_round(v):
    return int(math.floor(abs(v) + 0.5)) * (1 if v >= 0 else -1)


def rect_of_box(b):
    """boundingbox::box::rect(): std::round of xmin, ymin, width, height (src/box.hpp:53-57)."""
    return [c_round(b[0]), c_round(b[1]), c_round(b[2] - b[0] + 1), c_round(b[3] - b[1] + 1)]


def rects_named(body):
    """cv::Rect rN = cv::Rect(x, y, w, h) declarations in order -> boxes (xmin, ymin, xmax, ymax)."""
    out = []
    for m in re.finditer(r"cv::Rect\s+r\d+\s*=\s*cv::Rect\(([^)]*)\)", body):
        x, y, w, h = (int(v) for v in split_args(m.group(1)))
        out.append([x, y, x + w - 1, y + h - 1])
    return out


def expected_rects(body, env=None):
    """EXPECT_EQ(cv::Rect(...), tx_boxes[i].rect()) lines; cv::Rect is Rect_<int>: float arguments are truncated."""
    out = []
    for m in re.finditer(r"EXPECT_EQ\(cv::Rect\(", body):
        args, _ = call_args(body, m.end() - 1)
        out.append([int(c_eval(a, env)) for a in args])
    return out


def points(body, name):
    m = re.search(r"vector<cv::Point2f>\s+%s\s*=\s*\{" % name, body)
    seg = body[m.end():body.index("};", m.end())]
    return [[c_eval(a), c_eval(b)] for a, b in re.findall(r"cv::Point2f\(\s*(%s)\s*,\s*(%s)\s*\)" % (NUM, NUM), seg)]


def boundingbox_cases(src):
    cases = []
    base = dict(flip=False, expand_ratio=1.0, expand_offset=[0, 0], expand_size=[0, 0])

    def add(name, boxes, cropbox, out_size, expect, **kw):
        p = dict(base)
        p.update(kw)
        p.update(cropbox=cropbox, output_size=out_size)
        cases.append({"name": name, "boxes": boxes, "params": p, "expected_rects": expect})

    for name, flip in (("crop", False), ("crop_flip", True)):
        body = test_body(src, "boundingbox", name)
        crop = [int(v) for v in re.search(r"iparam->cropbox\s*=\s*cv::Rect\(([^)]*)\)", body).group(1).split(",")]
        add(name, rects_named(body), crop, crop[2:], expected_rects(body), flip=flip)
    body = test_body(src, "boundingbox", "rescale")
    ow, oh = (int(v) for v in re.search(r"output_size\s*=\s*cv::Size\((\d+),\s*(\d+)\)", body).groups())
    env = {"xscale": c_eval(re.search(r"xscale\s*=\s*([^;]*);", body).group(1)),
           "yscale": c_eval(re.search(r"yscale\s*=\s*([^;]*);", body).group(1))}
    add("rescale", rects_named(body), [0, 0, 256, 256], [ow, oh], expected_rects(body, env))
    body = test_body(src, "boundingbox", "flip")
    add("flip", rects_named(body), [0, 0, 256, 256], [256, 256], expected_rects(body), flip=True)

    # expand: the test builds inputs and expectations in a loop over b_off / b_size (test/test_bbox.cpp:335-401)
    body = test_body(src, "boundingbox", "expand")
    ints = {k: int(v) for k, v in re.findall(r"int\s+(\w+)\s*=\s*(\d+);", body)}
    off, size = points(body, "b_off"), points(body, "b_size")
    e = ints["expand_off"]
    boxes = [[o[0], o[1], o[0] + s[0] - 1, o[1] + s[1] - 1] for o, s in zip(off, size)]
    expect = [rect_of_box([b[0] + e, b[1] + e, b[2] + e, b[3] + e]) for b in boxes]
    add("expand", boxes, [0, 0, ints["out_width"], ints["out_height"]], [ints["out_width"], ints["out_height"]], expect,
        expand_ratio=ints["out_width"] / ints["width"], expand_offset=[e, e], expand_size=[ints["out_width"], ints["out_height"]],
        image_size=[ints["width"], ints["height"]])

    # expand_crop_flip_resize: same style (test/test_bbox.cpp:560-637); expectations in float32 as the test's bbox holds them
    import numpy as np
    f32 = np.float32
    body = test_body(src, "boundingbox", "expand_crop_flip_resize")
    ints = {k: int(v) for k, v in re.findall(r"int\s+(\w+)\s*=\s*(\d+);", body)}
    eo = [int(v) for v in re.search(r"cv::Point\s+expand_offset\(([^)]*)\)", body).group(1).split(",")]
    crop = [int(v) for v in re.search(r"cv::Rect\s+cropbox\(([^)]*)\)", body).group(1).split(",")]
    pos, size = points(body, "b_pos"), points(body, "b_size")
    xs, ys = f32(ints["output_width"]) / f32(crop[2]), f32(ints["output_height"]) / f32(crop[3])
    boxes, expect = [], []
    for o, s in zip(pos, size):
        boxes.append([o[0], o[1], o[0] + s[0] - 1, o[1] + s[1] - 1])
        b = [f32(o[0] + eo[0] - crop[0]), f32(o[1] + eo[1] - crop[1]), f32(o[0] + eo[0] - crop[0] + s[0] - 1),
             f32(o[1] + eo[1] - crop[1] + s[1] - 1)]
        fb = [f32((f32(crop[2]) - b[2] - f32(1)) * xs), f32(b[1] * ys), f32(((f32(crop[2]) - b[0] - f32(1)) + f32(1)) * xs - f32(1)),
              f32((b[3] + f32(1)) * ys - f32(1))]
        expect.append(rect_of_box([float(v) for v in fb]))
    add("expand_crop_flip_resize", boxes, crop, [ints["output_width"], ints["output_height"]], expect, flip=True,
        expand_ratio=float(ints["expand_size"] // ints["input_width"]), expand_offset=eo,
        expand_size=[ints["expand_size"], ints["expand_size"]], image_size=[ints["input_width"], ints["input_height"]])
    return cases


def ctor_values(text, kind, env):
    """bbox(...) / nbox(...) constructor arguments -> four floats; the default box is (0,0,-1,-1) / (0,0,0,0)."""
    text = text.strip()
    if text in env:
        return env[text]
    args, _ = call_args(text, text.index("("))
    if not args:
        return [0.0, 0.0, -1.0, -1.0] if kind == "bbox" else [0.0, 0.0, 0.0, 0.0]
    return [c_eval(a) for a in args[:4]]


def tuple_cases(src, suite, name, kind):
    body = test_body(src, suite, name)
    env = {}
    for m in re.finditer(r"\b%s\s+(box\d+)\(([^)]*)\);" % kind, body):
        env[m.group(1)] = [c_eval(a) for a in split_args(m.group(2))]
    out = []
    for m in re.finditer(r"make_tuple\(", body):
        args, _ = call_args(body, m.end() - 1)
        a, b = ctor_values(args[0], kind, env), ctor_values(args[1], kind, env)
        third = args[2].strip()
        if third.startswith(kind) or third in env:
            out.append({"a": a, "b": b, "expected": ctor_values(third, kind, env)})
        else:
            out.append({"a": a, "b": b, "expected": c_eval(third)})
    return out


def ssd_cases(root):
    src = open(os.path.join(root, "test", "test_localization_ssd.cpp")).read()
    body = test_body(src, "localization_ssd", "transform")
    ints = {k: int(v) for k, v in re.findall(r"int\s+(\w+)\s*=\s*(\d+);", body)}
    boxes_in = [[c_eval(v) for v in split_args(m)] for m in
                re.findall(r"bbox\(([^()]*)\)", body[body.index("m_boxes"):body.index("auto expected")])]
    seg = body[body.index("auto expected"):body.index("augment::image::param_factory")]
    expect = []
    for m in re.finditer(r"bbox\(([^()]*)\)\.rescale\(([^()]*)\)", seg):
        b = [c_eval(v) for v in split_args(m.group(1))]
        sx, sy = (c_eval(v) for v in split_args(m.group(2)))
        # boundingbox::box::rescale (src/boundingbox.cpp:78-86): min * s, (max + 1) * s - 1
        expect.append([b[0] * sx, b[1] * sy, (b[2] + 1) * sx - 1, (b[3] + 1) * sy - 1])
    transform = {"input_size": [ints["input_width"], ints["input_height"]], "output_size": [ints["output_width"], ints["output_height"]],
                 "flip": True, "boxes": boxes_in, "expected_boxes": expect}
    body = test_body(src, "localization_ssd", "loader")
    ints = {k: int(v) for k, v in re.findall(r"int\s+(\w+)\s*=\s*(\d+);", body)}
    seg = body[body.index("decoded->gt_boxes ="):body.index("decoded->gt_boxes[1]")]
    gt = [[c_eval(v) for v in split_args(m)] for m in re.findall(r"bbox\(([^()]*)\)", seg)]
    attrs = [{"difficult": False, "label": 0} for _ in gt]
    for i, key, val in re.findall(r"gt_boxes\[(\d)\]\.m_(difficult|label)\s*=\s*(\w+);", body):
        attrs[int(i)][key] = (val == "true") if key == "difficult" else int(val)
    loader = {"width": ints["width"], "height": ints["height"], "max_gt_boxes": ints["max_gt_boxes"], "gt_boxes": gt, "attrs": attrs}
    return {"transform": transform, "loader": loader}


def ssd_param_cases(root):
    src = open(os.path.join(root, "test", "test_augmentation.cpp")).read()
    out = {}
    for name in ("make_ssd_params_default", "make_ssd_params_transformations"):
        body = test_body(src, "image_augmentation", name)
        ints = {k: int(v) for k, v in re.findall(r"int\s+(\w+)\s*=\s*(\d+);", body)}
        exp = {}
        m = re.search(r"EXPECT_EQ\(params->cropbox,\s*cv::Rect\(([^)]*)\)\)", body)
        if m:
            exp["cropbox"] = [int(v) for v in m.group(1).split(",")]
        for key in ("cropbox.width", "cropbox.height"):
            m = re.search(r"EXPECT_EQ\(params->%s,\s*(\d+)\)" % re.escape(key), body)
            if m:
                exp[key] = int(m.group(1))
        for key in ("expand_offset.width", "expand_offset.height"):
            m = re.search(r"EXPECT_LE\(params->%s,\s*(\d+)\)" % re.escape(key), body)
            if m:
                exp[key + "_max"] = int(m.group(1))
        for key in ("expand_offset", "expand_size", "output_size"):
            m = re.search(r"EXPECT_EQ\(params->%s,\s*cv::Size2i\((\d+),\s*(\d+)\)\)" % key, body)
            if m:
                exp[key] = [int(m.group(1)), int(m.group(2))]
        for key in ("expand_ratio", "contrast", "brightness", "saturation", "emit_min_overlap"):
            m = re.search(r"EXPECT_EQ\(params->%s,\s*([\d.]+)f?\)" % key, body)
            if m:
                exp[key] = float(m.group(1))
        for key in ("angle", "hue"):
            exp[key] = int(re.search(r"EXPECT_EQ\(params->%s,\s*(\d+)\)" % key, body).group(1))
        exp["flip"] = re.search(r"EXPECT_EQ\(params->flip,\s*(\w+)\)", body).group(1) == "true"
        out[name] = {"input_size": [ints["input_width"], ints["input_height"]],
                     "output_size": [ints["output_width"], ints["output_height"]], "expected": exp}
    # the two configurations, restated from the nlohmann::json literals of the tests (test/test_augmentation.cpp:253,286-295)
    out["make_ssd_params_default"]["augmentation"] = {"type": "image", "crop_enable": False}
    out["make_ssd_params_default"]["boxes"] = []
    out["make_ssd_params_transformations"]["augmentation"] = {
        "type": "image", "crop_enable": False, "expand_ratio": [4.0, 4.0], "expand_probability": 1.0,
        "batch_samplers": [{"max_sample": 1, "max_trials": 50, "sampler": {"scale": [0.5, 0.5], "aspect_ratio": [1.0, 1.0]}}]}
    out["make_ssd_params_transformations"]["boxes"] = [[0.0, 0.0, 1.0, 1.0]]
    return out


def main(root):
    src = open(os.path.join(root, "test", "test_bbox.cpp")).read()
    out = {
        "source": "aeon test/test_bbox.cpp:283-637,761-912, test/test_localization_ssd.cpp:158-271, test/test_augmentation.cpp:246-317",
        "boundingbox_transform": boundingbox_cases(src),
        "bbox_intersect": tuple_cases(src, "boundingbox", "intersect_boundingbox", "bbox"),
        "nbox_intersect": tuple_cases(src, "normalized_box", "intersect_normalized_box", "nbox"),
        "bbox_jaccard": tuple_cases(src, "boundingbox", "jaccard_overlap_boundingbox", "bbox"),
        "nbox_jaccard": tuple_cases(src, "normalized_box", "jaccard_overlap_normalized_box", "nbox"),
        "nbox_coverage": tuple_cases(src, "normalized_box", "coverage_normalized_box", "nbox"),
        "bbox_coverage": tuple_cases(src, "boundingbox", "coverage_boundingbox", "bbox"),
        "localization_ssd": ssd_cases(root),
        "make_ssd_params": ssd_param_cases(root),
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bbox_known_answers.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print(path, {k: (len(v) if isinstance(v, list) else "-") for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
