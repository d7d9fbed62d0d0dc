"""Writes tests/golden/rcnn_loader_006637.json from the aeon tree: the known answers of the reference's own
TEST(localization_rcnn, loader) (test/test_localization_rcnn.cpp:595-1213) -- sampled foreground / background anchor
indices in deterministic mode, label-mask indices and box regression targets for test/test_data/006637.json at
1000 x 1000, fixed_scaling_factor 1.6 -- together with that annotation and the class list of the test file.

Usage: python tests/golden/make_rcnn_golden.py /path/to/aeon
"""
import json
import os
import re
import sys


def block(text, start_marker):
    a = text.index(start_marker)
    a = text.index("{", a)
    depth, i = 0, a
    while True:
        if text[i] == "{":
            depth += 1
        elif text[i] == "}":
            depth -= 1
            if depth == 0:
                return text[a + 1:i]
        i += 1


def main(root):
    src = open(os.path.join(root, "test", "test_localization_rcnn.cpp")).read()
    test = src[src.index("TEST(localization_rcnn, loader)"):src.index("TEST(localization_rcnn, loader_zero_gt_boxes)")]
    ints = lambda name: [int(v) for v in re.findall(r"-?\d+", block(test, name))]
    pairs = re.findall(r"\{\s*(\d+)\s*,\s*(-?[\d.]+(?:e-?\d+)?)\s*\}", block(test, "bbox_targets ="))
    labels = re.findall(r'"([^"]+)"', block(src, "vector<string> label_list"))
    out = {
        "source": "aeon test/test_localization_rcnn.cpp:595-1213, test/test_data/006637.json",
        "config": {"width": 1000, "height": 1000, "max_gt_boxes": 64, "fixed_scaling_factor": 1.6},
        "class_names": labels,
        "annotation": open(os.path.join(root, "test", "test_data", "006637.json")).read(),
        "bbox_mask_index": ints("bbox_mask_index ="),
        "bbox_targets": [[int(k), float(v)] for k, v in pairs],
        "fg_idx": ints("fg_idx ="),
        "bg_idx": ints("bg_idx ="),
        "labels_mask_idx": ints("labels_mask_idx ="),
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rcnn_loader_006637.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(path, {k: len(v) for k, v in out.items() if isinstance(v, list)})


if __name__ == "__main__":
    main(sys.argv[1])
