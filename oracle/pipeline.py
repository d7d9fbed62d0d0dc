"""Record-level oracle for a whole provider call: decode -> seeded params -> transform -> load
(TEST INFRASTRUCTURE ONLY; nothing in the shipped package imports this file).

What aeon's provider_base::provide does per record (src/provider.cpp:109-119, 160-216, 314-347, 489-517), built from the
other oracle modules.  cv2.imdecode is used for decoding because it is bit-identical to oracle.jpeg and far faster.
With fast=True the pixel work goes through the OpenCV binary (oracle.cv2_path) instead of the numpy restatement: the
same results, at the speed of the library the reference would spend its time in -- that is the CPU arm the benchmark
times beside the GPU path."""
import numpy as np

from . import image_ops as ops
from . import params as oparams
from . import rcnn as orcnn
from . import specgram as ospec
from . import ssd as ossd


class PipelineOracle:
    def __init__(self, config, fast=False):
        self.cfg = config
        if fast:
            from . import cv2_path
            self.px = cv2_path
        else:
            self.px = ops
        aug = (config.get("augmentation") or [{}])[0]
        self.aug = aug
        self.factory = ossd.SsdFactory(aug)
        self.video_factory = oparams.ParamFactory(aug.get("frame", {}))
        self.decode_size = config.get("decode_size", config["batch_size"])
        self.engines = oparams.slot_engines(config["random_seed"], self.decode_size)
        self.cursor = 0
        self._anchors = {}

    @staticmethod
    def decode(blob, channels=3):
        import cv2
        img = cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_COLOR if channels == 3 else cv2.IMREAD_GRAYSCALE)
        assert img is not None
        return img if channels == 3 else img[..., None]

    def image(self, etl, img, p):
        out = self.px.transform_single_image(img, p)
        h, w = etl["height"], etl["width"]
        kw = dict(channel_major=etl.get("channel_major", True), bgr_to_rgb=etl.get("bgr_to_rgb", False),
                  output_type=etl.get("output_type", "uint8_t"), mean=self.aug.get("mean"), stddev=self.aug.get("stddev"))
        if out.shape[:2] == (h, w):
            return self.px.load_image(out, **kw)
        z = ops.load_image(np.zeros((h, w, out.shape[2]), np.uint8), kw["channel_major"], kw["bgr_to_rgb"], kw["output_type"])
        roi = self.px.load_image(out, **kw)
        if kw["channel_major"]:
            z[:, :out.shape[0], :out.shape[1]] = roi
        else:
            z[:out.shape[0], :out.shape[1]] = roi
        return z

    def batch(self, records, video_frames=None):
        """records: list of tuples of bytes.  video_frames(blob) -> list of BGR frames for video elements."""
        outs = {}
        for r, rec in enumerate(records):
            g = self.engines[(self.cursor + r) % self.decode_size]
            p = None
            for etl, blob in zip(self.cfg["etl"], rec):
                name = (etl.get("name", "") + "." if etl.get("name") else "")
                if etl["type"] == "image":
                    img = self.decode(blob, etl.get("channels", 3))
                    if p is None:
                        p = self.factory.make_params(g, img.shape[1], img.shape[0], etl["width"], etl["height"])
                    outs.setdefault(name + "image", []).append(self.image(etl, img, p))
                elif etl["type"] == "pixelmask":
                    import cv2
                    mask = cv2.imdecode(np.frombuffer(blob, np.uint8), cv2.IMREAD_ANYDEPTH)   # src/etl_pixel_mask.cpp:39
                    assert mask is not None and mask.dtype == np.uint8
                    if p is None:
                        p = self.factory.make_params(g, mask.shape[1], mask.shape[0], etl["width"], etl["height"])
                    out = ops.transform_pixel_mask(mask[..., None], p)
                    assert out.shape[:2] == (etl["height"], etl["width"])
                    outs.setdefault(name + "pixelmask", []).append(ops.load_image(
                        out, etl.get("channel_major", True), False, etl.get("output_type", "uint8_t")))
                elif etl["type"] == "label":
                    v = int(np.frombuffer(blob, np.int32)[0]) if etl.get("binary") else int(blob.decode())
                    outs.setdefault(name + "label", []).append(np.array([v], ops._DTYPES[etl.get("output_type", "uint32_t")]))
                elif etl["type"] == "localization_ssd":
                    w, h, boxes = ossd.parse_annotation(blob, etl["class_names"])
                    if p is None:
                        p = self.factory.make_ssd_params(g, w, h, etl["width"], etl["height"], boxes)
                    gt = ossd.transform_boxes(boxes, p)
                    bufs = ossd.load_buffers(gt, etl["width"], etl["height"], etl.get("max_gt_boxes", 64))
                    for key, arr in zip(("image_shape", "gt_boxes", "gt_box_count", "gt_class_count", "difficult_flag"), bufs):
                        outs.setdefault(name + key, []).append(arr)
                elif etl["type"] == "localization_rcnn":
                    w, h, boxes = ossd.parse_annotation(blob, etl["class_names"])
                    if p is None:
                        p = self.factory.make_params(g, w, h, etl["width"], etl["height"])
                    anchors = self._anchors.setdefault(id(etl), orcnn.generate_anchors(etl))
                    res = orcnn.transform(etl, anchors, boxes, p, self.aug.get("fixed_scaling_factor", -1.0))  # deterministic sampling
                    for key, arr in orcnn.load(etl, len(anchors), res).items():
                        outs.setdefault(name + key, []).append(arr)
                elif etl["type"] == "boundingbox":
                    w, h, boxes = ossd.parse_annotation(blob, etl["class_names"])
                    if p is None:
                        p = self.factory.make_params(g, w, h, etl["width"], etl["height"])
                    rows = np.zeros((etl["max_bbox_count"], 16), ops._DTYPES[etl.get("output_type", "float")])
                    flat = rows.view(np.uint8).reshape(-1).view(np.float32)     # the loader writes floats from the start
                    for i, b in enumerate(ossd.transform_boxes(boxes, p)[:etl["max_bbox_count"]]):
                        flat[4 * i:4 * i + 4] = (b.xmin, b.ymin, b.xmax, b.ymax)
                    outs.setdefault(name + "boundingbox", []).append(rows)
                elif etl["type"] == "video":
                    frames = video_frames(blob)
                    fc = etl["frame"]
                    if p is None:
                        p = self.video_factory.make_params(g, frames[0].shape[1], frames[0].shape[0], fc["width"], fc["height"])
                    tx = [self.px.transform_single_image(f, p) for f in frames]
                    outs.setdefault(name + "video", []).append(ops.load_video(tx, etl["max_frame_count"]))
                elif etl["type"] == "audio":
                    # specgram::wav_to_specgram / specgram_to_cepsgram (src/specgram.cpp:26-137) on raw int16 samples
                    clip = np.frombuffer(blob, np.int16)[:etl["max_samples"]]
                    steps = (etl["max_samples"] - etl["frame_length"]) // etl["frame_stride"] + 1
                    outs.setdefault(name + "audio", []).append(ospec.log_mel(
                        clip, frame_length=etl["frame_length"], frame_stride=etl["frame_stride"], max_time_steps=steps,
                        num_filters=etl["num_filters"], sample_rate=etl["sample_rate"], window=etl.get("window_type", "hann")))
        self.cursor = (self.cursor + len(records)) % self.decode_size
        return {k: np.stack(v) for k, v in outs.items()}
