"""Thin python callers of the batch-kernel entry points (device tensors in, device tensors out).

torch is used for device memory only; every computation happens inside libaeon_b200.so.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib as L

_TORCH_DTYPE = {L.U8: torch.uint8, L.I8: torch.int8, L.I16: torch.int16, L.U16: torch.int16, L.I32: torch.int32,
                L.F32: torch.float32, L.F64: torch.float64}
DTYPE_BY_NAME = {"uint8_t": L.U8, "int8_t": L.I8, "char": L.I8, "int16_t": L.I16, "uint16_t": L.U16,
                 "int32_t": L.I32, "uint32_t": L.I32, "float": L.F32, "double": L.F64}
DTYPE_SIZE = {L.U8: 1, L.I8: 1, L.I16: 2, L.U16: 2, L.I32: 4, L.F32: 4, L.F64: 8}
INTERP_BY_NAME = {"NEAREST": L.INTERP_NEAREST, "LINEAR": L.INTERP_LINEAR}


class Context:
    """One GPU context of the library (aeonb_ctx)."""

    def __init__(self, device=0):
        self.lib = L.load()
        self.device = int(device)
        # The library runs on a stream torch knows about, so tensors allocated under
        # `with torch.cuda.stream(ctx.torch_stream)` are ordered with the kernels.
        self.torch_stream = torch.cuda.Stream(device=self.device)
        h = C.c_void_p()
        L.check(self.lib.aeonb_ctx_create(self.device, C.c_void_p(self.torch_stream.cuda_stream), C.byref(h)))
        self.handle = h

    def synchronize(self):
        L.check(self.lib.aeonb_ctx_synchronize(self.handle))

    def profile(self, enable=True):
        """Switches the per-kernel timing of this context on (clearing the totals) or off."""
        L.check(self.lib.aeonb_ctx_profile(self.handle, int(bool(enable))))

    def profile_read(self):
        """{kernel kind: {"launches", "ms", "algorithmic_bytes"}} of the launches since the profile was switched on."""
        out = (L.KernelProfile * len(L.KERNEL_KINDS))()
        L.check(self.lib.aeonb_ctx_profile_read(self.handle, out))
        return {name: {"launches": int(out[i].launches), "ms": float(out[i].ms), "algorithmic_bytes": int(out[i].algorithmic_bytes)}
                for i, name in enumerate(L.KERNEL_KINDS)}

    @property
    def stream(self):
        return self.lib.aeonb_ctx_stream(self.handle)

    def close(self):
        if self.handle:
            self.lib.aeonb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_layout(slot_w, slot_h, dtype=L.U8, channel_major=True, bgr_to_rgb=False, mean=None, stddev=None,
                strides=None):
    lay = L.ImageLayout()
    lay.slot_w, lay.slot_h, lay.channels, lay.dtype = slot_w, slot_h, 3, dtype
    lay.bgr_to_rgb = int(bool(bgr_to_rgb))
    if strides is None:
        strides = (slot_h * slot_w, slot_w, 1) if channel_major else (1, slot_w * 3, 3)
    lay.stride_c, lay.stride_y, lay.stride_x = strides
    if mean is not None and len(mean):
        lay.standardize = 1
        for c in range(3):
            r = 1.0 / stddev[c] if stddev[c] else 1.0
            lay.mean[c], lay.rstd[c] = mean[c], r
            lay.mean64[c], lay.rstd64[c] = mean[c], r
    return lay


def fill_desc(desc, src, p, dst_ptr, lib=None):
    """Fill an ImageDesc from a source tensor (H x W x 3|4 uint8 on the GPU, or None) and a parameter
    object with aeon's ``augment::image::params`` fields (see oracle.image_ops.ImageParams)."""
    lib = lib or L.load()
    desc.dst = dst_ptr
    if src is None:
        desc.src = None
        return
    h, w, pix = src.shape
    desc.src = src.data_ptr()
    desc.src_pitch = src.stride(0)
    desc.src_pixel_stride = pix
    desc.src_w, desc.src_h = w, h
    if float(np.float32(p.expand_ratio)) > 1.0:
        desc.canvas_w, desc.canvas_h = p.expand_size
        desc.canvas_x, desc.canvas_y = p.expand_offset
    elif p.padding and tuple(p.padding_crop_offset) != (p.padding, p.padding):
        desc.canvas_w, desc.canvas_h = w + 2 * p.padding, h + 2 * p.padding
        desc.canvas_x = desc.canvas_y = p.padding
    else:
        desc.canvas_w, desc.canvas_h, desc.canvas_x, desc.canvas_y = w, h, 0, 0
    x, y, cw, ch = p.cropbox
    if p.padding and tuple(p.padding_crop_offset) != (p.padding, p.padding):
        x, y = p.padding_crop_offset
    desc.crop_x, desc.crop_y, desc.crop_w, desc.crop_h = x, y, cw, ch
    desc.out_w, desc.out_h = p.output_size
    desc.interp = INTERP_BY_NAME[p.interpolation_method.upper()]
    desc.flip = int(bool(p.flip))
    light = (C.c_float * 3)(*[float(v) for v in p.lighting]) if len(p.lighting) else None
    L.check(lib.aeonb_image_desc_set_photometric(C.byref(desc), float(p.contrast), float(p.brightness),
                                                 float(p.saturation), int(p.hue), light, float(p.color_noise_std)))


def image_batch(ctx, sources, params, out, layout, record_stride=None):
    """Run the image kernel: sources[i] -> out[i].  `out` is a device tensor whose first dim is the batch."""
    n = len(sources)
    descs = (L.ImageDesc * n)()
    esz = out.element_size()
    stride = record_stride if record_stride is not None else out.stride(0)
    for i in range(n):
        fill_desc(descs[i], sources[i], params[i], out.data_ptr() + i * stride * esz, ctx.lib)
    L.check(ctx.lib.aeonb_image_batch(ctx.handle, descs, n, C.byref(layout)))
    return descs


def png_decode(data, grey=False):
    """Host PNG decode -> H x W x 3 uint8 numpy array (B,G,R), as cv2.imdecode(IMREAD_COLOR) returns it; with `grey`
    the H x W picture of cv2.imdecode(IMREAD_GRAYSCALE)."""
    lib = L.load()
    w, h = C.c_int32(), C.c_int32()
    buf = (C.c_char * len(data)).from_buffer_copy(data)
    L.check(lib.aeonb_png_info(buf, len(data), C.byref(w), C.byref(h)))
    if grey:
        out = np.zeros((h.value, w.value), np.uint8)
        L.check(lib.aeonb_png_decode_grey(buf, len(data), out.ctypes.data, w.value))
        return out
    out = np.zeros((h.value, w.value, 3), np.uint8)
    L.check(lib.aeonb_png_decode_bgr(buf, len(data), out.ctypes.data, w.value * 3))
    return out


def rcnn_config(width, height, base_size=16, scaling_factor=1.0 / 16.0, ratios=(0.5, 1, 2), scales=(8, 16, 32)):
    c = L.RcnnConfig()
    c.width, c.height, c.base_size, c.scaling_factor = width, height, base_size, scaling_factor
    c.n_ratios, c.n_scales = len(ratios), len(scales)
    for i, v in enumerate(ratios):
        c.ratios[i] = v
    for i, v in enumerate(scales):
        c.scales[i] = v
    return c


def rcnn_anchors(cfg):
    """Host anchor table of localization_rcnn -> (count, 4) float32 array."""
    lib = L.load()
    n = int(lib.aeonb_rcnn_anchor_count(C.byref(cfg)))
    out = np.zeros((n, 4), np.float32)
    L.check(lib.aeonb_rcnn_anchors(C.byref(cfg), out.ctypes.data))
    return out


def rcnn_label_batch(ctx, anchors, gt_boxes, im_sizes, negative_overlap=0.3, positive_overlap=0.7):
    """Labels (-1 / 0 / 1) and best-box index per anchor for each record.  anchors: (A, 4) float32; gt_boxes: list of
    (K_i, 4) float32 arrays; im_sizes: list of (width, height)."""
    import torch
    dev = torch.device("cuda", ctx.device)
    n, A = len(gt_boxes), len(anchors)
    with torch.cuda.stream(ctx.torch_stream):
        a = torch.from_numpy(np.ascontiguousarray(anchors, np.float32)).to(dev)
        labels = torch.full((n, A), 7, dtype=torch.int8, device=dev)
        best = torch.full((n, A), -7, dtype=torch.int16, device=dev)
        keep = []
        descs = (L.RcnnDesc * n)()
        for i, (g, (w, h)) in enumerate(zip(gt_boxes, im_sizes)):
            g = np.ascontiguousarray(g, np.float32).reshape(-1, 4)
            t = torch.from_numpy(g).to(dev) if len(g) else None
            keep.append(t)
            descs[i].gt_boxes, descs[i].n_gt = (t.data_ptr() if t is not None else None), len(g)
            descs[i].im_width, descs[i].im_height = int(w), int(h)
            descs[i].labels, descs[i].best_box = labels[i].data_ptr(), best[i].data_ptr()
        ctx.torch_stream.synchronize()
        L.check(ctx.lib.aeonb_rcnn_label_batch(ctx.handle, a.data_ptr(), A, descs, n, negative_overlap, positive_overlap))
        ctx.synchronize()
    return labels.cpu().numpy(), best.cpu().numpy()


def jpeg_parse(data):
    info = L.JpegInfo()
    buf = (C.c_char * len(data)).from_buffer_copy(data)
    L.check(L.load().aeonb_jpeg_parse(buf, len(data), C.byref(info)))
    return info


def jpeg_entropy_decode(data):
    """Host entropy decode -> (info, [coef planes as int16 numpy], [quant tables as uint16 numpy])."""
    lib = L.load()
    info = jpeg_parse(data)
    coefs = [np.zeros(max(int(info.coef_count[c]), 1), np.int16) for c in range(3)]
    quants = [np.zeros(64, np.uint16) for _ in range(3)]
    cp = (C.c_void_p * 3)(*[c.ctypes.data for c in coefs])
    qp = (C.c_void_p * 3)(*[q.ctypes.data for q in quants])
    buf = (C.c_char * len(data)).from_buffer_copy(data)
    L.check(lib.aeonb_jpeg_entropy_decode(buf, len(data), cp, qp))
    return info, coefs[:info.ncomp], quants[:info.ncomp]


def jpeg_entropy_decode_device(ctx, encoded, rois=None, parallel=True):
    """Device entropy decode of JPEG byte strings: with `parallel` a thread block per stream (streams with
    restart markers still take the one-warp serial kernel), without it the serial kernel for all.

    Returns a list of (info, [coef planes as int16 tensors], quant uint16 numpy (3 x 64), status int) per
    record; with `rois` (MCU rectangles) the planes are the compact region planes."""
    dev = torch.device("cuda", ctx.device)
    n = len(encoded)
    descs = (L.EntropyDesc * n)()
    status = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    keep, results = [], []
    for i, data in enumerate(encoded):
        info = L.JpegInfo()
        quant = np.zeros(192, np.uint16)
        tables = np.zeros(1088, np.uint8)
        off = C.c_size_t()
        buf = (C.c_char * len(data)).from_buffer_copy(data)
        L.check(ctx.lib.aeonb_jpeg_entropy_prepare(buf, len(data), C.byref(info), quant.ctypes.data_as(C.POINTER(C.c_uint16)),
                                                   tables.ctypes.data_as(C.POINTER(C.c_uint8)), C.byref(descs[i]),
                                                   C.byref(off)))
        d = descs[i]
        scan = torch.from_numpy(np.frombuffer(data, np.uint8)[off.value:off.value + d.scan_size].copy()).to(dev)
        tab = torch.from_numpy(tables).to(dev)
        if rois is not None and rois[i] is not None:
            for k in range(4):
                d.roi[k] = int(rois[i][k])
        planes = []
        for c in range(info.ncomp):
            nb = (d.roi[2] - d.roi[0]) * d.hs[c] * (d.roi[3] - d.roi[1]) * d.vs[c]
            t = torch.full((nb * 64,), 0x5555, dtype=torch.int16, device=dev)
            planes.append(t)
            d.coef[c] = t.data_ptr()
        d.scan, d.tables = scan.data_ptr(), tab.data_ptr()
        d.status = status.data_ptr() + 4 * i
        keep += [scan, tab]
        if parallel:
            nbytes = int(ctx.lib.aeonb_jpeg_entropy_scratch_bytes(C.byref(d)))
            work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            keep.append(work)
            d.scratch, d.scratch_bytes = work.data_ptr(), nbytes
        results.append([info, planes, quant.reshape(3, 64)])
    torch.cuda.synchronize(dev)
    L.check(ctx.lib.aeonb_jpeg_entropy_batch(ctx.handle, descs, n))
    ctx.synchronize()
    st = status.cpu().numpy()
    return [(info, planes, quant, int(st[i])) for i, (info, planes, quant) in enumerate(results)]


def jpeg_decode_batch(ctx, encoded, pixel_stride=3):
    """Decode JPEG byte strings: host entropy decode, device back end.  Returns H x W x pixel_stride tensors."""
    dev = torch.device("cuda", ctx.device)
    torch.cuda.synchronize(dev)
    n = len(encoded)
    descs = (L.JpegDesc * n)()
    keep, outs, infos = [], [], []
    for i, data in enumerate(encoded):
        info, coefs, quants = jpeg_entropy_decode(data)
        d = descs[i]
        d.width, d.height, d.ncomp = info.width, info.height, info.ncomp
        for c in range(info.ncomp):
            ct = torch.from_numpy(coefs[c]).to(dev)
            qt = torch.from_numpy(quants[c].view(np.int16)).to(dev)
            keep += [ct, qt]
            d.coef[c], d.quant[c] = ct.data_ptr(), qt.data_ptr()
            d.hs[c], d.vs[c] = info.hs[c], info.vs[c]
            d.blocks_w[c], d.blocks_h[c] = info.blocks_w[c], info.blocks_h[c]
        pitch = (info.width * pixel_stride + 15) // 16 * 16
        buf = torch.zeros((info.height, pitch), dtype=torch.uint8, device=dev)
        d.dst, d.dst_pitch, d.dst_pixel_stride = buf.data_ptr(), pitch, pixel_stride
        outs.append(torch.as_strided(buf, (info.height, info.width, pixel_stride), (pitch, pixel_stride, 1)))
        keep.append(buf)
        infos.append(info)
    torch.cuda.synchronize(dev)
    L.check(ctx.lib.aeonb_jpeg_backend_batch(ctx.handle, descs, n))
    # EXIF orientation, as cv::imdecode applies it after decoding
    turned = [i for i in range(n) if infos[i].orientation != 1]
    if turned:
        od = (L.OrientDesc * len(turned))()
        for k, i in enumerate(turned):
            info = infos[i]
            w, h = (info.height, info.width) if info.orientation >= 5 else (info.width, info.height)
            pitch = (w * pixel_stride + 15) // 16 * 16
            buf = torch.zeros((h, pitch), dtype=torch.uint8, device=dev)
            keep.append(buf)
            o = od[k]
            o.src, o.src_pitch, o.src_pixel_stride = descs[i].dst, descs[i].dst_pitch, pixel_stride
            o.width, o.height, o.orientation = info.width, info.height, info.orientation
            o.dst, o.dst_pitch, o.dst_pixel_stride = buf.data_ptr(), pitch, pixel_stride
            outs[i] = torch.as_strided(buf, (h, w, pixel_stride), (pitch, pixel_stride, 1))
        L.check(ctx.lib.aeonb_orient_batch(ctx.handle, od, len(turned)))
    ctx.synchronize()
    return outs, descs
