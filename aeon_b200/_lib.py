"""ctypes view of libaeon_b200.so: structures and prototypes of include/aeon_b200.h.

The shared library is the product; this module only loads it.  There is no fallback:
if the library has not been built (``python -m aeon_b200.build``) loading raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaeon_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_DECODE, ERR_IO, END = 0, -1, -2, -3, -4, -5, 1

U8, I8, I16, U16, I32, F32, F64 = range(7)
INTERP_NEAREST, INTERP_LINEAR, INTERP_CUBIC, INTERP_AREA, INTERP_LANCZOS4 = 0, 1, 2, 3, 4


class ImageDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("src_pitch", C.c_int32), ("src_pixel_stride", C.c_int32),
        ("src_w", C.c_int32), ("src_h", C.c_int32),
        ("canvas_w", C.c_int32), ("canvas_h", C.c_int32), ("canvas_x", C.c_int32), ("canvas_y", C.c_int32),
        ("crop_x", C.c_int32), ("crop_y", C.c_int32), ("crop_w", C.c_int32), ("crop_h", C.c_int32),
        ("out_w", C.c_int32), ("out_h", C.c_int32), ("interp", C.c_int32), ("flip", C.c_int32),
        ("color_enable", C.c_int32), ("color_matrix", C.c_int16 * 9), ("reserved0", C.c_int16),
        ("color_scale", C.c_float * 3),
        ("hue", C.c_int32), ("hsv_vector_cols", C.c_int32), ("contrast", C.c_float),
        ("lighting_enable", C.c_int32), ("lighting_scale", C.c_float), ("lighting_offset", C.c_int32 * 3),
        ("dst", C.c_void_p),
    ]


class ImageLayout(C.Structure):
    _fields_ = [
        ("slot_w", C.c_int32), ("slot_h", C.c_int32), ("channels", C.c_int32), ("dtype", C.c_int32),
        ("bgr_to_rgb", C.c_int32),
        ("stride_c", C.c_int64), ("stride_y", C.c_int64), ("stride_x", C.c_int64),
        ("standardize", C.c_int32), ("mean", C.c_float * 3), ("rstd", C.c_float * 3),
        ("mean64", C.c_double * 3), ("rstd64", C.c_double * 3),
    ]


class RotateDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("src_pitch", C.c_int32), ("src_pixel_stride", C.c_int32), ("width", C.c_int32),
        ("height", C.c_int32), ("angle", C.c_int32), ("nearest", C.c_int32), ("dst", C.c_void_p), ("dst_pitch", C.c_int32),
        ("dst_pixel_stride", C.c_int32),
    ]


class OrientDesc(C.Structure):
    _fields_ = RotateDesc._fields_[:5] + [("orientation", C.c_int32)] + RotateDesc._fields_[7:]


class ResizeDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("src_pitch", C.c_int32), ("src_pixel_stride", C.c_int32), ("src_w", C.c_int32), ("src_h", C.c_int32),
        ("canvas_x", C.c_int32), ("canvas_y", C.c_int32), ("crop_x", C.c_int32), ("crop_y", C.c_int32), ("crop_w", C.c_int32),
        ("crop_h", C.c_int32), ("interp", C.c_int32), ("out_w", C.c_int32), ("out_h", C.c_int32), ("dst", C.c_void_p),
        ("dst_pitch", C.c_int32), ("dst_pixel_stride", C.c_int32), ("channels", C.c_int32), ("reserved0", C.c_int32),
    ]


class RcnnConfig(C.Structure):
    _fields_ = [
        ("width", C.c_int32), ("height", C.c_int32), ("base_size", C.c_int32), ("n_ratios", C.c_int32), ("n_scales", C.c_int32),
        ("scaling_factor", C.c_float), ("ratios", C.c_float * 8), ("scales", C.c_float * 8),
    ]


class RcnnDesc(C.Structure):
    _fields_ = [
        ("gt_boxes", C.c_void_p), ("n_gt", C.c_int32), ("im_width", C.c_int32), ("im_height", C.c_int32),
        ("labels", C.c_void_p), ("best_box", C.c_void_p),
    ]


class JpegDesc(C.Structure):
    _fields_ = [
        ("coef", C.c_void_p * 3), ("quant", C.c_void_p * 3),
        ("width", C.c_int32), ("height", C.c_int32), ("ncomp", C.c_int32),
        ("hs", C.c_int32 * 3), ("vs", C.c_int32 * 3),
        ("blocks_w", C.c_int32 * 3), ("blocks_h", C.c_int32 * 3),
        ("dst", C.c_void_p), ("dst_pitch", C.c_int32), ("dst_pixel_stride", C.c_int32),
    ]


class EntropyDesc(C.Structure):
    _fields_ = [
        ("scan", C.c_void_p), ("scan_size", C.c_uint32), ("ncomp", C.c_int32), ("tables", C.c_void_p),
        ("hs", C.c_int32 * 3), ("vs", C.c_int32 * 3), ("dc_table", C.c_int32 * 3), ("ac_table", C.c_int32 * 3),
        ("mcux", C.c_int32), ("mcuy", C.c_int32), ("roi", C.c_int32 * 4), ("restart_interval", C.c_int32),
        ("reserved0", C.c_int32), ("coef", C.c_void_p * 3), ("status", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_uint64),
    ]


class JpegInfo(C.Structure):
    _fields_ = [
        ("width", C.c_int32), ("height", C.c_int32), ("ncomp", C.c_int32),
        ("hs", C.c_int32 * 3), ("vs", C.c_int32 * 3),
        ("blocks_w", C.c_int32 * 3), ("blocks_h", C.c_int32 * 3),
        ("coef_count", C.c_int64 * 3), ("orientation", C.c_int32), ("reserved0", C.c_int32),
    ]


class SpecgramDesc(C.Structure):
    _fields_ = [("samples", C.c_void_p), ("n_samples", C.c_int32), ("dst", C.c_void_p)]


class SpecgramConfig(C.Structure):
    _fields_ = [("frame_length", C.c_int32), ("frame_stride", C.c_int32), ("max_time_steps", C.c_int32),
                ("num_filters", C.c_int32), ("sample_rate", C.c_int32), ("window", C.c_int32),
                ("num_cepstra", C.c_int32), ("reserved0", C.c_int32)]


class KernelProfile(C.Structure):
    _fields_ = [("launches", C.c_int64), ("ms", C.c_double), ("algorithmic_bytes", C.c_int64)]


KERNEL_KINDS = ("jpeg_entropy", "jpeg_backend", "aug_pack", "specgram", "other")

# name -> (restype, argtypes); every symbol the header declares
PROTOTYPES = {
    "aeonb_last_error": (C.c_char_p, []),
    "aeonb_version": (C.c_char_p, []),
    "aeonb_ctx_create": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "aeonb_ctx_destroy": (None, [C.c_void_p]),
    "aeonb_ctx_stream": (C.c_void_p, [C.c_void_p]),
    "aeonb_ctx_synchronize": (C.c_int, [C.c_void_p]),
    "aeonb_ctx_profile": (C.c_int, [C.c_void_p, C.c_int]),
    "aeonb_ctx_profile_read": (C.c_int, [C.c_void_p, C.POINTER(KernelProfile)]),
    "aeonb_image_batch": (C.c_int, [C.c_void_p, C.POINTER(ImageDesc), C.c_int, C.POINTER(ImageLayout)]),
    "aeonb_image_batch_bytes": (C.c_int64, [C.POINTER(ImageDesc), C.c_int, C.POINTER(ImageLayout)]),
    "aeonb_image_batch_noalloc": (C.c_int, [C.POINTER(ImageDesc), C.c_int, C.POINTER(ImageLayout), C.c_void_p]),
    "aeonb_rotate_batch": (C.c_int, [C.c_void_p, C.POINTER(RotateDesc), C.c_int]),
    "aeonb_orient_batch": (C.c_int, [C.c_void_p, C.POINTER(OrientDesc), C.c_int]),
    "aeonb_resize_batch": (C.c_int, [C.c_void_p, C.POINTER(ResizeDesc), C.c_int]),
    "aeonb_jpeg_backend_batch": (C.c_int, [C.c_void_p, C.POINTER(JpegDesc), C.c_int]),
    "aeonb_jpeg_backend_bytes": (C.c_int64, [C.POINTER(JpegDesc), C.c_int]),
    "aeonb_jpeg_entropy_batch": (C.c_int, [C.c_void_p, C.POINTER(EntropyDesc), C.c_int]),
    "aeonb_jpeg_entropy_scratch_bytes": (C.c_int64, [C.POINTER(EntropyDesc)]),
    "aeonb_jpeg_entropy_prepare": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(JpegInfo), C.POINTER(C.c_uint16),
                                             C.POINTER(C.c_uint8), C.POINTER(EntropyDesc), C.POINTER(C.c_size_t)]),
    "aeonb_specgram_batch": (C.c_int, [C.c_void_p, C.POINTER(SpecgramDesc), C.c_int, C.POINTER(SpecgramConfig)]),
    "aeonb_specgram_bytes": (C.c_int64, [C.POINTER(SpecgramDesc), C.c_int, C.POINTER(SpecgramConfig)]),
    "aeonb_jpeg_parse": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(JpegInfo)]),
    "aeonb_jpeg_entropy_decode": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "aeonb_jpeg_roi_for_crop": (C.c_int, [C.POINTER(JpegInfo), C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int32)]),
    "aeonb_jpeg_entropy_decode_roi": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.c_void_p),
                                                C.POINTER(C.c_void_p)]),
    "aeonb_png_info": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "aeonb_png_decode_bgr": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "aeonb_png_decode_grey": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "aeonb_rcnn_anchor_count": (C.c_int64, [C.POINTER(RcnnConfig)]),
    "aeonb_rcnn_anchors": (C.c_int, [C.POINTER(RcnnConfig), C.c_void_p]),
    "aeonb_rcnn_label_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(RcnnDesc), C.c_int, C.c_float, C.c_float]),
    "aeonb_draw_params": (C.c_int, [C.c_char_p, C.c_uint32, C.c_int, C.c_int, C.POINTER(C.c_int32),
                                    C.POINTER(C.c_int32), C.c_int, C.c_int, C.POINTER(C.c_double)]),
    "aeonb_draw_ssd_params": (C.c_int, [C.c_char_p, C.c_uint32, C.c_int, C.c_int, C.POINTER(C.c_int32),
                                        C.POINTER(C.c_int32), C.c_int, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_float),
                                        C.POINTER(C.c_double)]),
    "aeonb_box_overlap": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "aeonb_transform_boxes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "aeonb_ssd_load_boxes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "aeonb_image_desc_set_photometric": (C.c_int, [C.POINTER(ImageDesc), C.c_float, C.c_float, C.c_float, C.c_int,
                                                   C.POINTER(C.c_float), C.c_float]),
    "aeonb_provider_create": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "aeonb_provider_destroy": (None, [C.c_void_p]),
    "aeonb_provider_input_count": (C.c_int, [C.c_void_p]),
    "aeonb_provider_output_count": (C.c_int, [C.c_void_p]),
    "aeonb_provider_output_name": (C.c_char_p, [C.c_void_p, C.c_int]),
    "aeonb_provider_output_shape": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "aeonb_provider_output_bytes": (C.c_int64, [C.c_void_p, C.c_int]),
    "aeonb_provider_run": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_int,
                                     C.POINTER(C.c_void_p), C.c_int]),
    "aeonb_provider_run_async": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_int,
                                           C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int64)]),
    "aeonb_provider_wait": (C.c_int, [C.c_void_p, C.c_int64]),
    "aeonb_provider_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "aeonb_loader_create": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]),
    "aeonb_loader_destroy": (None, [C.c_void_p]),
    "aeonb_loader_record_count": (C.c_int, [C.c_void_p]),
    "aeonb_loader_batch_size": (C.c_int, [C.c_void_p]),
    "aeonb_loader_batch_count": (C.c_int, [C.c_void_p]),
    "aeonb_loader_output_count": (C.c_int, [C.c_void_p]),
    "aeonb_loader_output_name": (C.c_char_p, [C.c_void_p, C.c_int]),
    "aeonb_loader_output_shape": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "aeonb_loader_axis_names": (C.c_char_p, [C.c_void_p, C.c_int]),
    "aeonb_loader_config": (C.c_char_p, [C.c_void_p]),
    "aeonb_loader_next": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "aeonb_loader_reset": (C.c_int, [C.c_void_p]),
    "aeonb_loader_position": (C.c_int, [C.c_void_p]),
    "aeonb_stream_create": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "aeonb_stream_destroy": (None, [C.c_void_p]),
    "aeonb_stream_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                    C.POINTER(C.c_int32), C.c_char_p, C.c_size_t]),
    "aeonb_stream_next": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "aeonb_stream_reset": (C.c_int, [C.c_void_p]),
    "aeonb_node_record_indices": (C.c_int64, [C.c_int64, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64)]),
}

# exported for the test suite only, not part of the public header
TEST_HOOKS = {
    "aeonb_selftest_worker_pool": (C.c_int64, [C.c_int, C.c_int]),
}

_lib = None
MISSING = []  # declared in the header but absent from the built library (must stay empty)


class AeonError(RuntimeError):
    """A failed library call (aeon raises std::runtime_error / std::invalid_argument; python sees RuntimeError)."""

    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


def load():
    """Load the shared library (once) and attach the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("libaeon_b200.so is not built; run `python -m aeon_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in list(PROTOTYPES.items()) + list(TEST_HOOKS.items()):
        fn = getattr(lib, name, None)
        if fn is None:
            MISSING.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    if MISSING:
        raise ImportError("libaeon_b200.so lacks %s; rebuild it with `python -m aeon_b200.build`" % ", ".join(MISSING))
    _lib = lib
    return lib


def check(status):
    if status < 0:
        raise AeonError(status, load().aeonb_last_error().decode("utf-8", "replace"))
    return status
