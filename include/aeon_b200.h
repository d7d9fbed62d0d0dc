/*
 * aeon_b200 -- C ABI of the B200 implementation of aeon's per-record ETL hot path.
 *
 * Every entry point takes plain pointers and sizes, returns 0 (AEONB_OK) or a
 * negative status, and never throws.  aeonb_last_error() gives the message of the
 * last failure on the calling thread.  Citations name the aeon source the entry
 * point stands in for (paths relative to the aeon tree).
 *
 * Levels, from the GPU up:
 *   1. batch kernels over device-resident data (aeonb_jpeg_entropy_batch, aeonb_jpeg_backend_batch,
 *      aeonb_orient_batch, aeonb_rotate_batch, aeonb_image_batch, aeonb_specgram_batch): one launch per batch;
 *   2. host helpers: header parsing, the host Huffman decoder (progressive files, or by choice), PNG decoding,
 *      AVI index parsing, augmentation parameter draws;
 *   3. the provider: encoded records in host memory -> augmented batch, i.e. what
 *      aeon's batch_decoder + provider_interface::provide do per decode chunk;
 *   4. the loader: manifest -> batches, i.e. aeon's loader / DataLoader iterator.
 */
#ifndef AEON_B200_H
#define AEON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AEONB_OK 0
#define AEONB_ERR_INVALID (-1)     /* bad argument or configuration (aeon: std::invalid_argument) */
#define AEONB_ERR_CUDA (-2)        /* a CUDA runtime call failed */
#define AEONB_ERR_UNSUPPORTED (-3) /* valid request outside what the kernels implement */
#define AEONB_ERR_DECODE (-4)      /* corrupt or unsupported encoded record (aeon: std::runtime_error) */
#define AEONB_ERR_IO (-5)          /* file or manifest problem */
#define AEONB_END 1                /* loader iteration finished (aeon: iterator == end) */

typedef struct aeonb_ctx      aeonb_ctx;      /* one GPU: device id, stream, descriptor staging, scratch arena */
typedef struct aeonb_provider aeonb_provider; /* aeon provider_base + batch_decoder for one configuration */
typedef struct aeonb_loader   aeonb_loader;   /* aeon loader_local */

const char* aeonb_last_error(void);
const char* aeonb_version(void);

/* ------------------------------------------------------------------------------------------------
 * Context
 * ---------------------------------------------------------------------------------------------- */

/* Creates the per-GPU context.  `stream` is a cudaStream_t to run on, or NULL to let the
 * context create its own non-blocking stream. */
int  aeonb_ctx_create(int device, void* stream, aeonb_ctx** out);
void aeonb_ctx_destroy(aeonb_ctx* ctx);
void* aeonb_ctx_stream(aeonb_ctx* ctx);
int  aeonb_ctx_synchronize(aeonb_ctx* ctx);

/* Per-kernel timing of a context: with the profile on, every batch call records a pair of CUDA events around its
 * kernel on the context's stream.  aeonb_ctx_profile_read waits for the stream, adds the finished launches up and
 * fills one entry per kernel kind: launches, summed device time, and the algorithmic bytes of those launches (each
 * unique input byte once + each output byte once: what a bandwidth roofline divides by the time).  Switching the
 * profile on clears the totals.  Works through every path that uses the context, the provider included. */
enum aeonb_kernel_kind
{
    AEONB_KERNEL_ENTROPY = 0,      /* jpeg_entropy_parallel_kernel / jpeg_entropy_kernel */
    AEONB_KERNEL_JPEG_BACKEND = 1, /* jpeg_backend_kernel */
    AEONB_KERNEL_IMAGE = 2,        /* aug_pack_kernel */
    AEONB_KERNEL_SPECGRAM = 3,     /* specgram_kernel / specgram_generic_kernel */
    AEONB_KERNEL_OTHER = 4,        /* rotate, orient, resize passes, rcnn labels */
    AEONB_KERNEL_KINDS = 5
};
typedef struct aeonb_kernel_profile
{
    int64_t launches;
    double  ms;
    int64_t algorithmic_bytes;
} aeonb_kernel_profile;
int aeonb_ctx_profile(aeonb_ctx* ctx, int enable);
int aeonb_ctx_profile_read(aeonb_ctx* ctx, aeonb_kernel_profile out[AEONB_KERNEL_KINDS]);

/* ------------------------------------------------------------------------------------------------
 * 1a. Image augmentation + packing kernel
 *     replaces image::transformer::transform_single_image (src/etl_image.cpp:146-202),
 *     photometric::cbsjitter / lighting (src/image.cpp:336-406) and image::loader::load
 *     (src/etl_image.cpp:246-341); with frame strides also video::loader::load
 *     (src/etl_video.cpp:76-107).
 * ---------------------------------------------------------------------------------------------- */

enum aeonb_dtype
{
    AEONB_U8 = 0,
    AEONB_I8 = 1,
    AEONB_I16 = 2,
    AEONB_U16 = 3,
    AEONB_I32 = 4,
    AEONB_F32 = 5,
    AEONB_F64 = 6
};

enum aeonb_interp
{
    AEONB_INTERP_NEAREST = 0,
    AEONB_INTERP_LINEAR = 1,
    AEONB_INTERP_CUBIC = 2, /* CUBIC, AREA and LANCZOS4 only through aeonb_resize_batch; aeonb_image_batch takes NEAREST and LINEAR */
    AEONB_INTERP_AREA = 3,
    AEONB_INTERP_LANCZOS4 = 4
};

/* One image (or video frame) to transform.  All coordinates are pixels.
 * The source is an 8-bit interleaved image in device memory (B,G,R[,x] per pixel).
 * The "canvas" models aeon's expand / padding: a zero image of canvas_w x canvas_h with
 * the source pasted at (canvas_x, canvas_y); without expand the canvas equals the source.
 * The crop box is given in canvas coordinates and is resized to out_w x out_h. */
typedef struct aeonb_image_desc
{
    const uint8_t* src;  /* device pointer; NULL produces an all-zero image (video padding frame) */
    int32_t src_pitch;   /* bytes between source rows */
    int32_t src_pixel_stride; /* 3 (BGR) or 4 (BGRx) bytes per pixel */
    int32_t src_w, src_h;
    int32_t canvas_w, canvas_h, canvas_x, canvas_y;
    int32_t crop_x, crop_y, crop_w, crop_h;
    int32_t out_w, out_h; /* size after resize; <= slot size, the rest of the slot is zero-filled */
    int32_t interp;       /* aeonb_interp */
    int32_t flip;         /* horizontal flip, applied last */
    /* photometric (src/image.cpp:358-406); every stage rounds to uint8 before the next */
    int32_t color_enable; /* 0: off; 1: dense 3x3 color_matrix; 2: diagonal matrix, per-channel color_scale */
    int16_t color_matrix[9]; /* round(m*1024), row-major, BGR order: the 10-bit form cv::transform uses */
    int16_t reserved0;
    float   color_scale[3];  /* diagonal case (brightness alone): cv::transform then scales each channel in float */
    int32_t hue;          /* added to H (units of 2 degrees); 0 disables the HSV round trip */
    int32_t hsv_vector_cols; /* columns [0, hsv_vector_cols) of each row truncate in HSV->BGR, the rest round */
    float   contrast;     /* 1.0f disables; otherwise x*c + (1-c)*channel mean of the image */
    int32_t lighting_enable;
    float   lighting_scale;     /* 1/(1+std) */
    int32_t lighting_offset[3]; /* round(pixel_c/(1+std)), BGR order */
    void*   dst;          /* device pointer to this record's slot (element (0,0,0)) */
} aeonb_image_desc;

/* Output slot geometry shared by the whole batch. */
typedef struct aeonb_image_layout
{
    int32_t slot_w, slot_h; /* spatial size of the slot */
    int32_t channels;       /* 3, or 1: only the first plane is written (grey pictures arrive as B = G = R) */
    int32_t dtype;          /* aeonb_dtype of the output elements */
    int32_t bgr_to_rgb;     /* reverse the channel order on output */
    int64_t stride_c, stride_y, stride_x; /* element strides of the slot; CHW: (H*W, W, 1); HWC: (1, W*C, C);
                                             video CTHW frame: (T*H*W, W, 1) */
    int32_t standardize;    /* apply x*(1/255) - mean[c], then *rstd[c] (src/image.cpp:129-174) */
    float   mean[3];        /* indexed by OUTPUT channel */
    float   rstd[3];        /* 1/std, or 1.0f where std == 0 */
    double  mean64[3];      /* same for AEONB_F64 output */
    double  rstd64[3];
} aeonb_image_layout;

/* Transforms n images with one kernel launch on the context's stream.  `descs` is host memory
 * and may be reused as soon as the call returns.  Asynchronous with respect to the host. */
int aeonb_image_batch(aeonb_ctx* ctx, const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout);

/* Bytes the kernel must read and write for this batch (unique source bytes inside the crop
 * boxes + output bytes): the figure a bandwidth roofline is computed from. */
int64_t aeonb_image_batch_bytes(const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout);

/* Same transformation as aeonb_image_batch for callers that are not allowed to allocate memory
 * (code running where the host framework forbids allocator calls, processes with a memory budget
 * fixed at start-up, loops that cannot tolerate the synchronisation an allocation can cause).
 * It has no counterpart in the reference.  It needs no context: it runs on the CURRENT device and
 * on `stream` (a cudaStream_t, NULL for the default stream), and calls neither cudaMalloc /
 * cudaFree nor any allocating library routine.  The device copy of the descriptors lives in a
 * fixed array inside the library (about 76 KB per GPU that loads the library, held until exit),
 * hence the limit of AEONB_NOALLOC_MAX_RECORDS (512) records per call; larger n is rejected with
 * AEONB_ERR_INVALID.  The first call on a device looks up the array's device address; make that
 * first call before starting any stream capture.  All calls share the one array: two calls whose
 * GPU work can overlap (different streams, or different host threads) race on it, so serialise
 * them.  `descs` must stay valid and unchanged until the call returns when it is pageable host
 * memory -- the copy of a pageable array is staged by the driver and the call then waits for it on
 * the host -- and until the stream has consumed the copy when it is pinned host memory (the call
 * then returns at once). */
#define AEONB_NOALLOC_MAX_RECORDS 512
int aeonb_image_batch_noalloc(const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout, void* stream);

/* Rotation pre-pass: image::rotate (src/image.cpp:53-75), i.e. cv::warpAffine with the matrix of
 * cv::getRotationMatrix2D(Point2i(width/2, height/2), angle, 1.0), INTER_LINEAR, BORDER_CONSTANT 0, same size.
 * aeon rotates the decoded picture before every other step (src/etl_image.cpp:150-151); the rotated picture is
 * then the source of aeonb_image_batch. */
typedef struct aeonb_rotate_desc
{
    const uint8_t* src;      /* device: interleaved B,G,R[,x] picture */
    int32_t src_pitch, src_pixel_stride;
    int32_t width, height;
    int32_t angle;           /* degrees, counter-clockwise */
    int32_t nearest;         /* 0: INTER_LINEAR (image::rotate's default); 1: INTER_NEAREST (interpolate == false, as the
                                pixelmask / depthmap transformers call it, src/etl_pixel_mask.cpp:71-73) */
    uint8_t* dst;            /* device: rotated picture, same size */
    int32_t dst_pitch, dst_pixel_stride;
} aeonb_rotate_desc;

int aeonb_rotate_batch(aeonb_ctx* ctx, const aeonb_rotate_desc* descs, int n);

/* EXIF orientation pass: what cv::imdecode (src/etl_image.cpp:90) applies after decoding when the file carries an
 * orientation tag other than 1: 2 mirror, 3 half turn, 4 flip, 5 transpose, 6 quarter turn clockwise, 7 transverse,
 * 8 quarter turn counter-clockwise.  width/height are those of the source; the destination is height x width for 5..8. */
typedef struct aeonb_orient_desc
{
    const uint8_t* src;      /* device: interleaved B,G,R[,x] picture as stored */
    int32_t src_pitch, src_pixel_stride;
    int32_t width, height;
    int32_t orientation;     /* 1..8 */
    uint8_t* dst;            /* device */
    int32_t dst_pitch, dst_pixel_stride;
} aeonb_orient_desc;

int aeonb_orient_batch(aeonb_ctx* ctx, const aeonb_orient_desc* descs, int n);

/* Resize pass for INTER_AREA, INTER_CUBIC and INTER_LANCZOS4: cv::resize(window, out, Size(out_w, out_h), 0, 0, interp) (image::resize
 * with interpolation_method "AREA" / "CUBIC" / "LANCZOS4", src/image.cpp:93-106), where the window is the crop box of a canvas on which the
 * source sits (zeros elsewhere), exactly as in aeonb_image_desc.  The output is an interleaved picture that
 * aeonb_image_batch then takes as a source of the same size (no further resampling). */
typedef struct aeonb_resize_desc
{
    const uint8_t* src;      /* device: interleaved B,G,R[,x]; NULL = all-zero canvas */
    int32_t src_pitch, src_pixel_stride;
    int32_t src_w, src_h;
    int32_t canvas_x, canvas_y;
    int32_t crop_x, crop_y, crop_w, crop_h;
    int32_t interp;          /* AEONB_INTERP_AREA, AEONB_INTERP_CUBIC or AEONB_INTERP_LANCZOS4 */
    int32_t out_w, out_h;
    uint8_t* dst;            /* device */
    int32_t dst_pitch, dst_pixel_stride;
    int32_t channels;        /* channels of the picture the reference resizes: 3, or 1 for a grey picture carried as
                                B = G = R (INTER_CUBIC's vertical pass depends on the length of the interleaved row) */
    int32_t reserved0;
} aeonb_resize_desc;

int aeonb_resize_batch(aeonb_ctx* ctx, const aeonb_resize_desc* descs, int n);

/* ------------------------------------------------------------------------------------------------
 * 1b. JPEG back end kernel: dequantisation + 8x8 integer inverse DCT + chroma upsampling +
 *     YCbCr->BGR, i.e. everything cv::imdecode (src/etl_image.cpp:90, src/cap_mjpeg_decoder.cpp:140)
 *     does after entropy decoding.
 * ---------------------------------------------------------------------------------------------- */

typedef struct aeonb_jpeg_desc
{
    const int16_t*  coef[3];  /* device: per component, blocks in raster order, 64 int16 each, stored
                                 COLUMN-major inside the block (element (row r, col c) at c*8+r) */
    const uint16_t* quant[3]; /* device: 64 quantiser steps per component, same column-major order */
    int32_t width, height;    /* image size in pixels */
    int32_t ncomp;            /* 1 (grey) or 3 (YCbCr) */
    int32_t hs[3], vs[3];     /* sampling factors; supported: grey, 4:4:4, 4:2:2 (2x1), 4:2:0 (2x2), 4:4:0 (1x2), 4:1:1 (4x1) */
    int32_t blocks_w[3], blocks_h[3]; /* coefficient plane size in blocks (padded to whole MCUs) */
    uint8_t* dst;             /* device: interleaved B,G,R[,x] output */
    int32_t dst_pitch;
    int32_t dst_pixel_stride; /* 3 or 4 */
} aeonb_jpeg_desc;

int aeonb_jpeg_backend_batch(aeonb_ctx* ctx, const aeonb_jpeg_desc* descs, int n);
int64_t aeonb_jpeg_backend_bytes(const aeonb_jpeg_desc* descs, int n);

/* ------------------------------------------------------------------------------------------------
 * 1b'. JPEG entropy decoding on the device: the Huffman stage of cv::imdecode
 *      (src/etl_image.cpp:90).  A stream without restart markers that is given a work area is decoded by a whole
 *      thread block (segments decoded speculatively, then synchronised on each other); other streams by one
 *      warp that walks the stream serially.  Fills the coefficient planes that
 *      aeonb_jpeg_desc describes, so aeonb_jpeg_entropy_batch followed by aeonb_jpeg_backend_batch
 *      decodes a batch of JPEG files without per-record host work beyond header parsing.
 * ---------------------------------------------------------------------------------------------- */

typedef struct aeonb_entropy_desc
{
    const uint8_t* scan;     /* device: entropy-coded bytes of the scan (after the SOS header).  Read in aligned 16-byte
                                vectors: the 16-byte groups holding its first and last byte must be readable memory,
                                which holds for any placement inside a cudaMalloc'd buffer */
    uint32_t scan_size;
    int32_t  ncomp;
    const uint8_t* tables;   /* device: 4 Huffman tables of 272 bytes each in DHT form (16 code counts, then the
                                values, zero padded): DC slot 0, DC slot 1, AC slot 0, AC slot 1 */
    int32_t hs[3], vs[3];    /* sampling factors */
    int32_t dc_table[3], ac_table[3]; /* slot (0 or 1) used by each component */
    int32_t mcux, mcuy;      /* picture size in MCUs */
    int32_t roi[4];          /* MCU rectangle {mx0, my0, mx1, my1} to store; {0, 0, mcux, mcuy} for the whole picture */
    int32_t restart_interval;/* MCUs between restart markers, 0 = none */
    int32_t reserved0;
    int16_t* coef[3];        /* device: compact planes of (mx1-mx0)*hs x (my1-my0)*vs blocks, layout as in aeonb_jpeg_desc,
                                16-byte aligned */
    int32_t* status;         /* device: set to 0 on success, 1 when the stream is malformed (may be NULL) */
    void*    scratch;        /* device: work area of aeonb_jpeg_entropy_scratch_bytes() bytes, 16-byte aligned.  With it, a
                                stream without restart markers is decoded by a whole thread block (speculative decoding
                                of segments that synchronise on each other); without it (NULL), or with restart markers,
                                by a single warp walking the stream serially */
    uint64_t scratch_bytes;
} aeonb_entropy_desc;

int aeonb_jpeg_entropy_batch(aeonb_ctx* ctx, const aeonb_entropy_desc* descs, int n);
int64_t aeonb_jpeg_entropy_scratch_bytes(const aeonb_entropy_desc* desc);

/* ------------------------------------------------------------------------------------------------
 * 1c. Spectrogram kernel: framing + window + DFT magnitude + mel filter bank + log [+ DCT]
 *     (specgram::wav_to_specgram / specgram_to_cepsgram / cepsgram_to_mfcc, src/specgram.cpp:26-154).
 * ---------------------------------------------------------------------------------------------- */

typedef struct aeonb_specgram_desc
{
    const int16_t* samples; /* device */
    int32_t n_samples;
    float*  dst;            /* device: max_time_steps x n_out floats, rows past the clip are zero-filled */
} aeonb_specgram_desc;

typedef struct aeonb_specgram_config
{
    int32_t frame_length;   /* samples per frame == DFT length */
    int32_t frame_stride;
    int32_t max_time_steps;
    int32_t num_filters;    /* mel filters; 0 = output the magnitude spectrogram (frame_length/2+1 bins) */
    int32_t sample_rate;
    int32_t window;         /* 0 none, 1 hann, 2 hamming, 3 blackman, 4 bartlett (src/specgram.cpp:156-189) */
    int32_t num_cepstra;    /* > 0 (needs num_filters > 0): MFCC, the first num_cepstra coefficients of the orthonormal
                               DCT-II of the log-mel row, zero-padded to an even length (specgram::cepsgram_to_mfcc,
                               src/specgram.cpp:139-154); rows are then num_cepstra floats */
    int32_t reserved0;
} aeonb_specgram_config;

int aeonb_specgram_batch(aeonb_ctx* ctx, const aeonb_specgram_desc* descs, int n, const aeonb_specgram_config* cfg);
int64_t aeonb_specgram_bytes(const aeonb_specgram_desc* descs, int n, const aeonb_specgram_config* cfg);

/* ------------------------------------------------------------------------------------------------
 * 2. Host helpers
 * ---------------------------------------------------------------------------------------------- */

/* Header-only parse of a baseline JPEG. */
typedef struct aeonb_jpeg_info
{
    int32_t width, height, ncomp;
    int32_t hs[3], vs[3];
    int32_t blocks_w[3], blocks_h[3];
    int64_t coef_count[3]; /* int16 elements per component plane */
    int32_t orientation;   /* EXIF orientation tag (1..8), 1 when absent.  width/height above are the stored size;
                              cv::imdecode hands aeon the picture turned as the tag says (sizes swapped for 5..8):
                              aeonb_orient_batch below does that turn */
    int32_t reserved0;
} aeonb_jpeg_info;

int aeonb_jpeg_parse(const void* data, size_t size, aeonb_jpeg_info* info);

/* Entropy-decodes a baseline JPEG into per-component coefficient planes (layout as in
 * aeonb_jpeg_desc) and quantiser tables, all host memory supplied by the caller. */
int aeonb_jpeg_entropy_decode(const void* data, size_t size, int16_t* coef[3], uint16_t* quant[3]);

/* Region decoding.  Only the part of a picture that the crop box can touch has to be decoded.
 * aeonb_jpeg_roi_for_crop turns a crop box (in picture pixels) into the rectangle of MCUs
 * roi = {mx0, my0, mx1, my1} (half open) that covers it plus the one chroma sample of context the
 * upsampling filter needs; aeonb_jpeg_entropy_decode_roi stores only the blocks of that rectangle, as compact
 * planes of (mx1-mx0)*hs[c] x (my1-my0)*vs[c] blocks, and stops parsing after its last MCU row.  The back-end
 * kernel is then given the region as if it were the picture: width/height = the region's extent in pixels
 * (clipped to the picture), blocks_w/h = the compact plane sizes. */
int aeonb_jpeg_roi_for_crop(const aeonb_jpeg_info* info, int crop_x, int crop_y, int crop_w, int crop_h, int32_t roi[4]);
int aeonb_jpeg_entropy_decode_roi(const void* data, size_t size, const int32_t roi[4], int16_t* coef[3], uint16_t* quant[3]);

/* Host side of aeonb_jpeg_entropy_batch: parses the headers of one JPEG file and fills `info`, the quantiser tables (3 x 64,
 * column-major), the four Huffman tables in the 4 x 272-byte form aeonb_entropy_desc.tables wants, and every field
 * of `desc` that does not depend on where the data will live (scan, tables, coef, status and roi are left for the
 * caller; scan_offset tells where the scan starts inside `data`).  AEONB_ERR_UNSUPPORTED when the file uses more
 * than two DC or two AC tables (decode such a file with aeonb_jpeg_entropy_decode). */
int aeonb_jpeg_entropy_prepare(const void* data, size_t size, aeonb_jpeg_info* info, uint16_t quant[192], uint8_t tables[1088],
                               aeonb_entropy_desc* desc, size_t* scan_offset);

/* PNG records (cv::imdecode reads them too, src/etl_image.cpp:90; aeon's own geometry tests feed PNG): decoded on the
 * host into the B,G,R picture IMREAD_COLOR delivers (palette expanded, grey replicated, 16-bit samples cut to the high
 * byte, alpha dropped; plain and Adam7-interlaced files).  dst: height rows of `pitch` >= 3*width bytes.
 * aeonb_png_decode_grey gives the one-channel picture of IMREAD_GRAYSCALE, which is also what the pixelmask extractor's
 * IMREAD_ANYDEPTH read (src/etl_pixel_mask.cpp:39) returns for 8-bit files: colour files go through libpng's integer
 * colour -> grey conversion; dst: height rows of `pitch` >= width bytes. */
int aeonb_png_info(const void* data, size_t size, int32_t* width, int32_t* height);
int aeonb_png_decode_bgr(const void* data, size_t size, uint8_t* dst, size_t pitch);
int aeonb_png_decode_grey(const void* data, size_t size, uint8_t* dst, size_t pitch);

/* localization_rcnn (src/etl_localization_rcnn.cpp): region-proposal training targets.
 *
 * aeonb_rcnn_anchors: anchor::generate (:434-472) -- every base anchor (ratios outermost, scales inner, :489-557) shifted
 * over the floor(width * scaling_factor) x floor(height * scaling_factor) grid, anchor-major then y then x; `out` takes
 * aeonb_rcnn_anchor_count() x 4 floats (xmin, ymin, xmax, ymax).  Host only.
 *
 * aeonb_rcnn_label_batch: the O(anchors x boxes) part of transformer::transform (:118-193) for a batch, one launch: for
 * the anchors that lie inside the record's scaled picture, intersection over union with every ground-truth box
 * (bbox_overlaps, :302-338, the same float32 operations), then the labels -- 0 below negative_overlap, 1 for every
 * anchor that equals a box's best overlap (ties included) or reaches positive_overlap, -1 otherwise and for anchors
 * outside the picture -- and the index of each anchor's best box (the first on ties, 0 when none overlaps).  A record
 * without boxes gets -1 everywhere, as in the reference (:181-208).  Sampling (transformer::sample_anchors, :218-263) and
 * the regression targets of the at most rois_per_image sampled anchors stay on the host. */
typedef struct aeonb_rcnn_config
{
    int32_t width, height;     /* output picture size the anchors cover */
    int32_t base_size;         /* 16 */
    int32_t n_ratios, n_scales;
    float   scaling_factor;    /* 1/16: the feature stride is its reciprocal */
    float   ratios[8], scales[8];
} aeonb_rcnn_config;

typedef struct aeonb_rcnn_desc
{
    const float* gt_boxes;     /* device: n_gt x 4 floats, boxes already transformed to the output picture */
    int32_t n_gt;              /* 0..1024 */
    int32_t im_width, im_height; /* the scaled picture: anchors must lie inside [0, im_width) x [0, im_height) */
    int8_t*  labels;           /* device: one per anchor: -1, 0, 1 */
    int16_t* best_box;         /* device: one per anchor */
} aeonb_rcnn_desc;

int64_t aeonb_rcnn_anchor_count(const aeonb_rcnn_config* cfg);
int     aeonb_rcnn_anchors(const aeonb_rcnn_config* cfg, float* out);
int     aeonb_rcnn_label_batch(aeonb_ctx* ctx, const float* anchors_dev, int32_t n_anchors, const aeonb_rcnn_desc* descs, int n,
                               float negative_overlap, float positive_overlap);

/* Draws augmentation parameters exactly as aeon's param_factory::make_params does
 * (src/augment_image.cpp:107-230) for `n` records whose decoded sizes are in_w/in_h,
 * using per-slot std::minstd_rand0 engines seeded as aeon's batch_decoder seeds them
 * (src/batch_decoder.cpp:47-54).  Writes 24 doubles per record:
 * crop x,y,w,h, out w,h, flip, angle, hue, contrast, brightness, saturation,
 * lighting0..2, color_noise_std, padding off x,y, expand ratio, expand off x,y, expand w,h, reserved. */
int aeonb_draw_params(const char* augmentation_json, uint32_t seed, int decode_size, int n, const int32_t* in_w,
                      const int32_t* in_h, int out_w, int out_h, double* out);

/* Same for the SSD path (param_factory::make_ssd_params, src/augment_image.cpp:232-310): record i has
 * box_counts[i] ground-truth boxes, given as consecutive (xmin, ymin, xmax, ymax) float quadruples in
 * `boxes`.  The output layout is that of aeonb_draw_params. */
int aeonb_draw_ssd_params(const char* augmentation_json, uint32_t seed, int decode_size, int n, const int32_t* in_w,
                          const int32_t* in_h, int out_w, int out_h, const int32_t* box_counts, const float* boxes,
                          double* out);

/* Host box arithmetic of the localisation providers.
 *
 * aeonb_box_overlap: intersect / jaccard_overlap / coverage of two boxes a, b = (xmin, ymin, xmax, ymax), either pixel
 * boxes with an inclusive max corner (boundingbox::box, src/boundingbox.cpp:105-148) or, with `normalized` != 0, boxes
 * in [0,1] with an exclusive max corner (normalized_box::box, src/normalized_box.cpp:47-88; AEONB_ERR_INVALID when a
 * box is not within [0,1]).  out = intersection (4 floats; the default box (0,0,-1,-1) resp. (0,0,0,0) when empty),
 * a.jaccard_overlap(b), a.coverage(b).
 *
 * aeonb_transform_boxes: boundingbox::transformer::transform_box (src/etl_boundingbox.cpp:146-261) for n pixel boxes:
 * expand shift, emit constraint, clip to the crop box, flip, rescale to the output size.  `out` takes up to n boxes,
 * `kept` (may be NULL) the input index of each surviving box, *n_out their number.
 *
 * aeonb_ssd_load_boxes: localization::ssd::loader::load (src/etl_localization_ssd.cpp:116-149): image_shape int32[2],
 * gt_boxes float[max_gt_boxes * 4] (normalised, zero rows after the boxes), gt_box_count int32, gt_class and
 * gt_difficult int32[max_gt_boxes]. */
typedef struct aeonb_box_params
{
    int32_t crop_x, crop_y, crop_w, crop_h;
    int32_t out_w, out_h;
    int32_t flip;
    float   expand_ratio;      /* boxes are shifted by the expand offset when > 1 */
    int32_t expand_off_x, expand_off_y, expand_w, expand_h;
    int32_t emit_type;         /* 0 none, 1 center, 2 min_overlap */
    float   emit_min_overlap;
} aeonb_box_params;

int aeonb_box_overlap(int normalized, const float a[4], const float b[4], float out[6]);
int aeonb_transform_boxes(const aeonb_box_params* p, const float* boxes, int n, float* out, int32_t* kept, int32_t* n_out);
int aeonb_ssd_load_boxes(const float* boxes, const int32_t* labels, const int32_t* difficult, int n, int width, int height,
                         int max_gt_boxes, int32_t* image_shape, float* gt_boxes, int32_t* gt_box_count, int32_t* gt_class,
                         int32_t* gt_difficult);

/* Fills the photometric fields of `desc` (colour matrix, hue, HSV vector columns, contrast,
 * lighting scale/offsets) from aeon's parameter values, doing on the host what
 * photometric::cbsjitter / lighting do before they touch pixels (src/image.cpp:336-346,362-371).
 * `lighting` is NULL or 3 floats; desc->out_w must already be set. */
int aeonb_image_desc_set_photometric(aeonb_image_desc* desc, float contrast, float brightness, float saturation, int hue,
                                     const float* lighting, float color_noise_std);

/* ------------------------------------------------------------------------------------------------
 * 3. Provider: encoded records -> augmented batch
 *    (provider_interface::provide, src/provider_interface.hpp:42-44, driven per decode chunk the
 *    way batch_decoder::filler / process do, src/batch_decoder.cpp:62-99)
 * ---------------------------------------------------------------------------------------------- */

/* `config_json` carries aeon's own keys: "etl", "augmentation", "batch_size", "random_seed",
 * "batch_major", plus optional "decode_size" (RNG slots, default batch_size) and
 * "decode_threads" (host entropy-decode workers, default: hardware threads). */
int  aeonb_provider_create(aeonb_ctx* ctx, const char* config_json, aeonb_provider** out);
void aeonb_provider_destroy(aeonb_provider* p);

int         aeonb_provider_input_count(const aeonb_provider* p);  /* elements per record */
int         aeonb_provider_output_count(const aeonb_provider* p); /* named output buffers */
const char* aeonb_provider_output_name(const aeonb_provider* p, int i);
/* Shape of one record of output i: up to 8 dims; returns the rank.  *dtype receives an aeonb_dtype. */
int     aeonb_provider_output_shape(const aeonb_provider* p, int i, int64_t* dims, int32_t* dtype);
int64_t aeonb_provider_output_bytes(const aeonb_provider* p, int i); /* bytes per record */

/* Processes n records (n <= batch_size).  elems[r*input_count + e] / sizes[...] address element e of
 * record r in host memory.  outputs[i] receives n records of output i; it is device memory when
 * outputs_on_device != 0, else host memory (copied back before the call returns).
 * The call returns after the batch is complete. */
int aeonb_provider_run(aeonb_provider* p, const void* const* elems, const size_t* sizes, int n, void* const* outputs,
                       int outputs_on_device);

/* Pipelined form: plans the batch on the calling thread (headers, seeded draws), hands it to the provider's driver
 * thread (staging, uploads, launches, output copies) and stores a ticket; aeonb_provider_wait(p, ticket) blocks until
 * that batch is complete and reports its errors.  Calling run_async for batch k+1 before waiting for batch k overlaps
 * the planning of k+1 with the staging of k and the kernels and copies of k-1 (aeon overlaps its stages with
 * double-buffered async_manager threads, src/async_manager.hpp:91-117).  Records and output buffers of a batch must
 * stay valid and untouched until its ticket has been waited for; each batch in flight needs its own output buffers;
 * at most 7 batches may be in flight, and a call blocks while the driver thread is two batches behind. */
int aeonb_provider_run_async(aeonb_provider* p, const void* const* elems, const size_t* sizes, int n, void* const* outputs,
                             int outputs_on_device, int64_t* ticket);
int aeonb_provider_wait(aeonb_provider* p, int64_t ticket);

/* Statistics of the last aeonb_provider_run: host->device and device->host bytes, kernel launches. */
int aeonb_provider_stats(const aeonb_provider* p, int64_t* h2d_bytes, int64_t* d2h_bytes, int32_t* launches);

/* ------------------------------------------------------------------------------------------------
 * 4. Loader (loader_factory::get_loader + loader::iterator, src/loader.hpp:112-175;
 *    python aeon.DataLoader, src/api.cpp:104-425)
 * ---------------------------------------------------------------------------------------------- */

int  aeonb_loader_create(const char* config_json, int device, aeonb_loader** out);
void aeonb_loader_destroy(aeonb_loader* l);
int  aeonb_loader_record_count(const aeonb_loader* l);
int  aeonb_loader_batch_size(const aeonb_loader* l);
int  aeonb_loader_batch_count(const aeonb_loader* l);
int  aeonb_loader_output_count(const aeonb_loader* l);
const char* aeonb_loader_output_name(const aeonb_loader* l, int i);
int  aeonb_loader_output_shape(const aeonb_loader* l, int i, int64_t* dims, int32_t* dtype);
const char* aeonb_loader_axis_names(const aeonb_loader* l, int i); /* comma separated */
const char* aeonb_loader_config(const aeonb_loader* l);            /* JSON of the effective configuration */
/* Advances to the next batch.  buffers[i] receives a pointer (host, or device when the loader
 * was configured with "device_output": true) valid until the next call.  Returns AEONB_END when
 * the iteration is complete. */
int aeonb_loader_next(aeonb_loader* l, void** buffers);
int aeonb_loader_reset(aeonb_loader* l);
int aeonb_loader_position(const aeonb_loader* l);

/* ------------------------------------------------------------------------------------------------
 * 5. Source side alone, host only (no GPU needed): the stream of encoded records the loader decodes --
 *    manifest_file -> block_loader_file -> block_manager with the CPIO block cache
 *    (src/manifest_file.cpp:115-330, src/block_loader_file.cpp:45-117, src/block_manager.cpp:61-106,
 *    src/cache_system.cpp:69-146, src/cpio.cpp).  Takes the loader's own JSON (manifest_filename, manifest_root,
 *    batch_size, block_size, subset_fraction, shuffle_enable, shuffle_manifest, random_seed, node_id, node_count,
 *    cache_directory); other keys are ignored here.  The stream never ends: after the last block it starts over,
 *    reshuffled as the configuration says.
 * ---------------------------------------------------------------------------------------------- */
typedef struct aeonb_stream aeonb_stream;
int  aeonb_stream_create(const char* config_json, aeonb_stream** out);
void aeonb_stream_destroy(aeonb_stream* s);
/* cache_state: 0 no cache_directory, 1 another process is writing the cache (this one reads the manifest's files),
 * 2 this process writes the cache during its first pass, 3 the cache is complete and is what gets read. */
int  aeonb_stream_info(const aeonb_stream* s, int64_t* record_count, int32_t* elements_per_record, int32_t* block_count,
                       int32_t* cache_state, char* cache_dir, size_t cache_dir_size);
/* The next record: elems[e] / sizes[e] for each of its elements, valid until the next call. */
int  aeonb_stream_next(aeonb_stream* s, const void** elems, size_t* sizes);
int  aeonb_stream_reset(aeonb_stream* s);

/* Which records of a manifest of `total` records node `node_id` of `node_count` reads (src/manifest_file.cpp:278-295):
 * batch-sized slices dealt round-robin, then an evenly divided tail.  Writes the indices to `out` (may be NULL) and
 * returns their number (total / node_count; total when node_count <= 1), negative on a bad argument.  It is also how
 * the records of a batch are sharded over the GPUs of one box. */
int64_t aeonb_node_record_indices(int64_t total, int node_id, int node_count, int batch_size, int64_t* out);

#ifdef __cplusplus
}
#endif
#endif /* AEON_B200_H */
