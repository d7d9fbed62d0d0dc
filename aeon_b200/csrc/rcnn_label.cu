// Anchor labelling for localization_rcnn on sm_100a.
//
// aeon's localization::rcnn::transformer::transform (src/etl_localization_rcnn.cpp:97-216) forms the full
// anchors x boxes overlap matrix per record on one CPU thread (34 596 anchors x up to 64 boxes for the default 1000 x 1000
// configuration), reduces it along both axes and derives a label per anchor.  Here one CTA per record does the same
// without storing the matrix: the boxes sit in shared memory, every thread walks a strided subset of the anchors,
//   pass 1: overlaps of its anchors with every box -> per-box maximum (shared-memory atomic max on the bit pattern of
//           the non-negative float, tried only when the value beats the maximum seen so far),
//   pass 2: the same overlaps again (identical instructions, so identical values) -> row maximum, first best box, and
//           the three labelling rules in the reference's order.
// The overlap arithmetic is bbox_overlaps' (:302-338) in IEEE float32 (explicit round-to-nearest operations, true
// division), so the comparisons with the thresholds and the equality test with the per-box maximum agree with the
// reference bit for bit.  The anchors are the same for every record and stay in L2 after the first CTA has read them.
#include <cuda_runtime.h>
#include <stdint.h>

#include <sstream>
#include <vector>

#include "context.hpp"

namespace aeonb
{
    namespace
    {
        constexpr int RCNN_THREADS = 1024;
        constexpr int RCNN_MAX_GT  = 1024;

        struct rcnn_launch
        {
            const float4*          anchors;
            int                    n_anchors;
            const aeonb_rcnn_desc* descs;
            float                  negative_overlap, positive_overlap;
        };

        // box::width / height (src/box.hpp:51-52): max - min + 1
        __device__ __forceinline__ float extent(float lo, float hi) { return __fadd_rn(__fsub_rn(hi, lo), 1.0f); }

        // One element of bbox_overlaps: 0 unless the boxes share at least one pixel.
        __device__ __forceinline__ float overlap(const float4 a, float a_area, const float4 g, float g_area)
        {
            const float iw = __fadd_rn(__fsub_rn(fminf(a.z, g.z), fmaxf(a.x, g.x)), 1.0f);
            if (!(iw > 0.0f))
                return 0.0f;
            const float ih = __fadd_rn(__fsub_rn(fminf(a.w, g.w), fmaxf(a.y, g.y)), 1.0f);
            if (!(ih > 0.0f))
                return 0.0f;
            const float inter = __fmul_rn(iw, ih);
            const float ua    = __fsub_rn(__fadd_rn(a_area, g_area), inter);
            return __fdiv_rn(inter, ua);
        }

        // COMPACT: the indices of the anchors inside the picture (typically a third of the table) are first gathered into
        // shared memory (16-bit, so for tables of up to 65 535 anchors), and both passes walk that list: every lane of a
        // warp then has an anchor to work on.  Larger tables take the plain strided walk.
        template <bool COMPACT>
        __global__ void __launch_bounds__(RCNN_THREADS) rcnn_label_kernel(const rcnn_launch L)
        {
            extern __shared__ uint16_t inside_list[];
            __shared__ float4       gt[RCNN_MAX_GT];
            __shared__ float        gt_area[RCNN_MAX_GT];
            __shared__ unsigned int col_max[RCNN_MAX_GT]; // bit patterns of non-negative floats order like the floats
            __shared__ int          n_inside;

            const aeonb_rcnn_desc d   = L.descs[blockIdx.x];
            const int             tid = threadIdx.x;
            const int             K   = d.n_gt;
            for (int k = tid; k < K; k += RCNN_THREADS)
            {
                const float4 g = reinterpret_cast<const float4*>(d.gt_boxes)[k];
                gt[k]          = g;
                gt_area[k]     = __fmul_rn(extent(g.x, g.z), extent(g.y, g.w));
                col_max[k]     = 0u;
            }
            if (tid == 0)
                n_inside = 0;
            __syncthreads();
            const float right = (float)d.im_width, bottom = (float)d.im_height;
            auto is_inside = [&](const float4 a) { return a.x >= 0.0f && a.y >= 0.0f && a.z < right && a.w < bottom; }; // :474-487

            if (COMPACT)
            {
                // every anchor gets its "outside / no boxes" answer; the inside ones are queued (order does not matter:
                // each anchor's result depends on that anchor alone, and the per-box maximum is order-free)
                const int rounds = (L.n_anchors + RCNN_THREADS - 1) / RCNN_THREADS;
                for (int r = 0; r < rounds; ++r)
                {
                    const int  i  = r * RCNN_THREADS + tid;
                    const bool in = i < L.n_anchors && K > 0 && is_inside(L.anchors[i]);
                    if (i < L.n_anchors)
                    {
                        d.labels[i]   = -1;
                        d.best_box[i] = 0;
                    }
                    const unsigned mask = __ballot_sync(0xFFFFFFFFu, in);
                    int            base = 0;
                    if ((tid & 31) == 0 && mask)
                        base = atomicAdd(&n_inside, __popc(mask));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    if (in)
                        inside_list[base + __popc(mask & ((1u << (tid & 31)) - 1))] = (uint16_t)i;
                }
                __syncthreads();
            }
            const int count = COMPACT ? n_inside : L.n_anchors;

            if (K > 0)
                for (int j = tid; j < count; j += RCNN_THREADS)
                {
                    const float4 a = L.anchors[COMPACT ? (int)inside_list[j] : j];
                    if (!COMPACT && !is_inside(a))
                        continue;
                    const float a_area = __fmul_rn(extent(a.x, a.z), extent(a.y, a.w));
                    for (int k = 0; k < K; ++k)
                    {
                        const unsigned int v = __float_as_uint(overlap(a, a_area, gt[k], gt_area[k]));
                        if (v > col_max[k])
                            atomicMax(&col_max[k], v);
                    }
                }
            __syncthreads();

            for (int j = tid; j < count; j += RCNN_THREADS)
            {
                const int    i      = COMPACT ? (int)inside_list[j] : j;
                const float4 a      = L.anchors[i];
                const bool   inside = COMPACT || is_inside(a);
                int          label = -1, best = 0;
                if (inside && K > 0)
                {
                    const float a_area  = __fmul_rn(extent(a.x, a.z), extent(a.y, a.w));
                    float       row_max = 0.0f;
                    bool        is_best = false;
                    for (int k = 0; k < K; ++k)
                    {
                        const float v = overlap(a, a_area, gt[k], gt_area[k]);
                        if (v > row_max)
                        {
                            row_max = v;
                            best    = k;
                        }
                        is_best |= __float_as_uint(v) == col_max[k];
                    }
                    if (row_max < L.negative_overlap)
                        label = 0;
                    if (is_best)
                        label = 1;
                    if (row_max >= L.positive_overlap)
                        label = 1;
                }
                d.labels[i]   = (int8_t)label;
                d.best_box[i] = (int16_t)best;
            }
        }
    }
}

using namespace aeonb;

extern "C" int aeonb_rcnn_label_batch(aeonb_ctx* ctx, const float* anchors_dev, int32_t n_anchors, const aeonb_rcnn_desc* descs, int n,
                                      float negative_overlap, float positive_overlap)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && (!descs || !anchors_dev)))
            throw std::invalid_argument("aeonb_rcnn_label_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        if (n_anchors <= 0 || ((uintptr_t)anchors_dev & 15))
            throw std::invalid_argument("aeonb_rcnn_label_batch: the anchors must be a non-empty, 16-byte aligned device array");
        for (int i = 0; i < n; ++i)
        {
            const aeonb_rcnn_desc& r = descs[i];
            std::ostringstream     ss;
            if (r.n_gt < 0 || r.n_gt > RCNN_MAX_GT)
                ss << "record " << i << ": between 0 and " << RCNN_MAX_GT << " ground-truth boxes per record";
            else if (r.n_gt > 0 && (!r.gt_boxes || ((uintptr_t)r.gt_boxes & 15)))
                ss << "record " << i << ": the boxes must be a 16-byte aligned device array";
            else if (!r.labels || !r.best_box || ((uintptr_t)r.best_box & 1))
                ss << "record " << i << ": NULL or misaligned output";
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
        }
        AEONB_CUDA(cudaSetDevice(ctx->device));
        rcnn_launch L;
        L.anchors          = reinterpret_cast<const float4*>(anchors_dev);
        L.n_anchors        = n_anchors;
        L.descs            = static_cast<const aeonb_rcnn_desc*>(ctx->upload(descs, sizeof(aeonb_rcnn_desc) * n));
        L.negative_overlap = negative_overlap;
        L.positive_overlap = positive_overlap;
        cudaError_t e = cudaSuccess;
        if (n_anchors <= 65535)
        {
            const size_t smem = ((size_t)n_anchors * sizeof(uint16_t) + 15) & ~(size_t)15;
            e = cudaFuncSetAttribute(rcnn_label_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                rcnn_label_kernel<true><<<n, RCNN_THREADS, smem, ctx->stream>>>(L);
        }
        else
            rcnn_label_kernel<false><<<n, RCNN_THREADS, 0, ctx->stream>>>(L);
        if (e == cudaSuccess)
            e = cudaGetLastError();
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("rcnn label kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}
