// Image augmentation + packing kernel for sm_100a.
//
// One launch transforms a whole batch.  A record is handled by a thread-block cluster of
// `bands` CTAs; CTA b owns a band of output rows, one thread per output column.  Each CTA
//   1. builds its tables in one phase: warp 0 the vertical taps of the crop->output resize (the
//      11-bit fixed-point form cv::resize(INTER_LINEAR) uses for 8-bit images) and the list of
//      source rows the band touches, every thread the horizontal taps of its column (registers),
//   2. stages the listed source rows -- only the columns the band reads -- into shared memory
//      with 16-byte cp.async copies, double-buffered in groups of rows so that the copies of the
//      next group run under the arithmetic of the current one (one barrier per group),
//   3. runs the horizontal pass ONCE per staged source row (two dot products per channel out
//      of three aligned shared-memory words, fetched one row ahead), keeps the last two
//      horizontal results in registers and emits every output row whose taps are complete:
//      vertical pass, colour matrix, HSV hue shift; the band is kept as planar uint8 in shared
//      memory, already flipped and in output channel order,
//   4. if contrast is active, reduces per-channel sums (warp shuffles, then shared memory)
//      and adds them into every CTA of the cluster through distributed shared memory, so the
//      per-image mean never touches global memory,
//   5. applies contrast and lighting, converts to the output type, standardises and
//      streams the band out with 128-bit stores, two in flight per thread.
//
// Pixels outside the source picture (expand canvas, padding) are never read: their taps get
// weight zero, which gives the same sums as a zero pixel.
//
// The arithmetic of every stage is the integer / float32 arithmetic OpenCV applies for the
// calls aeon makes (src/etl_image.cpp:146-202, src/image.cpp:336-406, src/etl_image.cpp:246-341);
// this file is compiled with -fmad=false and uses explicit fused operations only where
// OpenCV's own code is fused.
#include <algorithm>
#include <atomic>

#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aeon_b200.h"
#include "device_common.cuh"

namespace cg = cooperative_groups;

namespace aeonb
{
    namespace
    {
        constexpr int AUG_MAX_THREADS = 224;
        constexpr int AUG_MAX_BAND    = 8;  // portable cluster size limit
        constexpr int AUG_MAX_GROUP   = 16; // source rows staged per group, at most
        constexpr int AUG_STAGE_PAD   = 16; // bytes kept free before and after a staged row

        struct aug_launch
        {
            const aeonb_image_desc* descs; // device copy
            aeonb_image_layout      layout;
            int                     rows_per_band;
            int                     tile_pitch;  // bytes per tile row (multiple of 16)
            int                     vector_ok;   // slots are 16-byte aligned with unit x stride
            int                     n;           // records in the batch
            int                     stage_bytes; // shared memory for staged source rows (two buffers of half that)
        };

        __device__ __forceinline__ short sat_s16(int v) { return (short)min(max(v, -32768), 32767); }

        // Source index and tap weights for destination index d (cv::resize, INTER_LINEAR, 8-bit);
        // scale = 1 / (dst_len / src_len) in double, as cv::resize forms it.
        __device__ __forceinline__ void linear_tap(int d, int src_len, double scale, bool clamp_weights, int& s, short& w0, short& w1)
        {
            float f  = (float)(((double)d + 0.5) * scale - 0.5);
            float fl = floorf(f);
            s        = (int)fl;
            f        = f - fl;
            if (clamp_weights)
            {
                if (s < 0)
                {
                    f = 0.f;
                    s = 0;
                }
                if (s >= src_len - 1)
                {
                    f = 0.f;
                    s = src_len - 1;
                }
            }
            w0 = sat_s16(__float2int_rn((1.f - f) * 2048.f));
            w1 = sat_s16(__float2int_rn(f * 2048.f));
        }

        __device__ __forceinline__ int nearest_tap(int d, int src_len, double scale)
        {
            return min((int)floor((double)d * scale), src_len - 1);
        }

        struct bgr
        {
            int b, g, r;
        };

        // min(max(v, 0), 255) in one instruction (three-input integer min/max of sm_90 and later)
        __device__ __forceinline__ int clamp_u8(int v) { return __vimin_s32_relu(v, 255); }

        // The 12-bit reciprocals of 8-bit BGR->HSV: .x = round((255 << 12) / i), .y = round((180 << 12) / (6 i)).
        // No quotient falls on a half for i in 1..255, so the integer form equals OpenCV's rounded double division.
        struct hsv_div_table
        {
            int2 v[256];
        };
        constexpr hsv_div_table make_hsv_div()
        {
            hsv_div_table t{};
            for (int i = 1; i < 256; ++i)
            {
                t.v[i].x = (2 * (255 << 12) + i) / (2 * i);
                t.v[i].y = (2 * ((180 << 12) / 6) + i) / (2 * i);
            }
            return t;
        }
        __device__ const hsv_div_table k_hsv_div = make_hsv_div();

        // Per-CTA tables of the hue stage (all exact restatements of the per-pixel arithmetic, tabulated once):
        //   div      : the reciprocals above;
        //   sector_f : for a hue h in [0,180), after the shift uint8((h + hue) % 180) (C remainder, stored through a
        //              uint8_t): .x = byte selector that puts (p, q, v) of HSV->BGR into B,G,R order for the hue's
        //              sector, .y = the factor f of the sector's middle term: the fractional position in odd sectors,
        //              one minus it in even ones;
        //   unit     : x * (1/255) for x in [0,255] (the float S and V).
        struct hue_tables
        {
            int2   div[256];
            float2 sector_f[180];
            float  unit[256];
        };

        __device__ __forceinline__ void build_hue_tables(hue_tables& t, int hue, int tid, int nthreads)
        {
            for (int i = tid; i < 256; i += nthreads)
            {
                t.div[i]  = k_hsv_div.v[i];
                t.unit[i] = (float)i * (1.0f / 255.0f);
            }
            for (int h = tid; h < 180; h += nthreads)
            {
                const int   hs = ((h + hue) % 180) & 0xFF;
                const float hf = (float)hs * (6.0f / 180.0f);
                const float fl = floorf(hf);
                int         sector = (int)fl;
                if (sector >= 6)
                    sector -= 6; // hs <= 255 gives sector <= 8
                const float f = hf - fl;
                // (B, G, R) = sector 0 (p, t, v)  1 (p, v, q)  2 (t, v, p)  3 (v, q, p)  4 (v, p, t)  5 (q, p, v), with
                // p = v(1-s), q = v(1-sf), t = v(1-s(1-f)); the packed word holds p in byte 0, q or t in byte 1, v in byte 2
                const unsigned sel = sector == 0 ? 0x3210u : sector == 1 ? 0x3120u : sector == 2 ? 0x3021u : sector == 3 ? 0x3012u
                                   : sector == 4 ? 0x3102u : 0x3201u;
                t.sector_f[h] = make_float2(__uint_as_float(sel), (sector & 1) ? f : 1.0f - f);
            }
        }

        // 8-bit BGR->HSV (H in [0,180)), hue shift, float32 HSV->BGR, as OpenCV computes them.
        __device__ __forceinline__ bgr hue_rotate(bgr p, bool truncate, const hue_tables& t)
        {
            const int  v    = __vimax3_s32(p.b, p.g, p.r);
            const int  vmin = __vimin3_s32(p.b, p.g, p.r);
            const int  diff = v - vmin;
            const int2 dv   = t.div[v];
            const int  s    = (diff * dv.x + (1 << 11)) >> 12;
            int        h;
            if (v == p.r)
                h = p.g - p.b;
            else if (v == p.g)
                h = p.b - p.r + 2 * diff;
            else
                h = p.r - p.g + 4 * diff;
            h = (h * t.div[diff].y + (1 << 11)) >> 12;
            h += (h >> 31) & 180;
            const float2 sf2 = t.sector_f[h];
            const float  sf  = t.unit[s];
            const float  vf  = t.unit[v];
            const float  f1  = vf * (1.0f - sf);
            const float  f2  = vf * __fmaf_rn(-sf, sf2.y, 1.0f);
            int          a, b, c; // products of two factors in [0,1] times 255: already inside 0..255
            if (truncate)
            {
                a = __float2int_rz(f1 * 255.0f);
                b = __float2int_rz(f2 * 255.0f);
                c = __float2int_rz(vf * 255.0f);
            }
            else
            {
                a = __float2int_rn(f1 * 255.0f);
                b = __float2int_rn(f2 * 255.0f);
                c = __float2int_rn(vf * 255.0f);
            }
            const unsigned packed = __byte_perm(__byte_perm(a, b, 0x3340), c, 0x3410);
            const unsigned o      = __byte_perm(packed, 0u, __float_as_uint(sf2.x));
            bgr            q;
            q.b = o & 0xFF;
            q.g = (o >> 8) & 0xFF;
            q.r = o >> 16;
            return q;
        }

        template <typename T>
        __device__ __forceinline__ T convert_out(int v);
        template <>
        __device__ __forceinline__ uint8_t convert_out<uint8_t>(int v) { return (uint8_t)v; }
        template <>
        __device__ __forceinline__ int8_t convert_out<int8_t>(int v) { return (int8_t)min(v, 127); }
        template <>
        __device__ __forceinline__ int16_t convert_out<int16_t>(int v) { return (int16_t)v; }
        template <>
        __device__ __forceinline__ uint16_t convert_out<uint16_t>(int v) { return (uint16_t)v; }
        template <>
        __device__ __forceinline__ int32_t convert_out<int32_t>(int v) { return v; }
        template <>
        __device__ __forceinline__ float convert_out<float>(int v) { return (float)v; }
        template <>
        __device__ __forceinline__ double convert_out<double>(int v) { return (double)v; }

        template <typename T>
        struct alignas(16) out_vec
        {
            static constexpr int N = 16 / sizeof(T);
            T                    v[N];
        };

        // Final per-channel value map applied after the spatial stage: contrast (with the image mean),
        // lighting, conversion to the output type and standardisation depend only on the channel and on
        // the 8-bit value, so each CTA tabulates them once (3 x 256 entries) and the store loop is a lookup.
        template <typename T>
        __device__ __forceinline__ T final_value(int v, int c, int cin, const aeonb_image_desc& d, const aeonb_image_layout& lay,
                                                 bool use_ctr, float ctr_add)
        {
            if (use_ctr)
                v = clamp_u8(__float2int_rn((float)v * d.contrast + ctr_add));
            if (d.lighting_enable)
            {
                v = clamp_u8(__float2int_rn((float)v * d.lighting_scale));
                v = clamp_u8(v + d.lighting_offset[cin]);
            }
            T e = convert_out<T>(v);
            if (lay.standardize)
                e = standardize_value(e, lay, c);
            return e;
        }

        __device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src)
        {
            const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem_src) : "memory");
        }
        __device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
        __device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

        // Horizontal result of one source row at one column: (S0*a0 + S1*a1) >> 4 per channel, as the vertical
        // pass of cv::resize reads it.
        struct hrow
        {
            int b, g, r;
        };

        // The staged bytes around the two taps of a column: `at` = byte offset in shared memory of tap 0.  Six (PIX 3)
        // or eight (PIX 4) bytes are needed; the aligned words around them are fetched and cut later.
        struct tap_words
        {
            uint32_t w0, w1, w2;
            int      sh;
        };
        template <int PIX>
        __device__ __forceinline__ tap_words load_taps(const unsigned char* smem, int at)
        {
            const uint32_t* p = reinterpret_cast<const uint32_t*>(smem + (at & ~3));
            tap_words       t;
            t.w0 = p[0];
            t.w1 = p[1];
            t.w2 = PIX == 3 ? p[2] : 0u;
            t.sh = at << 3; // the funnel shift takes the amount modulo 32
            return t;
        }
        template <int PIX>
        __device__ __forceinline__ hrow hpass_words(const tap_words& t, unsigned aw)
        {
            uint32_t lo = t.w0, hi = t.w1;
            if (PIX == 3)
            {
                lo = __funnelshift_r(t.w0, t.w1, t.sh);
                hi = __funnelshift_r(t.w1, t.w2, t.sh);
            }
            // byte pairs (tap 0, tap 1) of each channel in the low half of a word
            const unsigned pb = __byte_perm(lo, hi, PIX == 3 ? 0x0030 : 0x0040);
            const unsigned pg = __byte_perm(lo, hi, PIX == 3 ? 0x0041 : 0x0051);
            const unsigned pr = __byte_perm(lo, hi, PIX == 3 ? 0x0052 : 0x0062);
            hrow           h;
            h.b = (int)__dp2a_lo(aw, pb, 0u) >> 4;
            h.g = (int)__dp2a_lo(aw, pg, 0u) >> 4;
            h.r = (int)__dp2a_lo(aw, pr, 0u) >> 4;
            return h;
        }

        // Same from global memory, for crops too wide to stage a single row; a tap with weight zero is not read.
        template <int PIX>
        __device__ __forceinline__ hrow hpass_global(const uint8_t* tap0, unsigned aw)
        {
            int b0 = 0, g0 = 0, r0 = 0, b1 = 0, g1 = 0, r1 = 0;
            if (aw & 0xFFFFu)
                b0 = __ldg(tap0), g0 = __ldg(tap0 + 1), r0 = __ldg(tap0 + 2);
            if (aw >> 16)
                b1 = __ldg(tap0 + PIX), g1 = __ldg(tap0 + PIX + 1), r1 = __ldg(tap0 + PIX + 2);
            hrow h;
            h.b = (int)__dp2a_lo(aw, (unsigned)(b0 | (b1 << 8)), 0u) >> 4;
            h.g = (int)__dp2a_lo(aw, (unsigned)(g0 | (g1 << 8)), 0u) >> 4;
            h.r = (int)__dp2a_lo(aw, (unsigned)(r0 | (r1 << 8)), 0u) >> 4;
            return h;
        }

        // Store phase of a band: its (channel, row) lines are cut into 16-byte output chunks.  A thread keeps its chunk
        // column and walks down the lines, `lpp` lines apart (threads side by side write side by side), two lines at a
        // time so that their loads and stores overlap; tile offset and output pointer are stepped, not recomputed.
        // WHOLE: the band has no zero margin; IDENT: 8-bit output equal to the tile (margins of the tile are zero).
        template <typename T>
        struct store_args
        {
            const unsigned char* smem; // tile at offset 0
            const T*             lut;  // [3][256]
            T*                   dst;
            int                  rows, row0, out_w, out_h, slot_w, channels, pitch, plane;
            bool                 vec_ok;
            int64_t              sc, sy, sx;
        };

        template <typename T, bool WHOLE, bool IDENT>
        __device__ __forceinline__ void store_band(const store_args<T>& A, int tid, int nt)
        {
            constexpr int VEC    = out_vec<T>::N;
            const int     chunks = (A.slot_w + VEC - 1) / VEC;
            const int     lpp    = chunks <= nt ? nt / chunks : 1;
            const int     chunk0 = chunks <= nt ? tid % chunks : tid;
            const int     line0  = chunks <= nt ? tid / chunks : 0;
            if (line0 >= lpp)
                return;
            const T zero = convert_out<T>(0);
            struct cursor
            {
                int r, c, toff;
                T*  g;
            };
            const int     t_step = 2 * lpp * A.pitch, t_wrap = A.plane - A.rows * A.pitch;
            const int64_t g_step = 2 * lpp * A.sy, g_wrap = A.sc - A.rows * A.sy;
            auto          place  = [&](int line, int x0) {
                cursor q;
                q.c    = (line >= A.rows) + (line >= 2 * A.rows) + (line >= 3 * A.rows);
                q.r    = line - q.c * A.rows;
                q.toff = q.c * A.plane + q.r * A.pitch + x0;
                q.g    = A.dst + q.c * A.sc + (A.row0 + q.r) * A.sy + x0 * A.sx;
                return q;
            };
            auto advance = [&](cursor& q) {
                q.r += 2 * lpp;
                q.toff += t_step;
                q.g += g_step;
                for (int it = 0; it < 3 && q.r >= A.rows; ++it)
                {
                    q.r -= A.rows;
                    ++q.c;
                    q.toff += t_wrap;
                    q.g += g_wrap;
                }
            };
            auto put = [&](const cursor& q, int x0) {
                const unsigned char* px     = A.smem + q.toff;
                const bool           row_in = A.row0 + q.r < A.out_h;
                const T*             map    = A.lut + q.c * 256;
                out_vec<T>           o;
                if (VEC >= 4)
                {
                    uint32_t raw[VEC >= 4 ? VEC / 4 : 1];
    #pragma unroll
                    for (int w = 0; w < VEC / 4; ++w)
                        raw[w] = reinterpret_cast<const uint32_t*>(px)[w];
    #pragma unroll
                    for (int k = 0; k < VEC; ++k)
                    {
                        const unsigned v = (raw[k >> 2] >> (8 * (k & 3))) & 0xFF;
                        if (IDENT)
                            o.v[k] = (T)v;
                        else
                            o.v[k] = (WHOLE || (row_in && x0 + k < A.out_w)) ? map[v] : zero;
                    }
                }
                else
                {
    #pragma unroll
                    for (int k = 0; k < VEC; ++k)
                        o.v[k] = (WHOLE || (row_in && x0 + k < A.out_w)) ? map[px[k]] : zero;
                }
                if (A.vec_ok && x0 + VEC <= A.slot_w)
                    *reinterpret_cast<int4*>(q.g) = *reinterpret_cast<const int4*>(o.v);
                else
                    for (int k = 0; k < VEC && x0 + k < A.slot_w; ++k)
                        q.g[k * A.sx] = o.v[k];
            };
            for (int chunk = chunk0; chunk < chunks; chunk += nt)
            {
                const int x0 = chunk * VEC;
                cursor    qa = place(line0, x0), qb = place(line0 + lpp, x0);
                // every pass a cursor moves 2 * lpp lines down; c counts the planes passed (capped at 3 = past the end)
                for (int guard = 0; guard < 3 * A.rows && qa.c < A.channels; ++guard)
                {
                    put(qa, x0);
                    if (qb.c < A.channels)
                        put(qb, x0);
                    advance(qa);
                    advance(qb);
                }
            }
        }

        template <typename T, int PIX>
        __global__ void __launch_bounds__(AUG_MAX_THREADS, 5) aug_pack_kernel(const aug_launch L)
        {
            // Dynamic shared memory, addressed by 32-bit byte offsets:
            //   tile     [3][rows_per_band][pitch]   the band, planar uint8, output channel order
            //   ytab     int4[rows_per_band + 1]     per output row: k1 (position of tap 1 in the source row list; tap 0 is
            //                                        the entry before it), unused, b0, b1; a last entry with k1 = -1 ends it
            //   ysrc     int2[rows_per_band]         source rows of the two taps
            //   srow     int[2 rows_per_band]        the source rows of the band in the order of the horizontal pass
            //   rowaddr  int[2 rows_per_band]        per listed source row: offset of its first staged byte in shared memory
            //   stage    two buffers of staged source rows
            extern __shared__ __align__(16) unsigned char smem[];
            __shared__ aeonb_image_desc d;
            __shared__ unsigned int     part_sum[3];  // per-channel sums of the whole picture (output channel order); every
                                                      // CTA of the cluster adds its band's sums into every CTA's copy
            __shared__ unsigned int     cta_sum[3];   // this band's sums
            __shared__ float            contrast_add[3];
            __shared__ hue_tables       hue_tab;
            __shared__ T                lut[3][256];
            __shared__ int              blk_cols[2];  // source column of tap 0 of the first / last column of the column block
            __shared__ int              n_src_rows;   // listed source rows of the band
            __shared__ double           tap_scale[2]; // source / output size, x and y

            cg::cluster_group cluster = cg::this_cluster();
            const int         band    = blockIdx.x;
            const int         bands   = gridDim.x;
            const int         tid     = threadIdx.x;
            const int         nt      = blockDim.x;
            const int         lane    = tid & 31;
            const int         warp    = tid >> 5;
            const int         nwarps  = nt >> 5;
            const aeonb_image_layout& lay = L.layout;
            const int         RPB     = L.rows_per_band;
            const int         pitch   = L.tile_pitch;
            const int         plane   = RPB * pitch;

            int4*     ytab      = reinterpret_cast<int4*>(smem + 3 * plane);
            int2*     ysrc      = reinterpret_cast<int2*>(ytab + RPB + 1);
            int*      srow      = reinterpret_cast<int*>(ysrc + RPB);
            int*      rowaddr   = srow + 2 * RPB;
            const int off_stage = (3 * plane + 40 * RPB + 16 + 15) & ~15;

            // A cluster takes records rec, rec + gridDim.y, ...; the launcher starts one cluster per record.
            for (int rec = blockIdx.y; rec < L.n; rec += gridDim.y)
            {
                // ---- record descriptor -> shared memory
                {
                    const int* g = reinterpret_cast<const int*>(L.descs + rec);
                    int*       s = reinterpret_cast<int*>(&d);
                    for (int i = tid; i < (int)(sizeof(aeonb_image_desc) / sizeof(int)); i += nt)
                        s[i] = g[i];
                    if (tid < 3)
                        part_sum[tid] = cta_sum[tid] = 0;
                    if (tid == 32 % nt) // the two scale factors of the resize, once per CTA (two double divisions each)
                    {
                        const aeonb_image_desc& gd = L.descs[rec];
                        tap_scale[0] = 1.0 / ((double)gd.out_w / (double)gd.crop_w);
                        tap_scale[1] = 1.0 / ((double)gd.out_h / (double)gd.crop_h);
                    }
                }
                __syncthreads();

                const int  out_w    = d.src ? d.out_w : 0;
                const int  out_h    = d.src ? d.out_h : 0;
                const int  row0     = band * RPB;
                const int  row_end  = min(row0 + RPB, lay.slot_h);
                const int  img_end  = min(row_end, out_h); // rows that carry image data
                const int  nrows    = max(img_end - row0, 0);
                const bool use_hue  = d.hue != 0;
                const bool use_ctr  = d.contrast != 1.0f;
                const bool swap_rb  = lay.bgr_to_rgb != 0;
                const bool linear   = d.interp == AEONB_INTERP_LINEAR;
                const bool flip     = d.flip != 0;
                const int  src_w    = d.src_w;
                // The contrast step needs the sums of all bands.  This first arrival says "my part_sum is cleared"; the
                // matching wait comes right before the band's sums are sent, long after every CTA has got here.
                if (use_ctr)
                    cluster.barrier_arrive();

                // horizontal taps of this thread's column in the column block starting at xb
                int   sx0 = 0;
                short a0 = 2048, a1 = 0;
                auto  column_taps = [&](int xb) {
                    const int x = xb + tid;
                    sx0 = 0, a0 = 2048, a1 = 0;
                    if (x < out_w)
                    {
                        int s;
                        if (linear)
                            linear_tap(x, d.crop_w, tap_scale[0], true, s, a0, a1);
                        else
                            s = nearest_tap(x, d.crop_w, tap_scale[0]);
                        sx0 = d.crop_x + s - d.canvas_x;
                        if (tid == 0)
                            blk_cols[0] = sx0;
                        if (x == min(xb + nt, out_w) - 1)
                            blk_cols[1] = sx0;
                    }
                };

                // ---- tables.  Warp 0: vertical taps, then the list of source rows; meanwhile every thread: its horizontal taps.
                if (warp == 0)
                {
                    // source rows (clamped into the picture, weight zero when off it) and weights
                    for (int r = lane; r < nrows; r += 32)
                    {
                        int   y0, y1;
                        short b0 = 2048, b1 = 0;
                        if (linear)
                        {
                            int s;
                            linear_tap(row0 + r, d.crop_h, tap_scale[1], false, s, b0, b1);
                            y0 = min(max(s, 0), d.crop_h - 1);
                            y1 = min(max(s + 1, 0), d.crop_h - 1);
                        }
                        else
                            y0 = y1 = nearest_tap(row0 + r, d.crop_h, tap_scale[1]);
                        int sy0 = d.crop_y + y0 - d.canvas_y, sy1 = d.crop_y + y1 - d.canvas_y;
                        if ((unsigned)sy0 >= (unsigned)d.src_h)
                        {
                            b0  = 0;
                            sy0 = min(max(sy0, 0), d.src_h - 1);
                        }
                        if ((unsigned)sy1 >= (unsigned)d.src_h)
                        {
                            b1  = 0;
                            sy1 = min(max(sy1, 0), d.src_h - 1);
                        }
                        ysrc[r] = make_int2(sy0, sy1);
                        ytab[r] = make_int4(0, 0, b0, b1);
                    }
                    __syncwarp();
                    // Source rows of the band in the order the horizontal pass takes them, such that every output row finds
                    // its tap 1 at some position k1 and its tap 0 right before it.  A row whose taps coincide (clamped at the
                    // picture's edge, or nearest) needs one listed row when a weight is zero -- the weight then moves to tap 1
                    // -- and the same row listed twice otherwise.
                    if (lane == 0)
                    {
                        int K = 0;
                        for (int r = 0; r < nrows; ++r)
                        {
                            const int2 y = ysrc[r];
                            int4       t = ytab[r];
                            if (y.x != y.y)
                            {
                                if (K >= 2 && srow[K - 1] == y.y && srow[K - 2] == y.x)
                                    ;
                                else if (K >= 1 && srow[K - 1] == y.x)
                                    srow[K++] = y.y;
                                else
                                {
                                    srow[K++] = y.x;
                                    srow[K++] = y.y;
                                }
                            }
                            else if (t.z == 0 || t.w == 0)
                            {
                                if (t.w == 0)
                                {
                                    t.w = t.z;
                                    t.z = 0;
                                }
                                if (!(K >= 1 && srow[K - 1] == y.x))
                                    srow[K++] = y.x;
                            }
                            else
                            {
                                if (K >= 2 && srow[K - 1] == y.x && srow[K - 2] == y.x)
                                    ;
                                else if (K >= 1 && srow[K - 1] == y.x)
                                    srow[K++] = y.x;
                                else
                                {
                                    srow[K++] = y.x;
                                    srow[K++] = y.x;
                                }
                            }
                            t.x     = K - 1;
                            ytab[r] = t;
                        }
                        ytab[nrows] = make_int4(-1, 0, 0, 0);
                        n_src_rows  = K;
                    }
                }
                column_taps(0);
                if (use_hue)
                    build_hue_tables(hue_tab, d.hue, tid, nt);
                // the slot may be larger than the image: clear what the spatial stage will not write
                if (out_w < lay.slot_w || img_end < row_end)
                    for (int i = tid; i < 3 * plane / 16; i += nt)
                        reinterpret_cast<int4*>(smem)[i] = make_int4(0, 0, 0, 0);
                __syncthreads();

                // ---- resize + per-pixel photometric stages into the tile; a thread owns one output column of the band
                unsigned int sum_b = 0, sum_g = 0, sum_r = 0;
                {
                    // Record constants live in shared memory; byte stores into the tile could alias them, so the
                    // ones the pixel loop needs are copied to registers once.
                    const int   color_enable = d.color_enable;
                    const float cs0 = d.color_scale[0], cs1 = d.color_scale[1], cs2 = d.color_scale[2];
                    const int   m0 = d.color_matrix[0], m1 = d.color_matrix[1], m2 = d.color_matrix[2], m3 = d.color_matrix[3],
                                m4 = d.color_matrix[4], m5 = d.color_matrix[5], m6 = d.color_matrix[6], m7 = d.color_matrix[7],
                                m8 = d.color_matrix[8];
                    const int   hsv_cols = d.hsv_vector_cols;
                    const int      K         = n_src_rows;
                    const int      src_pitch = d.src_pitch;
                    const uint8_t* src       = d.src;
                    // the picture's bytes: a staged 16-byte group that is not wholly inside is fetched byte by byte
                    const uint8_t* mem_lo = src;
                    const uint8_t* mem_hi = src + (ptrdiff_t)(d.src_h - 1) * src_pitch + (ptrdiff_t)src_w * PIX;

                    for (int xb = 0; xb < out_w; xb += nt)
                    {
                        if (xb > 0)
                        {
                            column_taps(xb);
                            __syncthreads();
                        }
                        const int  x      = xb + tid;
                        const bool active = x < out_w;
                        // columns staged for this block: the taps of its first to last column, cut to the picture
                        const int bsa  = min(max(blk_cols[0], 0), src_w);
                        const int bsb  = max(min(blk_cols[1] + 2, src_w), bsa);
                        const int span = (bsb - bsa) * PIX;
                        const int stage_pitch = ((span + 30) & ~15) + 2 * AUG_STAGE_PAD; // room for a lead of up to 15 bytes
                        const int R = min(AUG_MAX_GROUP, (L.stage_bytes / 2) / stage_pitch);
                        if (a0 != 0 && (unsigned)sx0 >= (unsigned)src_w)
                            a0 = 0;
                        if (a1 != 0 && (unsigned)(sx0 + 1) >= (unsigned)src_w)
                            a1 = 0;
                        const unsigned aw  = (unsigned)(unsigned short)a0 | ((unsigned)(unsigned short)a1 << 16);
                        const int      sxc = min(max(sx0, bsa - 1), max(bsb - 1, bsa - 1)); // keeps both taps next to the staged bytes
                        const int      off = (sxc - bsa) * PIX;
                        const int      xo_t = flip ? out_w - 1 - x : x;
                        const bool     truncate = x < hsv_cols;
                        // tile positions of this column's B, G, R bytes (output channel order), stepped down a row per pixel
                        int tb = (swap_rb ? 2 * plane : 0) + xo_t, tg = plane + xo_t, tr = (swap_rb ? 0 : 2 * plane) + xo_t;

                        hrow h_prev{0, 0, 0}, h_cur{0, 0, 0};
                        int  r   = 0;
                        int4 tap = ytab[0]; // taps of the next output row to emit
                        // rows whose second tap is listed row k are complete once that row's horizontal pass is done
                        auto emit_ready = [&](int k) {
                            for (int guard = 0; guard <= nrows && tap.x == k; ++guard)
                            {
                                const int b0 = tap.z, b1 = tap.w;
                                // vertical pass as in OpenCV's 8-bit path; with weights summing to 2048 the result stays in 0..255
                                const int pb = (((b0 * h_prev.b) >> 16) + ((b1 * h_cur.b) >> 16) + 2) >> 2;
                                const int pg = (((b0 * h_prev.g) >> 16) + ((b1 * h_cur.g) >> 16) + 2) >> 2;
                                const int pr = (((b0 * h_prev.r) >> 16) + ((b1 * h_cur.r) >> 16) + 2) >> 2;
                                ++r;
                                tap = ytab[r];
                                bgr px{pb, pg, pr};
                                if (color_enable == 2)
                                {
                                    px.b = clamp_u8(__float2int_rn((float)px.b * cs0));
                                    px.g = clamp_u8(__float2int_rn((float)px.g * cs1));
                                    px.r = clamp_u8(__float2int_rn((float)px.r * cs2));
                                }
                                else if (color_enable)
                                {
                                    const int b  = (px.b * m0 + px.g * m1 + px.r * m2 + 512) >> 10;
                                    const int g  = (px.b * m3 + px.g * m4 + px.r * m5 + 512) >> 10;
                                    const int rr = (px.b * m6 + px.g * m7 + px.r * m8 + 512) >> 10;
                                    px.b = clamp_u8(b);
                                    px.g = clamp_u8(g);
                                    px.r = clamp_u8(rr);
                                }
                                if (use_hue)
                                    px = hue_rotate(px, truncate, hue_tab);
                                smem[tb] = (unsigned char)px.b;
                                smem[tg] = (unsigned char)px.g;
                                smem[tr] = (unsigned char)px.r;
                                tb += pitch;
                                tg += pitch;
                                tr += pitch;
                                sum_b += px.b;
                                sum_g += px.g;
                                sum_r += px.r;
                            }
                        };

                        if (R >= 1)
                        {
                            // copies of group g (listed rows g*R ...) into buffer g & 1; a warp takes a row, a lane 16 bytes at a
                            // time; the staged copy keeps the row's alignment modulo 16
                            auto issue = [&](int g) {
                                const int k_end = min((g + 1) * R, K);
                                for (int k = g * R + warp; k < k_end; k += nwarps)
                                {
                                    const uint8_t* first = src + (ptrdiff_t)srow[k] * src_pitch + (ptrdiff_t)bsa * PIX;
                                    const int      lead  = (int)((uintptr_t)first & 15);
                                    const uint8_t* g0    = first - lead;
                                    const int      s0    = off_stage + ((g & 1) * R + (k - g * R)) * stage_pitch + AUG_STAGE_PAD;
                                    const int      nck   = span ? (lead + span + 15) >> 4 : 0;
                                    if (lane == 0)
                                        rowaddr[k] = s0 + lead;
                                    if (g0 >= mem_lo && g0 + nck * 16 <= mem_hi)
                                        for (int c = lane; c < nck; c += 32)
                                            cp_async_16(smem + s0 + c * 16, g0 + c * 16);
                                    else // first or last row of a picture that is not 16-byte aligned
                                        for (int c = lane; c < nck; c += 32)
                                        {
                                            const uint8_t* gp = g0 + c * 16;
                                            if (gp >= mem_lo && gp + 16 <= mem_hi)
                                                cp_async_16(smem + s0 + c * 16, gp);
                                            else
                                                for (int b = 0; b < 16; ++b)
                                                    smem[s0 + c * 16 + b] = (gp + b >= mem_lo && gp + b < mem_hi) ? __ldg(gp + b) : (uint8_t)0;
                                        }
                                }
                                cp_async_commit();
                            };
                            const int ngroups = (K + R - 1) / R;
                            if (ngroups > 0)
                                issue(0);
                            for (int g = 0; g < ngroups; ++g)
                            {
                                cp_async_wait_all();
                                __syncthreads(); // group g is in shared memory for every thread; group g - 1 has been consumed
                                if (g + 1 < ngroups)
                                    issue(g + 1); // into the buffer group g - 1 used; lands while group g is processed
                                if (active)
                                {
                                    const int k_end = min((g + 1) * R, K);
                                    // the words of the next row are fetched before the tile stores of this one
                                    tap_words next = load_taps<PIX>(smem, rowaddr[g * R] + off);
                                    for (int k = g * R; k < k_end; ++k)
                                    {
                                        const tap_words cur = next;
                                        if (k + 1 < k_end)
                                            next = load_taps<PIX>(smem, rowaddr[k + 1] + off);
                                        h_prev = h_cur;
                                        h_cur  = hpass_words<PIX>(cur, aw);
                                        emit_ready(k);
                                    }
                                }
                            }
                        }
                        else if (active)
                        {
                            // a single source row of this block does not fit the staging buffer: taps straight from global memory
                            for (int k = 0; k < K; ++k)
                            {
                                h_prev = h_cur;
                                h_cur  = hpass_global<PIX>(src + (ptrdiff_t)srow[k] * src_pitch + (ptrdiff_t)sxc * PIX, aw);
                                emit_ready(k);
                            }
                        }
                        __syncthreads(); // the band's pixels are in the tile; blk_cols, the row table and the staging buffers are free
                    }
                }

                if (use_ctr)
                {
                    sum_b = warp_sum(sum_b);
                    sum_g = warp_sum(sum_g);
                    sum_r = warp_sum(sum_r);
                    if (lane == 0)
                    {
                        atomicAdd(&cta_sum[swap_rb ? 2 : 0], sum_b);
                        atomicAdd(&cta_sum[1], sum_g);
                        atomicAdd(&cta_sum[swap_rb ? 0 : 2], sum_r);
                    }
                }

                // ---- per-image channel means for contrast: every CTA adds its sums into every CTA of the cluster through
                // distributed shared memory, so the mean never touches global memory
                if (use_ctr)
                {
                    __syncthreads();        // cta_sum complete
                    cluster.barrier_wait(); // every CTA of the cluster has cleared its part_sum (arrival at the top)
                    if (tid < 3 * bands)
                    {
                        const int peer = tid / 3, c = tid - 3 * peer;
                        atomicAdd(cluster.map_shared_rank(&part_sum[c], peer), cta_sum[c]);
                    }
                    cluster.sync(); // all bands' sums have arrived here; nothing touches another CTA's memory afterwards
                    if (tid < 3)
                    {
                        const double mean = (double)part_sum[tid] / (double)((long long)out_w * out_h);
                        contrast_add[tid] = (float)((1.0 - (double)d.contrast) * mean);
                    }
                    __syncthreads();
                }

                // ---- value map: contrast, lighting, conversion, standardisation
                // (8-bit output without contrast or lighting is the identity: the store loop then skips the lookup)
                const bool identity = sizeof(T) == 1 && !use_ctr && !d.lighting_enable && lay.dtype == AEONB_U8;
                if (!identity)
                {
                    for (int i = tid; i < 768; i += nt)
                    {
                        const int c   = i >> 8;
                        const int cin = swap_rb ? 2 - c : c; // channel index in BGR order
                        lut[c][i & 255] = final_value<T>(i & 255, c, cin, d, lay, use_ctr, use_ctr ? contrast_add[c] : 0.f);
                    }
                }
                __syncthreads(); // tile and value map complete

                // ---- store
                {
                    store_args<T> A;
                    A.smem = smem, A.lut = &lut[0][0], A.dst = reinterpret_cast<T*>(d.dst);
                    A.rows = row_end - row0, A.row0 = row0, A.out_w = out_w, A.out_h = out_h, A.slot_w = lay.slot_w;
                    A.channels = lay.channels, A.pitch = pitch, A.plane = plane, A.vec_ok = L.vector_ok != 0;
                    A.sc = lay.stride_c, A.sy = lay.stride_y, A.sx = lay.stride_x;
                    const bool whole = out_w == lay.slot_w && img_end == row_end; // no zero margin in this band
                    if (identity)
                        store_band<T, true, true>(A, tid, nt);
                    else if (whole)
                        store_band<T, true, false>(A, tid, nt);
                    else
                        store_band<T, false, false>(A, tid, nt);
                }

                __syncthreads(); // the next record reuses the descriptor, the tables and the tile
            }
        }

        template <typename T>
        cudaError_t launch_typed(const aug_launch& L, int clusters, int bands, int cluster_size, int threads, size_t smem, int pix,
                                 cudaStream_t stream)
        {
            auto kern = pix == 4 ? aug_pack_kernel<T, 4> : aug_pack_kernel<T, 3>;
            // the dynamic shared-memory limit of a kernel is a per-device setting: raised only when a launch needs more
            static std::atomic<int> limit[2][64];
            int                     device = 0;
            cudaError_t             err    = cudaGetDevice(&device);
            if (err != cudaSuccess)
                return err;
            std::atomic<int>& have = limit[pix == 4][device & 63];
            if ((int)smem > have.load(std::memory_order_relaxed))
            {
                err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (err != cudaSuccess)
                    return err;
                have.store((int)smem, std::memory_order_relaxed);
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim            = dim3(bands, clusters, 1);
            cfg.blockDim           = dim3(threads, 1, 1);
            cfg.dynamicSmemBytes   = smem;
            cfg.stream             = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id               = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = cluster_size;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs                = attr;
            cfg.numAttrs             = 1;
            return cudaLaunchKernelEx(&cfg, kern, L);
        }
    }

    // Host entry used by the C ABI: `descs_dev` is the device copy of the descriptors `descs_host`.
    // Returns a CUDA error; *why is set for configurations the kernel does not cover.
    cudaError_t launch_aug_pack(const aeonb_image_desc* descs_dev, const aeonb_image_desc* descs_host, int n,
                                const aeonb_image_layout& layout, int pixel_stride, bool slots_aligned, cudaStream_t stream,
                                const char** why)
    {
        *why = nullptr;
        bool any_contrast = false;
        int  max_cols     = 1; // widest stretch of source columns any record reads
        for (int i = 0; i < n; ++i)
        {
            const aeonb_image_desc& r = descs_host[i];
            any_contrast |= r.contrast != 1.0f;
            if (r.src)
                max_cols = std::max(max_cols, std::min(r.crop_w, r.src_w));
        }
        int bands = 1;
        while (bands < AUG_MAX_BAND && layout.slot_h / (bands * 2) >= 8)
            bands *= 2;
        aug_launch L;
        L.tile_pitch = (layout.slot_w + 15) / 16 * 16;
        // One thread per output column; wider outputs are cut into equal column blocks.
        const int col_blocks = (layout.slot_w + AUG_MAX_THREADS - 1) / AUG_MAX_THREADS;
        const int threads    = std::min(AUG_MAX_THREADS, std::max(64, ((layout.slot_w + col_blocks - 1) / col_blocks + 31) / 32 * 32));
        // Staging: two buffers of up to 8 source rows of the widest crop (a column block of a wide output reads a part
        // of the row only), at most 16 KB each; a record whose rows are longer stages fewer rows per group.
        const int row_bytes = std::min(max_cols, (max_cols + col_blocks - 1) / col_blocks + 2) * pixel_stride + 30 + 2 * AUG_STAGE_PAD;
        L.stage_bytes       = std::min(2 * 8 * ((row_bytes + 15) & ~15), 16 * 1024);
        auto smem_for = [&](int nb) {
            const int rows = (layout.slot_h + nb - 1) / nb;
            size_t    s    = (size_t)3 * rows * L.tile_pitch + (size_t)rows * 40 + 16; // tile + the row tables of the kernel
            return ((s + 15) & ~(size_t)15) + L.stage_bytes;
        };
        // A band has to fit the shared memory of one CTA.  Up to AUG_MAX_BAND bands form one cluster, which is what the
        // contrast step needs (the per-image mean travels through distributed shared memory).  Larger outputs (a
        // 1000 x 1000 detection input, say) take more, independent bands -- possible whenever no record of the batch
        // changes the contrast.
        while (smem_for(bands) > 200 * 1024 && bands < 256 && layout.slot_h / (bands * 2) >= 1)
            bands *= 2;
        if (bands > AUG_MAX_BAND && any_contrast)
        {
            *why = "a contrast change on an output too large for 8 on-chip bands (rows/8 * width * 3 over 200 KB) is outside the accelerated path";
            return cudaErrorInvalidValue;
        }
        L.descs         = descs_dev;
        L.layout        = layout;
        L.rows_per_band = (layout.slot_h + bands - 1) / bands;
        const size_t elem = layout.dtype == AEONB_F64 ? 8 : layout.dtype == AEONB_F32 || layout.dtype == AEONB_I32 ? 4
                          : layout.dtype == AEONB_I16 || layout.dtype == AEONB_U16 ? 2 : 1;
        L.n         = n;
        L.vector_ok = slots_aligned && layout.stride_x == 1 && (layout.stride_y * elem) % 16 == 0 &&
                      (layout.stride_c * elem) % 16 == 0;
        const size_t smem = smem_for(bands);
        if (smem > 200 * 1024)
        {
            *why = "output image too large for the on-chip band tile (one row of width * 3 bytes must stay under 200 KB)";
            return cudaErrorInvalidValue;
        }
        const int cluster_size = bands <= AUG_MAX_BAND ? bands : 1;
        // One cluster per record.  (The kernel can also run as fewer, persistent clusters that loop over records;
        // measured on B200 that was slower because records differ in cost and the hardware's own dispatch balances
        // them better than a static round-robin.)
        const int clusters = n;
        switch (layout.dtype)
        {
        case AEONB_U8: return launch_typed<uint8_t>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_I8: return launch_typed<int8_t>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_I16: return launch_typed<int16_t>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_U16: return launch_typed<uint16_t>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_I32: return launch_typed<int32_t>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_F32: return launch_typed<float>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        case AEONB_F64: return launch_typed<double>(L, clusters, bands, cluster_size, threads, smem, pixel_stride, stream);
        }
        *why = "unknown output dtype";
        return cudaErrorInvalidValue;
    }
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the image batch call.
//
// aeonb_image_batch keeps a device copy of the descriptor array in buffers it obtains with
// cudaMalloc / cudaMallocHost.  Some callers must not allocate: code running inside a memory-pool
// or graph-building phase of a framework that forbids allocator calls, processes that were handed
// a fixed memory budget at start-up, and latency-critical loops that cannot afford the implicit
// device synchronisation an allocation may cause.  For them the descriptor copy below lives in a
// fixed array inside the library image itself.
// ------------------------------------------------------------------------------------------------

#include <mutex>
#include <string>

#include "context.hpp"



namespace aeonb
{
    namespace
    {
        // Device copy of the descriptors of one call.  Every GPU that loads the library holds these
        // AEONB_NOALLOC_MAX_RECORDS * sizeof(aeonb_image_desc) bytes (about 76 KB) until the process exits.
        static __device__ __align__(256) unsigned char g_noalloc_descs[AEONB_NOALLOC_MAX_RECORDS * sizeof(aeonb_image_desc)];

        constexpr int MAX_DEVICES = 64;
        void*         g_noalloc_addr[MAX_DEVICES]; // per-device address of g_noalloc_descs, 0 until set up
        std::mutex    g_noalloc_mutex;

        // In host code `g_noalloc_descs` names a host-side shadow, not device memory; the address a
        // kernel may use comes from cudaGetSymbolAddress, asked once per device with that device current.
        void* noalloc_scratch(int device)
        {
            std::lock_guard<std::mutex> lk(g_noalloc_mutex);
            if (!g_noalloc_addr[device])
            {
                void* p = nullptr;
                AEONB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_descs));
                g_noalloc_addr[device] = p;
            }
            return g_noalloc_addr[device];
        }
    }
}

extern "C" int aeonb_image_batch_noalloc(const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout, void* stream)
{
    using namespace aeonb;
    return guarded([&]() {
        if (!layout || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_image_batch_noalloc: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        if (n > AEONB_NOALLOC_MAX_RECORDS)
            throw std::invalid_argument("aeonb_image_batch_noalloc: at most " + std::to_string(AEONB_NOALLOC_MAX_RECORDS) +
                                        " records per call (the descriptor scratch is a fixed array); split the batch");
        int  pixel_stride;
        bool aligned;
        check_image_batch(descs, n, *layout, pixel_stride, aligned);
        int device = 0;
        AEONB_CUDA(cudaGetDevice(&device));
        if (device < 0 || device >= MAX_DEVICES)
            throw std::invalid_argument("aeonb_image_batch_noalloc: device index out of range");
        auto*        scratch = static_cast<aeonb_image_desc*>(noalloc_scratch(device));
        cudaStream_t st      = static_cast<cudaStream_t>(stream);
        // Every descriptor the kernel reads is overwritten here, so nothing of the previous call survives.
        AEONB_CUDA(cudaMemcpyAsync(scratch, descs, sizeof(aeonb_image_desc) * n, cudaMemcpyHostToDevice, st));
        const char* why = nullptr;
        cudaError_t e   = launch_aug_pack(scratch, descs, n, *layout, pixel_stride, aligned, st, &why);
        if (why)
            throw error(AEONB_ERR_UNSUPPORTED, why);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("image kernel launch", e));
        return AEONB_OK;
    });
}
