// Image augmentation + packing kernel for sm_100a.
//
// One launch transforms a whole batch.  A record is handled by a thread-block cluster of
// `bands` CTAs; CTA b owns a band of output rows.  Each CTA
//   1. builds the horizontal / vertical bilinear tap tables of the crop->output resize
//      (the 11-bit fixed-point form cv::resize(INTER_LINEAR) uses for 8-bit images),
//   2. resizes its band straight from the source image in global memory, applies the
//      brightness/saturation matrix and the HSV hue shift per pixel, and keeps the band
//      as planar uint8 in shared memory, already flipped and in output channel order,
//   3. if contrast is active, reduces per-channel sums (warp shuffles, then shared memory)
//      and exchanges the partial sums with the other CTAs of the cluster through
//      distributed shared memory, so the per-image mean never touches global memory,
//   4. applies contrast and lighting, converts to the output type, standardises and
//      streams the band out with 128-bit stores into the record's slot of the batch buffer.
//
// The arithmetic of every stage is the integer / float32 arithmetic OpenCV applies for the
// calls aeon makes (src/etl_image.cpp:146-202, src/image.cpp:336-406, src/etl_image.cpp:246-341);
// this file is compiled with -fmad=false and uses explicit fused operations only where
// OpenCV's own code is fused.
#include <algorithm>

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
        constexpr int AUG_THREADS  = 256;
        constexpr int AUG_MAX_BAND = 8; // portable cluster size limit

        struct aug_launch
        {
            const aeonb_image_desc* descs; // device copy
            aeonb_image_layout      layout;
            int                     rows_per_band;
            int                     tile_pitch; // bytes per tile row (multiple of 16)
            int                     vector_ok;  // slots are 16-byte aligned with unit x stride
            int                     n;          // records in the batch
        };

        struct row_tap
        {
            int   y0, y1; // source rows inside the crop box (already clamped)
            short b0, b1;
        };

        __device__ __forceinline__ int clamp_u8(int v) { return min(max(v, 0), 255); }

        __device__ __forceinline__ short sat_s16(int v) { return (short)min(max(v, -32768), 32767); }

        // Source index and tap weights for destination index d (cv::resize, INTER_LINEAR, 8-bit).
        __device__ __forceinline__ void linear_tap(int d, int src_len, int dst_len, bool clamp_weights, int& s, short& w0, short& w1)
        {
            const double scale = 1.0 / ((double)dst_len / (double)src_len);
            float        f     = (float)(((double)d + 0.5) * scale - 0.5);
            float        fl    = floorf(f);
            s                  = (int)fl;
            f                  = f - fl;
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

        __device__ __forceinline__ int nearest_tap(int d, int src_len, int dst_len)
        {
            const double scale = 1.0 / ((double)dst_len / (double)src_len);
            return min((int)floor((double)d * scale), src_len - 1);
        }

        struct bgr
        {
            int b, g, r;
        };

        // Pixel of the (virtual) canvas at crop-relative coordinates.
        template <int PIX>
        __device__ __forceinline__ bgr fetch(const aeonb_image_desc& d, int x, int y)
        {
            const int sx = d.crop_x + x - d.canvas_x;
            const int sy = d.crop_y + y - d.canvas_y;
            bgr       p{0, 0, 0};
            if ((unsigned)sx < (unsigned)d.src_w && (unsigned)sy < (unsigned)d.src_h)
            {
                const uint8_t* s = d.src + (size_t)sy * d.src_pitch + (size_t)sx * PIX;
                if (PIX == 4)
                {
                    const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(s));
                    p.b              = v & 0xFF;
                    p.g              = (v >> 8) & 0xFF;
                    p.r              = (v >> 16) & 0xFF;
                }
                else
                {
                    p.b = __ldg(s);
                    p.g = __ldg(s + 1);
                    p.r = __ldg(s + 2);
                }
            }
            return p;
        }

        template <int PIX>
        __device__ __forceinline__ bgr load_px(const uint8_t* s)
        {
            bgr p;
            if (PIX == 4)
            {
                const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(s));
                p.b              = v & 0xFF;
                p.g              = (v >> 8) & 0xFF;
                p.r              = (v >> 16) & 0xFF;
            }
            else
            {
                p.b = __ldg(s);
                p.g = __ldg(s + 1);
                p.r = __ldg(s + 2);
            }
            return p;
        }

        // 8-bit BGR->HSV (H in [0,180)) with 12-bit reciprocal tables, then the hue shift with C
        // remainder semantics stored through a uint8_t, then float32 HSV->BGR.
        // Per-CTA tables of the hue stage (all exact restatements of the per-pixel arithmetic, tabulated once):
        //   sdiv/hdiv : the 12-bit reciprocals of 8-bit BGR->HSV;
        //   sector_f  : for a hue h in [0,180), after the shift uint8((h + hue) % 180): the HSV->BGR sector and
        //               the fractional position inside it;
        //   unit      : x * (1/255) for x in [0,255] (the float S and V).
        struct hue_tables
        {
            int    sdiv[256];
            int    hdiv[256];
            float2 sector_f[180]; // .x = sector as a float bit pattern of an int, .y = f
            float  unit[256];
        };

        __device__ __forceinline__ void build_hue_tables(hue_tables& t, int hue, int tid, int nthreads)
        {
            for (int i = tid; i < 256; i += nthreads)
            {
                t.sdiv[i] = i ? __double2int_rn((double)(255 << 12) / (double)i) : 0;
                t.hdiv[i] = i ? __double2int_rn((double)(180 << 12) / (6.0 * (double)i)) : 0;
                t.unit[i] = (float)i * (1.0f / 255.0f);
            }
            for (int h = tid; h < 180; h += nthreads)
            {
                const int   hs = ((h + hue) % 180) & 0xFF; // C remainder, stored through a uint8_t
                const float hf = (float)hs * (6.0f / 180.0f);
                const float fl = floorf(hf);
                int         sector = (int)fl;
                if (sector >= 6)
                    sector -= 6; // hs <= 255 gives sector <= 8
                t.sector_f[h] = make_float2(__int_as_float(sector), hf - fl);
            }
        }

        // 8-bit BGR->HSV (H in [0,180)), hue shift, float32 HSV->BGR, as OpenCV computes them.
        __device__ __forceinline__ bgr hue_rotate(bgr p, bool truncate, const hue_tables& t)
        {
            const int v    = max(max(p.b, p.g), p.r);
            const int vmin = min(min(p.b, p.g), p.r);
            const int diff = v - vmin;
            const int s    = (diff * t.sdiv[v] + (1 << 11)) >> 12;
            int       h;
            if (v == p.r)
                h = p.g - p.b;
            else if (v == p.g)
                h = p.b - p.r + 2 * diff;
            else
                h = p.r - p.g + 4 * diff;
            h = (h * t.hdiv[diff] + (1 << 11)) >> 12;
            if (h < 0)
                h += 180;
            const float2 sf2    = t.sector_f[h];
            const int    sector = __float_as_int(sf2.x);
            const float  f      = sf2.y;
            const float  sf     = t.unit[s];
            const float  vf     = t.unit[v];
            const float t1 = vf * (1.0f - sf);
            const float t2 = vf * __fmaf_rn(-sf, f, 1.0f);
            const float t3 = vf * __fmaf_rn(-sf, 1.0f - f, 1.0f);
            // sector -> (b, g, r): 0 (t1,t3,v) 1 (t1,v,t2) 2 (t3,v,t1) 3 (v,t2,t1) 4 (v,t1,t3) 5 (t2,t1,v); selects, no branches
            const float fb = sector < 2 ? t1 : sector == 2 ? t3 : sector < 5 ? vf : t2;
            const float fg = sector == 0 ? t3 : sector < 3 ? vf : sector == 3 ? t2 : t1;
            const float fr = sector == 0 ? vf : sector == 1 ? t2 : sector < 4 ? t1 : sector == 4 ? t3 : vf;
            bgr o; // products of two factors in [0,1] times 255: already inside 0..255
            if (truncate)
            {
                o.b = __float2int_rz(fb * 255.0f);
                o.g = __float2int_rz(fg * 255.0f);
                o.r = __float2int_rz(fr * 255.0f);
            }
            else
            {
                o.b = __float2int_rn(fb * 255.0f);
                o.g = __float2int_rn(fg * 255.0f);
                o.r = __float2int_rn(fr * 255.0f);
            }
            return o;
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
        struct out_vec
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

        template <typename T, int PIX>
        __global__ void __launch_bounds__(AUG_THREADS, 4) aug_pack_kernel(const aug_launch L)
        {
            extern __shared__ __align__(16) unsigned char smem[];
            __shared__ aeonb_image_desc d;
            __shared__ unsigned int     part_sum[3];  // this CTA's per-channel sums (output channel order)
            __shared__ float            contrast_add[3];
            __shared__ hue_tables       hue_tab;
            __shared__ T                lut[3][256];

            cg::cluster_group cluster = cg::this_cluster();
            const int         band    = blockIdx.x;
            const int         bands   = gridDim.x;
            const int         tid     = threadIdx.x;
            const int         lane    = tid & 31;
            const int         warp    = tid >> 5;
            constexpr int     WARPS   = AUG_THREADS / 32;
            const aeonb_image_layout& lay = L.layout;

            // A cluster takes records rec, rec + gridDim.y, ...; the launcher starts one cluster per record.
            for (int rec = blockIdx.y; rec < L.n; rec += gridDim.y)
            {
                // ---- record descriptor -> shared memory
                {
                    const int* g = reinterpret_cast<const int*>(L.descs + rec);
                    int*       s = reinterpret_cast<int*>(&d);
                    for (int i = tid; i < (int)(sizeof(aeonb_image_desc) / sizeof(int)); i += AUG_THREADS)
                        s[i] = g[i];
                    if (tid < 3)
                        part_sum[tid] = 0;
                }
                __syncthreads();

                const int  out_w    = d.src ? d.out_w : 0;
                const int  out_h    = d.src ? d.out_h : 0;
                const int  row0     = band * L.rows_per_band;
                const int  row_end  = min(row0 + L.rows_per_band, lay.slot_h);
                const int  img_end  = min(row_end, out_h); // rows that carry image data
                const int  pitch    = L.tile_pitch;
                const int  plane    = L.rows_per_band * pitch;
                const bool use_hue  = d.hue != 0;
                const bool use_ctr  = d.contrast != 1.0f;
                const bool swap_rb  = lay.bgr_to_rgb != 0;
                const bool linear   = d.interp == AEONB_INTERP_LINEAR;
                // the whole crop box lies on the source picture: no canvas test per tap
                const bool inside = d.crop_x >= d.canvas_x && d.crop_y >= d.canvas_y && d.crop_x + d.crop_w <= d.canvas_x + d.src_w &&
                                    d.crop_y + d.crop_h <= d.canvas_y + d.src_h;

                unsigned char* tile = smem;                                            // [3][rows_per_band][pitch]
                int2*          xofs = reinterpret_cast<int2*>(smem + 3 * plane);       // [out_w] byte offsets of the two taps
                short2*        xw   = reinterpret_cast<short2*>(xofs + lay.slot_w);    // [out_w]
                row_tap*       ytab = reinterpret_cast<row_tap*>(xw + lay.slot_w);     // [rows_per_band]

                // ---- tap tables
                for (int x = tid; x < out_w; x += AUG_THREADS)
                {
                    int   s;
                    short a0 = 2048, a1 = 0;
                    if (linear)
                        linear_tap(x, d.crop_w, out_w, true, s, a0, a1);
                    else
                        s = nearest_tap(x, d.crop_w, out_w);
                    const int s1 = min(s + 1, d.crop_w - 1);
                    xofs[x]      = inside ? make_int2(s * PIX, s1 * PIX) : make_int2(s, s1);
                    xw[x]        = make_short2(a0, a1);
                }
                for (int r = tid; r < img_end - row0; r += AUG_THREADS)
                {
                    row_tap t;
                    if (linear)
                    {
                        int s;
                        linear_tap(row0 + r, d.crop_h, out_h, false, s, t.b0, t.b1);
                        t.y0 = min(max(s, 0), d.crop_h - 1);
                        t.y1 = min(max(s + 1, 0), d.crop_h - 1);
                    }
                    else
                    {
                        t.y0 = t.y1 = nearest_tap(row0 + r, d.crop_h, out_h);
                        t.b0        = 2048;
                        t.b1        = 0;
                    }
                    ytab[r] = t;
                }
                if (use_hue)
                    build_hue_tables(hue_tab, d.hue, tid, AUG_THREADS);
                // the slot may be larger than the image: clear what the spatial stage will not write
                if (out_w < lay.slot_w || img_end < row_end)
                    for (int i = tid; i < 3 * plane / 16; i += AUG_THREADS)
                        reinterpret_cast<int4*>(tile)[i] = make_int4(0, 0, 0, 0);
                __syncthreads();

                // ---- resize + per-pixel photometric into the tile; a warp takes 32 consecutive pixels of a row
                unsigned int sum0 = 0, sum1 = 0, sum2 = 0;
                {
                    const int      rows  = max(img_end - row0, 0);
                    const int      nseg  = (out_w + 31) >> 5;
                    const int      units = rows * nseg;
                    const uint8_t* base  = d.src + (ptrdiff_t)(d.crop_y - d.canvas_y) * d.src_pitch + (ptrdiff_t)(d.crop_x - d.canvas_x) * PIX;
                    // Record constants live in shared memory; byte stores into the tile could alias them, so the
                    // ones the pixel loop needs are copied to registers once.
                    const int   src_pitch    = d.src_pitch;
                    const int   color_enable = d.color_enable;
                    const float cs0 = d.color_scale[0], cs1 = d.color_scale[1], cs2 = d.color_scale[2];
                    const int   m0 = d.color_matrix[0], m1 = d.color_matrix[1], m2 = d.color_matrix[2], m3 = d.color_matrix[3],
                                m4 = d.color_matrix[4], m5 = d.color_matrix[5], m6 = d.color_matrix[6], m7 = d.color_matrix[7],
                                m8 = d.color_matrix[8];
                    const int   hsv_cols = d.hsv_vector_cols;
                    const bool  flip = d.flip != 0;

                    struct taps
                    {
                        bgr     p00, p01, p10, p11;
                        short2  a;
                        short   b0, b1;
                        int     x, r;
                        bool    valid;
                    };
                    // all global loads of one unit (32 pixels of a row), issued before any arithmetic on them
                    auto load_unit = [&](int r, int seg) {
                        taps k;
                        k.r     = r;
                        k.x     = seg * 32 + lane;
                        k.valid = r < rows && k.x < out_w;
                        if (!k.valid)
                            return k;
                        const row_tap t  = ytab[k.r];
                        const int2    xo = xofs[k.x];
                        k.a  = xw[k.x];
                        k.b0 = t.b0;
                        k.b1 = t.b1;
                        if (inside)
                        {
                            const uint8_t* r0 = base + (ptrdiff_t)t.y0 * src_pitch;
                            const uint8_t* r1 = base + (ptrdiff_t)t.y1 * src_pitch;
                            k.p00 = load_px<PIX>(r0 + xo.x);
                            if (linear)
                            {
                                k.p01 = load_px<PIX>(r0 + xo.y);
                                k.p10 = load_px<PIX>(r1 + xo.x);
                                k.p11 = load_px<PIX>(r1 + xo.y);
                            }
                        }
                        else
                        {
                            k.p00 = fetch<PIX>(d, xo.x, t.y0);
                            if (linear)
                            {
                                k.p01 = fetch<PIX>(d, xo.y, t.y0);
                                k.p10 = fetch<PIX>(d, xo.x, t.y1);
                                k.p11 = fetch<PIX>(d, xo.y, t.y1);
                            }
                        }
                        return k;
                    };
                    auto finish_unit = [&](const taps& k) {
                        if (!k.valid)
                            return;
                        bgr px = k.p00;
                        if (linear)
                        {
                            // horizontal pass keeps 11 fractional bits; vertical pass as in OpenCV's 8-bit path
                            const int      b0 = k.b0, b1 = k.b1;
                            const unsigned aw = (unsigned)(unsigned short)k.a.x | ((unsigned)(unsigned short)k.a.y << 16);
                            // two-way dot product: low 16 bits of aw times byte 0, high 16 bits times byte 1 (weights are 0..2048)
                            const int hb0 = (int)__dp2a_lo(aw, (unsigned)(k.p00.b | (k.p01.b << 8)), 0u);
                            const int hb1 = (int)__dp2a_lo(aw, (unsigned)(k.p10.b | (k.p11.b << 8)), 0u);
                            const int hg0 = (int)__dp2a_lo(aw, (unsigned)(k.p00.g | (k.p01.g << 8)), 0u);
                            const int hg1 = (int)__dp2a_lo(aw, (unsigned)(k.p10.g | (k.p11.g << 8)), 0u);
                            const int hr0 = (int)__dp2a_lo(aw, (unsigned)(k.p00.r | (k.p01.r << 8)), 0u);
                            const int hr1 = (int)__dp2a_lo(aw, (unsigned)(k.p10.r | (k.p11.r << 8)), 0u);
                            // vertical pass as in OpenCV's 8-bit path; with weights summing to 2048 the result stays in 0..255
                            px.b = (((b0 * (hb0 >> 4)) >> 16) + ((b1 * (hb1 >> 4)) >> 16) + 2) >> 2;
                            px.g = (((b0 * (hg0 >> 4)) >> 16) + ((b1 * (hg1 >> 4)) >> 16) + 2) >> 2;
                            px.r = (((b0 * (hr0 >> 4)) >> 16) + ((b1 * (hr1 >> 4)) >> 16) + 2) >> 2;
                        }
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
                            px = hue_rotate(px, k.x < hsv_cols, hue_tab);

                        const int xo_t = flip ? out_w - 1 - k.x : k.x;
                        const int c0   = swap_rb ? px.r : px.b;
                        const int c2   = swap_rb ? px.b : px.r;
                        unsigned char* o = tile + k.r * pitch + xo_t;
                        o[0]             = (unsigned char)c0;
                        o[plane]         = (unsigned char)px.g;
                        o[2 * plane]     = (unsigned char)c2;
                        sum0 += c0;
                        sum1 += px.g;
                        sum2 += c2;
                    };
                    // two units in flight per warp: the loads of the second overlap the arithmetic of the first.
                    // Unit u = (row, 32-pixel segment); the warp steps through its units without dividing.
                    // (nseg >= 1 here; the wrap loop is bounded by the step because each wrap removes at least 1.)
                    auto advance = [&](int& r, int& seg, int by) {
                        seg += by;
                        for (int it = 0; it < 2 * WARPS && seg >= nseg; ++it)
                        {
                            seg -= nseg;
                            ++r;
                        }
                    };
                    int ra = 0, sa = 0;
                    advance(ra, sa, warp);
                    int rb = ra, sb = sa;
                    advance(rb, sb, WARPS);
                    (void)units;
                    // an empty image (zero-filled slot) has no units at all
                    for (int guard = 0; nseg > 0 && ra < rows && guard < units; ++guard)
                    {
                        const taps ka = load_unit(ra, sa);
                        const taps kb = load_unit(rb, sb);
                        finish_unit(ka);
                        finish_unit(kb);
                        advance(ra, sa, 2 * WARPS);
                        advance(rb, sb, 2 * WARPS);
                    }
                }

                // ---- per-image channel means for contrast, exchanged across the cluster
                if (use_ctr)
                {
                    sum0 = warp_sum(sum0);
                    sum1 = warp_sum(sum1);
                    sum2 = warp_sum(sum2);
                    if (lane == 0)
                    {
                        atomicAdd(&part_sum[0], sum0);
                        atomicAdd(&part_sum[1], sum1);
                        atomicAdd(&part_sum[2], sum2);
                    }
                    cluster.sync(); // all partial sums of the record are in place (also a CTA barrier)
                    if (tid < 3)
                    {
                        unsigned long long total = 0;
                        for (int b = 0; b < bands; ++b)
                            total += *cluster.map_shared_rank(&part_sum[tid], b);
                        const double mean = (double)total / (double)((long long)out_w * out_h);
                        contrast_add[tid] = (float)((1.0 - (double)d.contrast) * mean);
                    }
                    cluster.sync(); // remote reads done before any CTA of the cluster may exit
                }
                else
                {
                    __syncthreads();
                }

                // ---- value map: contrast, lighting, conversion, standardisation
                for (int i = tid; i < 768; i += AUG_THREADS)
                {
                    const int c   = i >> 8;
                    const int cin = swap_rb ? 2 - c : c; // channel index in BGR order
                    lut[c][i & 255] = final_value<T>(i & 255, c, cin, d, lay, use_ctr, use_ctr ? contrast_add[c] : 0.f);
                }
                __syncthreads();

                // ---- store: a warp takes one (channel, row) line at a time, lanes take 16-byte chunks
                {
                    constexpr int VEC    = out_vec<T>::N;
                    const int     rows   = row_end - row0;
                    const int     chunks = (lay.slot_w + VEC - 1) / VEC;
                    T*            dst    = reinterpret_cast<T*>(d.dst);
                    const T       zero   = convert_out<T>(0);
                    for (int line = warp; line < lay.channels * rows; line += WARPS) // 1 channel: the B plane of a grey picture
                    {
                        const int  c      = (line >= rows) + (line >= 2 * rows);
                        const int  r      = line - c * rows;
                        const int  y      = row0 + r;
                        const bool row_in = y < out_h;
                        const unsigned char* src = tile + c * plane + r * pitch;
                        T*                   g0  = dst + (int64_t)c * lay.stride_c + (int64_t)y * lay.stride_y;
                        for (int chunk = lane; chunk < chunks; chunk += 32)
                        {
                            const int  x0 = chunk * VEC;
                            out_vec<T> o;
                            if (VEC == 4)
                            {
                                const uint32_t v4 = *reinterpret_cast<const uint32_t*>(src + x0);
    #pragma unroll
                                for (int k = 0; k < VEC; ++k)
                                    o.v[k] = (row_in && x0 + k < out_w) ? lut[c][(v4 >> (8 * k)) & 0xFF] : zero;
                            }
                            else
                            {
    #pragma unroll
                                for (int k = 0; k < VEC; ++k)
                                    o.v[k] = (row_in && x0 + k < out_w) ? lut[c][src[x0 + k]] : zero;
                            }
                            T* g = g0 + (int64_t)x0 * lay.stride_x;
                            if (L.vector_ok && x0 + VEC <= lay.slot_w)
                                *reinterpret_cast<int4*>(g) = *reinterpret_cast<const int4*>(o.v);
                            else
                                for (int k = 0; k < VEC && x0 + k < lay.slot_w; ++k)
                                    g[(int64_t)k * lay.stride_x] = o.v[k];
                        }
                    }
                }
        
                __syncthreads(); // the next record reuses the descriptor, the tables and the tile
            }
        }

        template <typename T>
        cudaError_t launch_typed(const aug_launch& L, int clusters, int bands, int cluster_size, size_t smem, int pix, cudaStream_t stream)
        {
            auto kern = pix == 4 ? aug_pack_kernel<T, 4> : aug_pack_kernel<T, 3>;
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess)
                return err;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim            = dim3(bands, clusters, 1);
            cfg.blockDim           = dim3(AUG_THREADS, 1, 1);
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

    // Host entry used by the C ABI: `descs_dev` is the device copy of the descriptors.
    // Returns a CUDA error; *why is set for configurations the kernel does not cover.
    cudaError_t launch_aug_pack(const aeonb_image_desc* descs_dev, int n, const aeonb_image_layout& layout, int pixel_stride,
                                bool slots_aligned, bool any_contrast, cudaStream_t stream, const char** why)
    {
        *why = nullptr;
        int bands = 1;
        while (bands < AUG_MAX_BAND && layout.slot_h / (bands * 2) >= 8)
            bands *= 2;
        aug_launch L;
        L.tile_pitch = (layout.slot_w + 15) / 16 * 16;
        auto smem_for = [&](int nb) {
            const int rows = (layout.slot_h + nb - 1) / nb;
            return (size_t)3 * rows * L.tile_pitch + (size_t)layout.slot_w * (sizeof(int2) + sizeof(short2)) + (size_t)rows * sizeof(row_tap) + 16;
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
        // measured on B200 that was slower -- 0.228 ms against 0.181 ms for 256 records -- because records differ in
        // cost and the hardware's own dispatch balances them better than a static round-robin.)
        const int clusters = n;
        switch (layout.dtype)
        {
        case AEONB_U8: return launch_typed<uint8_t>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_I8: return launch_typed<int8_t>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_I16: return launch_typed<int16_t>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_U16: return launch_typed<uint16_t>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_I32: return launch_typed<int32_t>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_F32: return launch_typed<float>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
        case AEONB_F64: return launch_typed<double>(L, clusters, bands, cluster_size, smem, pixel_stride, stream);
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
        bool any_contrast = false;
        for (int i = 0; i < n; ++i)
            any_contrast |= descs[i].contrast != 1.0f;
        cudaError_t e   = launch_aug_pack(scratch, n, *layout, pixel_stride, aligned, any_contrast, st, &why);
        if (why)
            throw error(AEONB_ERR_UNSUPPORTED, why);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("image kernel launch", e));
        return AEONB_OK;
    });
}
