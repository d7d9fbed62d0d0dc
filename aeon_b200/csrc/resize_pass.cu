// Resize pass for the interpolation methods the image kernel does not carry (sm_100a): cv::resize(crop, out, size,
// 0, 0, INTER_AREA or INTER_CUBIC) on 8-bit interleaved pictures, bit for bit with OpenCV's own code (aeon:
// image::resize with interpolation_method "AREA" / "CUBIC", src/image.cpp:93-106).
//
// INTER_CUBIC: four taps per axis, the weights of cv::interpolateCubic (A = -0.75) evaluated in float32 in OpenCV's
// order and rounded to 11-bit fixed point; integer horizontal pass; the vertical pass runs over the interleaved row
// of out_w * channels values, the first floor(n / 8) * 8 of them in float32 (OpenCV's 128-bit vector loop: value *
// (weight / 2^22) summed from the last tap to the first, rounded half to even), the rest as (sum + 2^21) >> 22;
// taps beyond the window repeat its edge.  (An OpenCV built with Intel IPP routes 8-bit cubic resizes to IPP, whose
// results differ by one level in a few percent of the pixels; the target here is OpenCV's own implementation.)
//
// INTER_LANCZOS4: eight taps per axis; cv::interpolateLanczos4 forms the weights from double-precision sines and
// cosines, so they are computed on the host with the C library OpenCV itself calls and shipped as tables (start
// index + eight 11-bit weights per destination column and row); both passes are integer, the vertical one rounded
// as (sum + 2^21) >> 22.
//
// INTER_AREA has three regimes and the kernel reproduces each per destination pixel:
//   * both axes shrink by whole factors: box sums; a 2x2 box rounds as (sum + 2) >> 2, any other box as
//     round-half-even(sum * float(1 / area));
//   * both axes shrink: float32 weights from the overlap of the destination cell with the source pixels; the
//     taps of a source row are summed first (left to right), the rows are then accumulated top to bottom, and the
//     float is rounded half to even -- the order of the float32 additions is OpenCV's;
//   * otherwise (an axis grows): the fixed-point bilinear interpolation of INTER_LINEAR, with INTER_AREA's own tap
//     positions (sx = floor(dx * scale), fx = (dx + 1) - (sx + 1) / scale folded into [0, 1)).
// Scales are 1 / (dst / src) in float64, as OpenCV computes them.  The window that is resized is the crop box of a
// canvas on which the source picture sits (zeros elsewhere), as in the image kernel.  One thread per destination
// pixel; this pass exists for parity, the common LINEAR path never runs it.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <sstream>
#include <vector>

#include "context.hpp"

namespace aeonb
{
    namespace
    {
        struct area_job
        {
            const uint8_t* src;
            uint8_t*       dst;
            int32_t        src_pitch, src_stride, src_w, src_h, canvas_x, canvas_y;
            int32_t        crop_x, crop_y, crop_w, crop_h;
            int32_t        dst_pitch, dst_stride, out_w, out_h;
            int32_t        mode; // 0: whole-factor boxes, 1: weighted cells, 2: bilinear with area taps, 3: bicubic, 4: Lanczos
            const int32_t* lanczos; // mode 4: out_w x (start, 8 weights), then out_h x (start, 8 weights), 9 ints each
            int32_t        ix, iy;
            int32_t        channels; // of the cv::Mat the reference resizes (3, or 1 for a grey picture carried as B = G = R)
            double         scale_x, scale_y, inv_x, inv_y;
        };

        // pixel (x, y) of the crop window, channel c; the canvas is zero outside the source picture
        __device__ __forceinline__ int window_pixel(const area_job& J, int x, int y, int c)
        {
            const int sx = J.crop_x + x - J.canvas_x, sy = J.crop_y + y - J.canvas_y;
            if (sx < 0 || sy < 0 || sx >= J.src_w || sy >= J.src_h)
                return 0;
            return J.src[(size_t)sy * J.src_pitch + (size_t)sx * J.src_stride + c];
        }

        struct cell_taps // the source pixels one destination cell overlaps along one axis
        {
            int   first, count;       // first source index; number of taps
            float w_first, w_mid, w_last;
            bool  has_first, has_last; // partial pixels at the two ends
        };

        __device__ __forceinline__ cell_taps area_cell(int d, double scale, int src_len)
        {
            const double f1 = (double)d * scale, f2 = f1 + scale;
            const double cell = fmin(scale, (double)src_len - f1);
            int          s1 = (int)ceil(f1), s2 = (int)floor(f2);
            s2 = min(s2, src_len - 1);
            s1 = min(s1, s2);
            cell_taps t;
            t.has_first = (double)s1 - f1 > 1e-3;
            t.has_last  = f2 - (double)s2 > 1e-3;
            t.w_first   = (float)(((double)s1 - f1) / cell);
            t.w_mid     = (float)(1.0 / cell);
            t.w_last    = (float)(fmin(fmin(f2 - (double)s2, 1.0), cell) / cell);
            t.first     = t.has_first ? s1 - 1 : s1;
            t.count     = (s2 - s1) + (t.has_first ? 1 : 0) + (t.has_last ? 1 : 0);
            return t;
        }
        __device__ __forceinline__ float tap_weight(const cell_taps& t, int k)
        {
            if (k == 0 && t.has_first)
                return t.w_first;
            if (k == t.count - 1 && t.has_last)
                return t.w_last;
            return t.w_mid;
        }

        struct linear_tap
        {
            int s, s1, w0, w1;
        };
        __device__ __forceinline__ linear_tap area_linear_tap(int d, double scale, double inv, int src_len)
        {
            int   s = (int)floor((double)d * scale);
            float f = (float)((double)(d + 1) - (double)(s + 1) * inv);
            f       = f <= 0.f ? 0.f : f - floorf(f);
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
            linear_tap t;
            t.s  = s;
            t.s1 = min(s + 1, src_len - 1);
            t.w0 = max(-32768, min(32767, __float2int_rn(__fmul_rn(__fsub_rn(1.f, f), 2048.f))));
            t.w1 = max(-32768, min(32767, __float2int_rn(__fmul_rn(f, 2048.f))));
            return t;
        }

        struct cubic_tap
        {
            int s[4], w[4];
        };
        // cv::resize's tap set for INTER_CUBIC: position as for INTER_LINEAR, weights from interpolateCubic in float32
        __device__ __forceinline__ cubic_tap cubic_taps(int d, double scale, int src_len)
        {
            float     f  = (float)(((double)d + 0.5) * scale - 0.5);
            const int s0 = (int)floorf(f);
            f            = __fsub_rn(f, (float)s0);
            const float A = -0.75f, x1 = __fadd_rn(f, 1.f), xm = __fsub_rn(1.f, f);
            float       c[4];
            c[0] = __fsub_rn(__fmul_rn(__fadd_rn(__fmul_rn(__fsub_rn(__fmul_rn(A, x1), 5.f * A), x1), 8.f * A), x1), 4.f * A);
            c[1] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(__fmul_rn(A + 2.f, f), A + 3.f), f), f), 1.f);
            c[2] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(__fmul_rn(A + 2.f, xm), A + 3.f), xm), xm), 1.f);
            c[3] = __fsub_rn(__fsub_rn(__fsub_rn(1.f, c[0]), c[1]), c[2]);
            cubic_tap t;
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                t.s[k] = max(0, min(src_len - 1, s0 - 1 + k));
                t.w[k] = max(-32768, min(32767, __float2int_rn(__fmul_rn(c[k], 2048.f))));
            }
            return t;
        }

        __global__ void __launch_bounds__(256) resize_area_kernel(const area_job* __restrict__ jobs)
        {
            const area_job J      = jobs[blockIdx.y];
            const int      pixels = J.out_w * J.out_h;
            for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pixels; i += gridDim.x * blockDim.x)
            {
                const int dy = i / J.out_w, dx = i - dy * J.out_w;
                int       out[3];
                if (J.mode == 0)
                {
                    const float scale = 1.f / (float)(J.ix * J.iy);
                    for (int c = 0; c < 3; ++c)
                    {
                        int sum = 0;
                        for (int y = 0; y < J.iy; ++y)
                            for (int x = 0; x < J.ix; ++x)
                                sum += window_pixel(J, dx * J.ix + x, dy * J.iy + y, c);
                        out[c] = (J.ix == 2 && J.iy == 2) ? (sum + 2) >> 2 : __float2int_rn(__fmul_rn((float)sum, scale));
                    }
                }
                else if (J.mode == 1)
                {
                    const cell_taps tx = area_cell(dx, J.scale_x, J.crop_w), ty = area_cell(dy, J.scale_y, J.crop_h);
                    float           acc[3] = {0.f, 0.f, 0.f};
                    for (int ky = 0; ky < ty.count; ++ky)
                    {
                        const float beta = tap_weight(ty, ky);
                        float       buf[3] = {0.f, 0.f, 0.f};
                        for (int kx = 0; kx < tx.count; ++kx)
                        {
                            const float alpha = tap_weight(tx, kx);
#pragma unroll
                            for (int c = 0; c < 3; ++c)
                                buf[c] = __fadd_rn(buf[c], __fmul_rn((float)window_pixel(J, tx.first + kx, ty.first + ky, c), alpha));
                        }
#pragma unroll
                        for (int c = 0; c < 3; ++c)
                            acc[c] = ky == 0 ? __fmul_rn(beta, buf[c]) : __fadd_rn(acc[c], __fmul_rn(beta, buf[c]));
                    }
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        out[c] = __float2int_rn(acc[c]);
                }
                else if (J.mode == 4)
                {
                    const int32_t* tx = J.lanczos + 9 * dx;
                    const int32_t* ty = J.lanczos + 9 * (J.out_w + dy);
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                    {
                        long long v = 0;
                        for (int ky = 0; ky < 8; ++ky)
                        {
                            const int sy = max(0, min(J.crop_h - 1, ty[0] - 3 + ky));
                            int       h  = 0;
#pragma unroll
                            for (int kx = 0; kx < 8; ++kx)
                                h += window_pixel(J, max(0, min(J.crop_w - 1, tx[0] - 3 + kx)), sy, c) * tx[1 + kx];
                            v += (long long)h * ty[1 + ky];
                        }
                        out[c] = (int)((v + (1ll << 21)) >> 22);
                    }
                }
                else if (J.mode == 3)
                {
                    const cubic_tap tx = cubic_taps(dx, J.scale_x, J.crop_w), ty = cubic_taps(dy, J.scale_y, J.crop_h);
                    const int       n    = J.out_w * J.channels, body = n - n % 8; // values of the row the vector loop takes
                    const float     unit = 1.f / (2048.f * 2048.f);
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                    {
                        int h[4];
#pragma unroll
                        for (int ky = 0; ky < 4; ++ky)
                        {
                            h[ky] = 0;
#pragma unroll
                            for (int kx = 0; kx < 4; ++kx)
                                h[ky] += window_pixel(J, tx.s[kx], ty.s[ky], c) * tx.w[kx];
                        }
                        const int e = dx * J.channels + (J.channels == 3 ? c : 0); // position in the interleaved row
                        if (e < body)
                        {
                            float t = __fmul_rn((float)h[3], __fmul_rn((float)ty.w[3], unit));
#pragma unroll
                            for (int ky = 2; ky >= 0; --ky)
                                t = __fadd_rn(__fmul_rn((float)h[ky], __fmul_rn((float)ty.w[ky], unit)), t);
                            out[c] = __float2int_rn(t);
                        }
                        else
                        {
                            long long v = 0;
#pragma unroll
                            for (int ky = 0; ky < 4; ++ky)
                                v += (long long)h[ky] * ty.w[ky];
                            out[c] = (int)((v + (1ll << 21)) >> 22);
                        }
                    }
                }
                else
                {
                    const linear_tap tx = area_linear_tap(dx, J.scale_x, J.inv_x, J.crop_w), ty = area_linear_tap(dy, J.scale_y, J.inv_y, J.crop_h);
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                    {
                        const int h0 = window_pixel(J, tx.s, ty.s, c) * tx.w0 + window_pixel(J, tx.s1, ty.s, c) * tx.w1;
                        const int h1 = window_pixel(J, tx.s, ty.s1, c) * tx.w0 + window_pixel(J, tx.s1, ty.s1, c) * tx.w1;
                        out[c]       = (((ty.w0 * (h0 >> 4)) >> 16) + ((ty.w1 * (h1 >> 4)) >> 16) + 2) >> 2;
                    }
                }
                uint8_t* d = J.dst + (size_t)dy * J.dst_pitch + (size_t)dx * J.dst_stride;
#pragma unroll
                for (int c = 0; c < 3; ++c)
                    d[c] = (uint8_t)max(0, min(255, out[c]));
            }
        }
    }
}

namespace aeonb
{
    namespace
    {
        // cv::interpolateLanczos4 and the tap position of cv::resize for one axis: per destination index the start
        // index and eight weights rounded to 11-bit fixed point.
        void lanczos_axis(int src_len, int dst_len, std::vector<int32_t>& out)
        {
            static const double s45      = 0.70710678118654752440084436210485;
            static const double cs[8][2] = {{1, 0}, {-s45, -s45}, {0, 1}, {s45, -s45}, {-1, 0}, {s45, s45}, {0, -1}, {-s45, s45}};
            const double        scale    = 1.0 / ((double)dst_len / (double)src_len);
            const double        pi       = 3.1415926535897932384626433832795;
            for (int d = 0; d < dst_len; ++d)
            {
                float     x = (float)(((double)d + 0.5) * scale - 0.5);
                const int s = (int)std::floor(x);
                x -= (float)s;
                float c[8];
                if (x < FLT_EPSILON)
                {
                    for (int i = 0; i < 8; ++i)
                        c[i] = 0.f;
                    c[3] = 1.f;
                }
                else
                {
                    float        sum = 0.f;
                    const double y0 = -(x + 3) * pi * 0.25, s0 = std::sin(y0), c0 = std::cos(y0);
                    for (int i = 0; i < 8; ++i)
                    {
                        const double y = -(x + 3 - i) * pi * 0.25;
                        c[i]           = (float)((cs[i][0] * s0 + cs[i][1] * c0) / (y * y));
                        sum += c[i];
                    }
                    sum = 1.f / sum;
                    for (int i = 0; i < 8; ++i)
                        c[i] *= sum;
                }
                out.push_back(s);
                for (int i = 0; i < 8; ++i)
                    out.push_back((int32_t)std::max(-32768l, std::min(32767l, std::lrint(c[i] * 2048.f))));
            }
        }
    }
}

using namespace aeonb;

extern "C" int aeonb_resize_batch(aeonb_ctx* ctx, const aeonb_resize_desc* descs, int n)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_resize_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        std::vector<area_job> jobs(n);
        std::vector<int32_t>  tables;      // Lanczos taps of every record that wants them
        std::vector<size_t>   table_first(n, 0);
        int64_t               most = 0;
        for (int i = 0; i < n; ++i)
        {
            const aeonb_resize_desc& r = descs[i];
            std::ostringstream       ss;
            if (!r.dst || r.crop_w <= 0 || r.crop_h <= 0 || r.out_w <= 0 || r.out_h <= 0 || (int64_t)r.out_w * r.out_h > (1ll << 30))
                ss << "record " << i << ": NULL destination or empty size";
            else if (r.interp != AEONB_INTERP_AREA && r.interp != AEONB_INTERP_CUBIC && r.interp != AEONB_INTERP_LANCZOS4)
                ss << "record " << i << ": this pass handles INTER_AREA, INTER_CUBIC and INTER_LANCZOS4";
            else if (r.src && ((r.src_pixel_stride != 3 && r.src_pixel_stride != 4) || r.src_pitch < r.src_w * r.src_pixel_stride))
                ss << "record " << i << ": source pixel stride must be 3 or 4 and the pitch at least a row";
            else if ((r.dst_pixel_stride != 3 && r.dst_pixel_stride != 4) || r.dst_pitch < r.out_w * r.dst_pixel_stride)
                ss << "record " << i << ": destination pixel stride must be 3 or 4 and the pitch at least a row";
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
            area_job& j  = jobs[i];
            j.src        = r.src;
            j.dst        = r.dst;
            j.src_pitch  = r.src_pitch;
            j.src_stride = r.src_pixel_stride;
            j.src_w      = r.src ? r.src_w : 0; // no source: an all-zero canvas
            j.src_h      = r.src ? r.src_h : 0;
            j.canvas_x   = r.canvas_x;
            j.canvas_y   = r.canvas_y;
            j.crop_x     = r.crop_x;
            j.crop_y     = r.crop_y;
            j.crop_w     = r.crop_w;
            j.crop_h     = r.crop_h;
            j.dst_pitch  = r.dst_pitch;
            j.dst_stride = r.dst_pixel_stride;
            j.out_w      = r.out_w;
            j.out_h      = r.out_h;
            j.channels   = r.channels == 1 ? 1 : 3;
            // cv::resize: inv_scale = dst / src, scale = 1 / inv_scale, both float64
            j.inv_x   = (double)r.out_w / (double)r.crop_w;
            j.inv_y   = (double)r.out_h / (double)r.crop_h;
            j.scale_x = 1.0 / j.inv_x;
            j.scale_y = 1.0 / j.inv_y;
            j.ix      = (int)std::lrint(j.scale_x);
            j.iy      = (int)std::lrint(j.scale_y);
            j.lanczos = nullptr;
            if (r.interp == AEONB_INTERP_LANCZOS4)
            {
                j.mode         = 4;
                table_first[i] = tables.size();
                lanczos_axis(r.crop_w, r.out_w, tables);
                lanczos_axis(r.crop_h, r.out_h, tables);
            }
            else if (r.interp == AEONB_INTERP_CUBIC)
                j.mode = 3;
            else if (j.scale_x >= 1 && j.scale_y >= 1)
                j.mode = std::fabs(j.scale_x - j.ix) < DBL_EPSILON && std::fabs(j.scale_y - j.iy) < DBL_EPSILON ? 0 : 1;
            else
                j.mode = 2;
            most = std::max<int64_t>(most, (int64_t)r.out_w * r.out_h);
        }
        AEONB_CUDA(cudaSetDevice(ctx->device));
        if (!tables.empty())
        {
            const int32_t* tdev = static_cast<const int32_t*>(ctx->upload(tables.data(), sizeof(int32_t) * tables.size()));
            for (int i = 0; i < n; ++i)
                if (jobs[i].mode == 4)
                    jobs[i].lanczos = tdev + table_first[i];
        }
        auto*      jdev = static_cast<const area_job*>(ctx->upload(jobs.data(), sizeof(area_job) * n));
        const int  per  = (int)std::min<int64_t>((most + 255) / 256, 148 * 8);
        const dim3 grid((unsigned)std::max(per, 1), (unsigned)n);
        launch_timer timer(ctx, AEONB_KERNEL_OTHER, 0);
        resize_area_kernel<<<grid, 256, 0, ctx->stream>>>(jdev);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("area resize kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}
