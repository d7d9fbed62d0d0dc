// Whole-picture pre-passes of the image path for sm_100a.
//
// orient_kernel: the EXIF orientation turn cv::imdecode applies after decoding (a pure permutation of pixels).
//
// rotate_kernel: aeon's image::rotate (src/image.cpp:53-75), i.e.
// cv::warpAffine(src, dst, getRotationMatrix2D(centre, angle, 1), src.size(), INTER_LINEAR, BORDER_CONSTANT, 0)
// on 8-bit interleaved pictures, bit for bit; and its INTER_NEAREST form (interpolate == false), which the
// pixelmask and depthmap transformers use (src/etl_pixel_mask.cpp:71-73): the same fixed-point source coordinates
// rounded to the nearest whole pixel.
//
// OpenCV maps every destination pixel back through the inverted matrix in 10-bit fixed point -- the products are
// formed in float64 and rounded half to even per column (M0*x*1024, M3*x*1024) and per row ((M1*y+M2)*1024,
// (M4*y+M5)*1024) -- keeps 5 fractional bits, and blends the four neighbours with integer weights
// (32-fx)(32-fy)*32 ... that sum to 2^15; neighbours outside the picture count as zero.  The kernel does exactly
// that per destination pixel: the float64 products with explicit round-to-nearest multiplies (no contraction),
// __double2int_rn for the rounding, then integer arithmetic.  One thread per destination pixel, a grid-stride
// loop per record; HBM traffic is one read of the source (neighbouring threads share their taps through L1/L2)
// and one write of the destination.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>
#include <sstream>
#include <vector>

#include "context.hpp"

namespace aeonb
{
    namespace
    {
        struct rotate_job
        {
            const uint8_t* src;
            uint8_t*       dst;
            int32_t        src_pitch, src_stride, dst_pitch, dst_stride, width, height;
            int32_t        nearest; // INTER_NEAREST instead of INTER_LINEAR
            double         m[6]; // inverse map: source = m * (x, y, 1)
        };

        __global__ void __launch_bounds__(256) rotate_kernel(const rotate_job* __restrict__ jobs)
        {
            const rotate_job J      = jobs[blockIdx.y];
            const int        pixels = J.width * J.height;
            for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pixels; i += gridDim.x * blockDim.x)
            {
                const int y = i / J.width, x = i - y * J.width;
                const int adelta = __double2int_rn(__dmul_rn(__dmul_rn(J.m[0], (double)x), 1024.0));
                const int bdelta = __double2int_rn(__dmul_rn(__dmul_rn(J.m[3], (double)x), 1024.0));
                const int round  = J.nearest ? 512 : 16; // half of the last kept bit: 10 bits dropped, or 5
                const int x0     = __double2int_rn(__dmul_rn(__dadd_rn(__dmul_rn(J.m[1], (double)y), J.m[2]), 1024.0)) + round;
                const int y0     = __double2int_rn(__dmul_rn(__dadd_rn(__dmul_rn(J.m[4], (double)y), J.m[5]), 1024.0)) + round;
                if (J.nearest)
                {
                    // the source pixel the fixed-point coordinate rounds to, zero outside the picture
                    const int nx = max(-32768, min(32767, (x0 + adelta) >> 10)), ny = max(-32768, min(32767, (y0 + bdelta) >> 10));
                    const bool     in = nx >= 0 && nx < J.width && ny >= 0 && ny < J.height;
                    const uint8_t* sp = J.src + (size_t)(in ? ny : 0) * J.src_pitch + (size_t)(in ? nx : 0) * J.src_stride;
                    uint8_t*       dp = J.dst + (size_t)y * J.dst_pitch + (size_t)x * J.dst_stride;
                    dp[0] = in ? sp[0] : 0;
                    dp[1] = in ? sp[1] : 0;
                    dp[2] = in ? sp[2] : 0;
                    continue;
                }
                const int X = (x0 + adelta) >> 5, Y = (y0 + bdelta) >> 5;
                const int sx = max(-32768, min(32767, X >> 5)), sy = max(-32768, min(32767, Y >> 5)); // saturate_cast<short>
                const int fx = X & 31, fy = Y & 31;
                const int w00 = (32 - fx) * (32 - fy) * 32, w01 = fx * (32 - fy) * 32, w10 = (32 - fx) * fy * 32, w11 = fx * fy * 32;
                const bool in_x0 = sx >= 0 && sx < J.width, in_x1 = sx + 1 >= 0 && sx + 1 < J.width;
                const bool in_y0 = sy >= 0 && sy < J.height, in_y1 = sy + 1 >= 0 && sy + 1 < J.height;
                const uint8_t* r0 = J.src + (size_t)(in_y0 ? sy : 0) * J.src_pitch;
                const uint8_t* r1 = J.src + (size_t)(in_y1 ? sy + 1 : 0) * J.src_pitch;
                const int      o0 = (in_x0 ? sx : 0) * J.src_stride, o1 = (in_x1 ? sx + 1 : 0) * J.src_stride;
                uint8_t*       d  = J.dst + (size_t)y * J.dst_pitch + (size_t)x * J.dst_stride;
#pragma unroll
                for (int c = 0; c < 3; ++c)
                {
                    const int p00 = in_y0 && in_x0 ? r0[o0 + c] : 0, p01 = in_y0 && in_x1 ? r0[o1 + c] : 0;
                    const int p10 = in_y1 && in_x0 ? r1[o0 + c] : 0, p11 = in_y1 && in_x1 ? r1[o1 + c] : 0;
                    d[c] = (uint8_t)((p00 * w00 + p01 * w01 + p10 * w10 + p11 * w11 + (1 << 14)) >> 15);
                }
            }
        }
    }

    namespace
    {
        struct orient_job
        {
            const uint8_t* src;
            uint8_t*       dst;
            int32_t        src_pitch, src_stride, dst_pitch, dst_stride, width, height, orientation;
        };

        // EXIF orientation as OpenCV applies it after decoding: destination pixel (x, y) comes from source column /
        // row as below (w, h: source size; the destination is h wide and w high for the transposed cases 5..8).
        __global__ void __launch_bounds__(256) orient_kernel(const orient_job* __restrict__ jobs)
        {
            const orient_job J  = jobs[blockIdx.y];
            const int        w = J.width, h = J.height;
            const bool       swapped = J.orientation >= 5;
            const int        dw = swapped ? h : w, pixels = w * h;
            for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pixels; i += gridDim.x * blockDim.x)
            {
                const int y = i / dw, x = i - y * dw;
                int       sc, sr;
                switch (J.orientation)
                {
                case 2: sc = w - 1 - x, sr = y; break;         // mirror
                case 3: sc = w - 1 - x, sr = h - 1 - y; break; // half turn
                case 4: sc = x, sr = h - 1 - y; break;         // flip
                case 5: sc = y, sr = x; break;                 // transpose
                case 6: sc = y, sr = h - 1 - x; break;         // quarter turn clockwise
                case 7: sc = w - 1 - y, sr = h - 1 - x; break; // transverse
                case 8: sc = w - 1 - y, sr = x; break;         // quarter turn counter-clockwise
                default: sc = x, sr = y; break;
                }
                const uint8_t* s = J.src + (size_t)sr * J.src_pitch + (size_t)sc * J.src_stride;
                uint8_t*       d = J.dst + (size_t)y * J.dst_pitch + (size_t)x * J.dst_stride;
                d[0] = s[0];
                d[1] = s[1];
                d[2] = s[2];
            }
        }
    }

    // The inverse of getRotationMatrix2D(Point2i(width/2, height/2), angle, 1.0), with the operation order of
    // cv::getRotationMatrix2D and of cv::warpAffine's own inversion, in float64.
    void rotation_inverse_map(int width, int height, int angle, double m[6])
    {
        const double cx = (double)(float)(width / 2), cy = (double)(float)(height / 2);
        const double a     = angle * (3.1415926535897932384626433832795 / 180.);
        const double alpha = std::cos(a), beta = std::sin(a);
        double       M[6]  = {alpha, beta, (1 - alpha) * cx - beta * cy, -beta, alpha, beta * cx + (1 - alpha) * cy};
        double       D     = M[0] * M[4] - M[1] * M[3];
        D                  = D != 0 ? 1. / D : 0;
        const double A11 = M[4] * D, A22 = M[0] * D;
        M[0] = A11;
        M[1] *= -D;
        M[3] *= -D;
        M[4]            = A22;
        const double b1 = -M[0] * M[2] - M[1] * M[5];
        const double b2 = -M[3] * M[2] - M[4] * M[5];
        M[2]            = b1;
        M[5]            = b2;
        for (int i = 0; i < 6; ++i)
            m[i] = M[i];
    }
}

using namespace aeonb;

extern "C" int aeonb_rotate_batch(aeonb_ctx* ctx, const aeonb_rotate_desc* descs, int n)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_rotate_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        std::vector<rotate_job> jobs(n);
        int64_t                 most = 0;
        for (int i = 0; i < n; ++i)
        {
            const aeonb_rotate_desc& r = descs[i];
            std::ostringstream       ss;
            if (!r.src || !r.dst || r.width <= 0 || r.height <= 0 || r.width > 32767 || r.height > 32767)
                ss << "record " << i << ": NULL picture or size outside 1..32767";
            else if ((r.src_pixel_stride != 3 && r.src_pixel_stride != 4) || (r.dst_pixel_stride != 3 && r.dst_pixel_stride != 4))
                ss << "record " << i << ": pixel strides must be 3 or 4";
            else if (r.src_pitch < r.width * r.src_pixel_stride || r.dst_pitch < r.width * r.dst_pixel_stride)
                ss << "record " << i << ": pitch smaller than a row";
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
            rotate_job& j = jobs[i];
            j.src         = r.src;
            j.dst         = r.dst;
            j.src_pitch   = r.src_pitch;
            j.src_stride  = r.src_pixel_stride;
            j.dst_pitch   = r.dst_pitch;
            j.dst_stride  = r.dst_pixel_stride;
            j.width       = r.width;
            j.height      = r.height;
            j.nearest     = r.nearest != 0;
            rotation_inverse_map(r.width, r.height, r.angle, j.m);
            most = std::max<int64_t>(most, (int64_t)r.width * r.height);
        }
        AEONB_CUDA(cudaSetDevice(ctx->device));
        auto*      jdev = static_cast<const rotate_job*>(ctx->upload(jobs.data(), sizeof(rotate_job) * n));
        const int  per  = (int)std::min<int64_t>((most + 255) / 256, 148 * 8); // blocks per record
        const dim3 grid((unsigned)std::max(per, 1), (unsigned)n);
        launch_timer timer(ctx, AEONB_KERNEL_OTHER, 0);
        rotate_kernel<<<grid, 256, 0, ctx->stream>>>(jdev);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("rotate kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}

extern "C" int aeonb_orient_batch(aeonb_ctx* ctx, const aeonb_orient_desc* descs, int n)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_orient_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        std::vector<orient_job> jobs(n);
        int64_t                 most = 0;
        for (int i = 0; i < n; ++i)
        {
            const aeonb_orient_desc& r = descs[i];
            std::ostringstream       ss;
            const int                dw = r.orientation >= 5 ? r.height : r.width;
            if (!r.src || !r.dst || r.width <= 0 || r.height <= 0 || (int64_t)r.width * r.height > (1ll << 30))
                ss << "record " << i << ": NULL picture or bad size";
            else if (r.orientation < 1 || r.orientation > 8)
                ss << "record " << i << ": orientation must be 1..8";
            else if ((r.src_pixel_stride != 3 && r.src_pixel_stride != 4) || (r.dst_pixel_stride != 3 && r.dst_pixel_stride != 4))
                ss << "record " << i << ": pixel strides must be 3 or 4";
            else if (r.src_pitch < r.width * r.src_pixel_stride || r.dst_pitch < dw * r.dst_pixel_stride)
                ss << "record " << i << ": pitch smaller than a row";
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
            jobs[i] = orient_job{r.src, r.dst, r.src_pitch, r.src_pixel_stride, r.dst_pitch, r.dst_pixel_stride, r.width, r.height, r.orientation};
            most    = std::max<int64_t>(most, (int64_t)r.width * r.height);
        }
        AEONB_CUDA(cudaSetDevice(ctx->device));
        auto*      jdev = static_cast<const orient_job*>(ctx->upload(jobs.data(), sizeof(orient_job) * n));
        const int  per  = (int)std::min<int64_t>((most + 255) / 256, 148 * 8);
        const dim3 grid((unsigned)std::max(per, 1), (unsigned)n);
        launch_timer timer(ctx, AEONB_KERNEL_OTHER, 0);
        orient_kernel<<<grid, 256, 0, ctx->stream>>>(jdev);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("orientation kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}
