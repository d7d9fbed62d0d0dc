// Log-mel spectrogram kernel for sm_100a: framing + window + real DFT magnitude + mel filter
// bank + natural log, one launch per batch of clips.
//
// Follows aeon's specgram::wav_to_specgram and specgram_to_cepsgram (src/specgram.cpp:26-137):
//   frames = (n - L)/S + 1 (capped), sample -> float, * window, length-L DFT, bins 0..L/2,
//   magnitude; then (mag*mag / (2*(L/2))) x filter bank, natural log.  Rows past the last
//   frame of a clip are written as zeros.
//
// One warp owns one frame and never leaves registers for the transform itself: the L real
// samples are packed into L/2 complex values, L/2 = R*32, lane n holds the R values
// z[32*r + n].  An R-point DFT runs in registers, the results are twiddled, and R independent
// 32-point transforms run ACROSS the warp with shuffle butterflies.  The packed spectrum is
// unfolded into the L/2+1 real-signal bins through a small per-warp shared-memory buffer,
// which also feeds the sparse triangular mel filters (at most two filters touch a bin).
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    namespace
    {
        constexpr int SPEC_WARPS   = 8;
        constexpr int SPEC_THREADS = SPEC_WARPS * 32;
        constexpr int SPEC_MAX_R   = 10;

        struct spec_launch
        {
            const aeonb_specgram_desc* descs;
            aeonb_specgram_config      cfg;
            const float*               window;    // L floats, or nullptr
            const float2*              twiddle;   // L/2 entries of exp(-2*pi*i*k/(L/2)) followed by L/2+1 of exp(-2*pi*i*k/L)
            const int*                 filt_start; // num_filters+1 offsets into filt_bin / filt_weight
            const int*                 filt_bin;
            const float*               filt_weight;
            const float*               dct;       // num_cepstra x dct_n cosine table with the orthonormal scale, or nullptr
            int                        dct_n;     // num_filters rounded up to even
            int                        n_out;     // floats per output row
        };

        __device__ __forceinline__ float2 cmul(float2 a, float2 b)
        {
            return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
        }

        // Power row -> sparse mel filters -> log [-> first num_cepstra rows of the orthonormal DCT-II].  `cep` is scratch for
        // the log-mel vector when a DCT follows (num_filters floats, may not alias `power`).
        __device__ __forceinline__ void finish_mel(const spec_launch& P, const float* power, float* cep, float* out, int lane)
        {
            for (int j = lane; j < P.cfg.num_filters; j += 32)
            {
                float acc = 0.f;
                for (int i = P.filt_start[j]; i < P.filt_start[j + 1]; ++i)
                    acc += power[P.filt_bin[i]] * P.filt_weight[i];
                if (P.dct)
                    cep[j] = logf(acc);
                else
                    out[j] = logf(acc);
            }
            if (!P.dct)
                return;
            __syncwarp();
            for (int j = lane; j < P.cfg.num_cepstra; j += 32)
            {
                const float* row = P.dct + (size_t)j * P.dct_n;
                float        acc = 0.f;
                for (int k = 0; k < P.cfg.num_filters; ++k)
                    acc += cep[k] * __ldg(row + k);
                out[j] = acc;
            }
        }

        template <int R>
        __global__ void __launch_bounds__(SPEC_THREADS) specgram_kernel(const spec_launch P)
        {
            constexpr int H = R * 32; // complex transform length
            constexpr int L = 2 * H;  // frame length
            __shared__ float2 zbuf[SPEC_WARPS][H + 1];
            __shared__ float  pbuf[SPEC_WARPS][H + 1];

            const int lane = threadIdx.x & 31;
            const int warp = threadIdx.x >> 5;
            const aeonb_specgram_desc d = P.descs[blockIdx.y];
            const int frame = blockIdx.x * SPEC_WARPS + warp;
            if (frame >= P.cfg.max_time_steps)
                return;
            float* out = d.dst + (size_t)frame * P.n_out;
            int    frames = d.n_samples >= L ? (d.n_samples - L) / P.cfg.frame_stride + 1 : 0;
            frames        = min(frames, P.cfg.max_time_steps);
            if (frame >= frames)
            {
                for (int j = lane; j < P.n_out; j += 32)
                    out[j] = 0.f;
                return;
            }

            // ---- load + window + pack: z[m] = x[2m] + i*x[2m+1], lane holds m = 32*r + lane
            const int16_t* x = d.samples + (size_t)frame * P.cfg.frame_stride;
            float2         z[R];
#pragma unroll
            for (int r = 0; r < R; ++r)
            {
                const int m = 32 * r + lane;
                float     a = (float)x[2 * m], b = (float)x[2 * m + 1];
                if (P.window)
                {
                    a *= __ldg(P.window + 2 * m);
                    b *= __ldg(P.window + 2 * m + 1);
                }
                z[r] = make_float2(a, b);
            }

            // ---- R-point DFT over r (in registers), then twiddle by W_H^(lane*k1)
            float2 y[R];
#pragma unroll
            for (int k1 = 0; k1 < R; ++k1)
            {
                float2 acc = z[0];
#pragma unroll
                for (int r = 1; r < R; ++r)
                {
                    // W_R^(r*k1) = W_H^(32*r*k1)
                    const float2 w = __ldg(P.twiddle + ((32 * r * k1) % H));
                    const float2 t = cmul(z[r], w);
                    acc.x += t.x;
                    acc.y += t.y;
                }
                y[k1] = cmul(acc, __ldg(P.twiddle + ((lane * k1) % H)));
            }

            // ---- R independent 32-point transforms across the lanes (decimation in frequency)
#pragma unroll
            for (int half = 16; half >= 1; half >>= 1)
            {
                const bool   upper = (lane & half) != 0;
                // twiddle W_(2*half)^(lane mod half) = W_H^((lane mod half) * H/(2*half))
                const float2 w = __ldg(P.twiddle + ((lane & (half - 1)) * (H / (2 * half))));
#pragma unroll
                for (int k1 = 0; k1 < R; ++k1)
                {
                    const float ox = __shfl_xor_sync(0xffffffffu, y[k1].x, half);
                    const float oy = __shfl_xor_sync(0xffffffffu, y[k1].y, half);
                    if (upper)
                        y[k1] = cmul(make_float2(ox - y[k1].x, oy - y[k1].y), w);
                    else
                        y[k1] = make_float2(y[k1].x + ox, y[k1].y + oy);
                }
            }
            // lane now holds Z[k1 + R*k2] with k2 = bit-reversed lane
            const int k2 = __brev((unsigned)lane) >> 27;
#pragma unroll
            for (int k1 = 0; k1 < R; ++k1)
                zbuf[warp][k1 + R * k2] = y[k1];
            __syncwarp();

            // ---- unfold to the real-signal bins 0..H and take the power
            const float2* wl = P.twiddle + H; // exp(-2*pi*i*k/L)
            const float   scale = 1.0f / (float)(2 * H);
            for (int k = lane; k <= H; k += 32)
            {
                const float2 a = zbuf[warp][k == H ? 0 : k];
                const float2 b = zbuf[warp][k == 0 || k == H ? 0 : H - k];
                // even part (a + conj b)/2, odd part (a - conj b)/(2i)
                const float2 ev = make_float2(0.5f * (a.x + b.x), 0.5f * (a.y - b.y));
                const float2 od = make_float2(0.5f * (a.y + b.y), -0.5f * (a.x - b.x));
                const float2 t  = cmul(od, __ldg(wl + k));
                const float  re = ev.x + t.x, im = ev.y + t.y;
                const float  mag = sqrtf(re * re + im * im);
                if (P.cfg.num_filters > 0)
                    pbuf[warp][k] = scale * mag * mag;
                else
                    out[k] = mag;
            }
            if (P.cfg.num_filters <= 0)
                return;
            __syncwarp();

            finish_mel(P, pbuf[warp], reinterpret_cast<float*>(zbuf[warp]), out, lane);
        }

        // Any frame length: one warp per frame, lanes take the bins, each bin a direct sum over the frame with the
        // twiddles from a table of L entries (index k*n mod L kept by addition).  O(L^2) per frame instead of the
        // O(L log L) of the kernel above, but the whole spectrogram stage is small next to the HBM traffic of its
        // output, and frame lengths such as 400 (25 ms at 16 kHz) have no factor of 64.
        constexpr int SPEC_GENERIC_WARPS = 4;
        __global__ void __launch_bounds__(SPEC_GENERIC_WARPS * 32) specgram_generic_kernel(const spec_launch P)
        {
            extern __shared__ float gsm[];
            const int L = P.cfg.frame_length, H = L / 2; // bins 0..H
            float*    xs   = gsm + (size_t)(threadIdx.x >> 5) * (L + H + 1); // this warp's windowed samples, then its power row
            float*    pw   = xs + L;
            const int lane = threadIdx.x & 31;
            const aeonb_specgram_desc d = P.descs[blockIdx.y];
            const int frame = blockIdx.x * SPEC_GENERIC_WARPS + (threadIdx.x >> 5);
            if (frame >= P.cfg.max_time_steps)
                return;
            float* out = d.dst + (size_t)frame * P.n_out;
            int    frames = d.n_samples >= L ? (d.n_samples - L) / P.cfg.frame_stride + 1 : 0;
            frames        = min(frames, P.cfg.max_time_steps);
            if (frame >= frames)
            {
                for (int j = lane; j < P.n_out; j += 32)
                    out[j] = 0.f;
                return;
            }
            const int16_t* x = d.samples + (size_t)frame * P.cfg.frame_stride;
            for (int n = lane; n < L; n += 32)
                xs[n] = (float)x[n] * (P.window ? __ldg(P.window + n) : 1.f);
            __syncwarp();
            const float scale = 1.0f / (float)(2 * H);
            for (int k = lane; k <= H; k += 32)
            {
                float re = 0.f, im = 0.f;
                int   idx = 0; // k*n mod L
                for (int n = 0; n < L; ++n)
                {
                    const float2 w = __ldg(P.twiddle + idx); // exp(-2*pi*i*idx/L)
                    re += xs[n] * w.x;
                    im += xs[n] * w.y;
                    idx += k;
                    if (idx >= L)
                        idx -= L;
                }
                const float mag = sqrtf(re * re + im * im);
                if (P.cfg.num_filters > 0)
                    pw[k] = scale * mag * mag;
                else
                    out[k] = mag;
            }
            if (P.cfg.num_filters <= 0)
                return;
            __syncwarp();
            finish_mel(P, pw, xs, out, lane);
        }

        template <int R>
        cudaError_t launch_r(const spec_launch& P, int n, cudaStream_t stream)
        {
            dim3 grid((P.cfg.max_time_steps + SPEC_WARPS - 1) / SPEC_WARPS, n, 1);
            specgram_kernel<R><<<grid, SPEC_THREADS, 0, stream>>>(P);
            return cudaGetLastError();
        }
    }

    bool specgram_frame_length_supported(int frame_length)
    {
        const int r = frame_length / 64;
        return frame_length >= 64 && frame_length % 64 == 0 && r <= SPEC_MAX_R && r != 7 && r != 9;
    }

    cudaError_t launch_specgram(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg,
                                const float* window_dev, const float2* twiddle_dev, const int* filt_start_dev,
                                const int* filt_bin_dev, const float* filt_weight_dev, const float* dct_dev, int dct_n, int n_out,
                                cudaStream_t stream)
    {
        spec_launch P{descs_dev, cfg, window_dev, twiddle_dev, filt_start_dev, filt_bin_dev, filt_weight_dev, dct_dev, dct_n, n_out};
        switch (cfg.frame_length / 64)
        {
        case 1: return launch_r<1>(P, n, stream);
        case 2: return launch_r<2>(P, n, stream);
        case 3: return launch_r<3>(P, n, stream);
        case 4: return launch_r<4>(P, n, stream);
        case 5: return launch_r<5>(P, n, stream);
        case 6: return launch_r<6>(P, n, stream);
        case 8: return launch_r<8>(P, n, stream);
        case 10: return launch_r<10>(P, n, stream);
        default: return cudaErrorInvalidValue;
        }
    }

    size_t specgram_generic_smem(int frame_length) { return (size_t)SPEC_GENERIC_WARPS * (frame_length + frame_length / 2 + 1) * sizeof(float); }

    // Frame lengths the shuffle-FFT kernel does not take: `twiddle_dev` then holds frame_length entries exp(-2*pi*i*k/L).
    cudaError_t launch_specgram_generic(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg,
                                        const float* window_dev, const float2* twiddle_dev, const int* filt_start_dev,
                                        const int* filt_bin_dev, const float* filt_weight_dev, const float* dct_dev, int dct_n,
                                        int n_out, cudaStream_t stream)
    {
        spec_launch  P{descs_dev, cfg, window_dev, twiddle_dev, filt_start_dev, filt_bin_dev, filt_weight_dev, dct_dev, dct_n, n_out};
        const size_t smem = specgram_generic_smem(cfg.frame_length);
        cudaError_t  err  = cudaFuncSetAttribute(specgram_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess)
            return err;
        dim3 grid((cfg.max_time_steps + SPEC_GENERIC_WARPS - 1) / SPEC_GENERIC_WARPS, n, 1);
        specgram_generic_kernel<<<grid, SPEC_GENERIC_WARPS * 32, smem, stream>>>(P);
        return cudaGetLastError();
    }
}
