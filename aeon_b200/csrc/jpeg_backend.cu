// JPEG back-end kernel for sm_100a: dequantisation, 8x8 integer inverse DCT, chroma
// upsampling and YCbCr->BGR for a whole batch in one launch.
//
// The host has already undone the entropy coding; this kernel does everything else
// cv::imdecode does for a baseline JPEG (aeon: src/etl_image.cpp:83-99,
// src/cap_mjpeg_decoder.cpp:132-147), with the arithmetic of libjpeg's default decoder
// settings: the 13-bit-constant Loeffler-Ligtenberg-Moschytz inverse DCT with two guard
// bits between the column and row passes, triangle-filter ("fancy") chroma upsampling and
// 16-bit fixed-point colour conversion.
//
// Work decomposition: one CTA per (record, strip of two MCU rows).  The coefficient blocks the CTA needs are
// staged in shared memory with coalesced 16-byte asynchronous copies (XOR-swizzled so that the
// next step is free of bank conflicts); then ONE THREAD transforms ONE 8x8 BLOCK entirely in
// registers: eight 128-bit shared loads (the host stores blocks column-major, so a load is a
// block column), column pass, row pass (the transpose is register renaming), saturating pack,
// 8-byte stores into shared component planes.  The CTA also transforms the chroma blocks of the
// MCU rows above and below its strip (only the one sample row the triangle filter needs on either side).  A second phase upsamples, converts and writes 4 pixels per thread
// (one 128-bit store per thread for 4-byte pixels, three 32-bit stores for 3-byte pixels).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    namespace
    {
        constexpr int JPG_THREADS = 256;
        constexpr int JPG_STRIP   = 2; // MCU rows per CTA: the chroma context rows are transformed once per strip

        struct jpeg_launch
        {
            const aeonb_jpeg_desc* descs; // device
            const int2*            work;  // device: (record, mcu row) per CTA
        };

        __device__ __forceinline__ int clamp255(int v) { return min(max(v, 0), 255); }

        constexpr int CONST_BITS = 13;
        constexpr int PASS1_BITS = 2;
        constexpr int C_0_298631336 = 2446;
        constexpr int C_0_390180644 = 3196;
        constexpr int C_0_541196100 = 4433;
        constexpr int C_0_765366865 = 6270;
        constexpr int C_0_899976223 = 7373;
        constexpr int C_1_175875602 = 9633;
        constexpr int C_1_501321110 = 12299;
        constexpr int C_1_847759065 = 15137;
        constexpr int C_1_961570560 = 16069;
        constexpr int C_2_053119869 = 16819;
        constexpr int C_2_562915447 = 20995;
        constexpr int C_3_072711026 = 25172;

        // One 8-point inverse DCT (LLM factorisation); inputs x[0..7] are frequency samples,
        // outputs are descaled by `shift` with round-half-up.
        template <int SHIFT, int LEVEL>
        __device__ __forceinline__ void idct8(const int (&x)[8], int (&o)[8])
        {
            int z1 = (x[2] + x[6]) * C_0_541196100;
            int t2 = z1 - x[6] * C_1_847759065;
            int t3 = z1 + x[2] * C_0_765366865;
            int t0 = (x[0] + x[4]) << CONST_BITS;
            int t1 = (x[0] - x[4]) << CONST_BITS;
            const int e0 = t0 + t3, e3 = t0 - t3, e1 = t1 + t2, e2 = t1 - t2;

            int o0 = x[7], o1 = x[5], o2 = x[3], o3 = x[1];
            z1       = o0 + o3;
            int z2   = o1 + o2;
            int z3   = o0 + o2;
            int z4   = o1 + o3;
            const int z5 = (z3 + z4) * C_1_175875602;
            o0 *= C_0_298631336;
            o1 *= C_2_053119869;
            o2 *= C_3_072711026;
            o3 *= C_1_501321110;
            z1 = -z1 * C_0_899976223;
            z2 = -z2 * C_2_562915447;
            z3 = -z3 * C_1_961570560 + z5;
            z4 = -z4 * C_0_390180644 + z5;
            o0 += z1 + z3;
            o1 += z2 + z4;
            o2 += z2 + z3;
            o3 += z1 + z4;
            constexpr int RND = (1 << (SHIFT - 1)) + LEVEL * (1 << SHIFT); // rounding, plus an optional level shift of the result
            o[0] = (e0 + o3 + RND) >> SHIFT;
            o[7] = (e0 - o3 + RND) >> SHIFT;
            o[1] = (e1 + o2 + RND) >> SHIFT;
            o[6] = (e1 - o2 + RND) >> SHIFT;
            o[2] = (e2 + o1 + RND) >> SHIFT;
            o[5] = (e2 - o1 + RND) >> SHIFT;
            o[3] = (e3 + o0 + RND) >> SHIFT;
            o[4] = (e3 - o0 + RND) >> SHIFT;
        }

        // Four signed values saturated to 0..255 and packed little-endian into one word (two instructions).
        __device__ __forceinline__ uint32_t pack_sat_u8(int v0, int v1, int v2, int v3)
        {
            uint32_t hi, w;
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(v3), "r"(v2), "r"(0));
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(v1), "r"(v0), "r"(hi));
            return w;
        }

        // A list of block rows to transform: component, block row in the coefficient plane,
        // destination row in the shared sample plane, and which sample rows are wanted.
        struct block_row_job
        {
            int comp;
            int block_row;
            int dst_row;   // sample row in the shared plane where block row 0 would land
            int only_row;  // -1: all eight rows; else only this row of the block is stored
        };

        __device__ __forceinline__ void store_bgr4(uint8_t* dst, int pix, const int (&b)[4], const int (&g)[4], const int (&r)[4], int n)
        {
            if (pix == 4 && n == 4)
            {
                uint4 v;
                v.x = b[0] | (g[0] << 8) | (r[0] << 16);
                v.y = b[1] | (g[1] << 8) | (r[1] << 16);
                v.z = b[2] | (g[2] << 8) | (r[2] << 16);
                v.w = b[3] | (g[3] << 8) | (r[3] << 16);
                *reinterpret_cast<uint4*>(dst) = v;
            }
            else if (pix == 3 && n == 4)
            {
                uint32_t* d = reinterpret_cast<uint32_t*>(dst);
                d[0]        = b[0] | (g[0] << 8) | (r[0] << 16) | (b[1] << 24);
                d[1]        = g[1] | (r[1] << 8) | (b[2] << 16) | (g[2] << 24);
                d[2]        = r[2] | (b[3] << 8) | (g[3] << 16) | (r[3] << 24);
            }
            else
            {
                for (int k = 0; k < n; ++k)
                {
                    dst[k * pix + 0] = (uint8_t)b[k];
                    dst[k * pix + 1] = (uint8_t)g[k];
                    dst[k * pix + 2] = (uint8_t)r[k];
                    if (pix == 4)
                        dst[k * pix + 3] = 0;
                }
            }
        }

        __global__ void __launch_bounds__(JPG_THREADS, 3) jpeg_backend_kernel(const jpeg_launch L)
        {
            extern __shared__ __align__(16) unsigned char smem[];
            __shared__ aeonb_jpeg_desc d;
            __shared__ __align__(16) uint16_t quant[3][64];
            __shared__ block_row_job   jobs[JPG_STRIP * 4 + 4];
            __shared__ int             njobs;
            __shared__ int             job_first[JPG_STRIP * 4 + 5]; // first work item of each job, and the total

            const int  tid  = threadIdx.x;
            const int2 wk   = L.work[blockIdx.x];
            const int  mrow = wk.y; // first MCU row of this CTA's strip
            {
                const int* g = reinterpret_cast<const int*>(L.descs + wk.x);
                int*       s = reinterpret_cast<int*>(&d);
                for (int i = tid; i < (int)(sizeof(aeonb_jpeg_desc) / sizeof(int)); i += JPG_THREADS)
                    s[i] = g[i];
            }
            __syncthreads();
            for (int i = tid; i < d.ncomp * 64; i += JPG_THREADS)
                quant[i >> 6][i & 63] = __ldg(d.quant[i >> 6] + (i & 63));

            const int ncomp = d.ncomp;
            const int hs0 = d.hs[0], vs0 = d.vs[0];           // luma sampling == MCU size in blocks
            const int fh = ncomp == 3 ? hs0 : 1;              // horizontal / vertical chroma upsampling factors
            const int fv = ncomp == 3 ? vs0 : 1;
            const int yw = d.blocks_w[0] * 8;                 // luma plane pitch (bytes)
            const int cwp = ncomp == 3 ? d.blocks_w[1] * 8 : 0; // chroma plane pitch
            const int mcu_rows = d.blocks_h[0] / vs0;
            const int strip = min(JPG_STRIP, mcu_rows - mrow); // MCU rows handled here
            const int yrows = JPG_STRIP * vs0 * 8;             // plane capacity (rows)
            const int crows = JPG_STRIP * 8 + (fv == 2 ? 2 : 0); // chroma rows kept, incl. one halo row above/below for 2x vertical
            uint8_t*  yplane  = smem;
            uint8_t*  cbplane = yplane + yrows * yw;
            uint8_t*  crplane = cbplane + crows * cwp;
            unsigned char* coefs = smem + ((yrows * yw + 2 * crows * cwp + 127) & ~127); // staged coefficient blocks

            if (tid == 0)
            {
                // full block rows first, halo rows (one sample row wanted) last, so that warps do not mix them
                int n = 0;
                for (int v = 0; v < strip * vs0; ++v)
                    jobs[n++] = block_row_job{0, mrow * vs0 + v, v * 8, -1};
                if (ncomp == 3)
                {
                    const int halo = fv == 2 ? 1 : 0;
                    for (int c = 1; c < 3; ++c)
                        for (int m = 0; m < strip; ++m)
                            jobs[n++] = block_row_job{c, mrow + m, halo + 8 * m, -1};
                    for (int c = 1; c < 3 && halo; ++c)
                    {
                        if (mrow > 0)
                            jobs[n++] = block_row_job{c, mrow - 1, halo - 8, 7};
                        if (mrow + strip < d.blocks_h[c])
                            jobs[n++] = block_row_job{c, mrow + strip, halo + 8 * strip, 0};
                    }
                }
                int total = 0;
                for (int j = 0; j < n; ++j)
                {
                    job_first[j] = total;
                    total += d.blocks_w[jobs[j].comp];
                }
                job_first[n] = total;
                njobs        = n;
            }
            __syncthreads();

            // ---- phase 1a: stage the coefficient blocks of this CTA in shared memory with coalesced 16-byte
            //      asynchronous copies.  Chunk c (one block column) of block b lands at chunk (c ^ (b & 7)) of the
            //      block's 128 bytes, so that threads owning neighbouring blocks read different banks in phase 1b.
            const int total = job_first[njobs];
            {
                for (int i = tid; i < total * 8; i += JPG_THREADS)
                {
                    const int item = i >> 3, c = i & 7;
                    int       j    = 0;
                    while (j + 1 < njobs && item >= job_first[j + 1])
                        ++j;
                    const int      b   = item - job_first[j];
                    const int16_t* src = d.coef[jobs[j].comp] + ((size_t)jobs[j].block_row * d.blocks_w[jobs[j].comp] + b) * 64 + c * 8;
                    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(coefs + item * 128 + ((c ^ (item & 7)) << 4));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();

            // ---- phase 1b: dequantise + inverse DCT into the shared sample planes; one thread = one 8x8 block
            {
                for (int item = tid; item < total; item += JPG_THREADS)
                {
                    int j = 0;
                    while (j + 1 < njobs && item >= job_first[j + 1])
                        ++j;
                    const block_row_job job   = jobs[j];
                    const int           b     = item - job_first[j];
                    const int4*         q4    = reinterpret_cast<const int4*>(quant[job.comp]);
                    uint8_t*            plane = job.comp == 0 ? yplane : job.comp == 1 ? cbplane : crplane;
                    const int           pitch = job.comp == 0 ? yw : cwp;
                    const unsigned char* blk  = coefs + item * 128;
                    int                 ws[8][8]; // [row][column] after the column pass
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                    {
                        const int4 raw = *reinterpret_cast<const int4*>(blk + ((c ^ (item & 7)) << 4));
                        const int4 q   = q4[c];
                        int        x[8], o[8];
                        x[0] = (short)(raw.x & 0xFFFF) * (q.x & 0xFFFF);
                        x[1] = (raw.x >> 16) * (int)((unsigned)q.x >> 16);
                        x[2] = (short)(raw.y & 0xFFFF) * (q.y & 0xFFFF);
                        x[3] = (raw.y >> 16) * (int)((unsigned)q.y >> 16);
                        x[4] = (short)(raw.z & 0xFFFF) * (q.z & 0xFFFF);
                        x[5] = (raw.z >> 16) * (int)((unsigned)q.z >> 16);
                        x[6] = (short)(raw.w & 0xFFFF) * (q.w & 0xFFFF);
                        x[7] = (raw.w >> 16) * (int)((unsigned)q.w >> 16);
                        idct8<CONST_BITS - PASS1_BITS, 0>(x, o);
#pragma unroll
                        for (int r = 0; r < 8; ++r)
                            ws[r][c] = o[r];
                    }
                    uint8_t* out = plane + job.dst_row * pitch + b * 8;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                    {
                        if (job.only_row >= 0 && job.only_row != r)
                            continue;
                        int o[8];
                        // the +128 level shift rides on the rounding constant
                        idct8<CONST_BITS + PASS1_BITS + 3, 128>(ws[r], o);
                        *reinterpret_cast<uint2*>(out + r * pitch) = make_uint2(pack_sat_u8(o[0], o[1], o[2], o[3]),
                                                                                pack_sat_u8(o[4], o[5], o[6], o[7]));
                    }
                }
            }
            __syncthreads();

            // ---- phase 2: upsample, convert, store; one thread = 4 pixels of one row
            {
                const int W = d.width, H = d.height;
                const int pix   = d.dst_pixel_stride;
                const int y0    = mrow * vs0 * 8;
                const int rows  = min(strip * vs0 * 8, H - y0);
                const int quads = (W + 3) / 4;
                const int chh   = ncomp == 3 ? (H * d.vs[1] + vs0 - 1) / vs0 : 0; // real chroma rows / cols
                const int cw    = ncomp == 3 ? (W * d.hs[1] + hs0 - 1) / hs0 : 0;
                const int crow_base = mrow * 8 - (fv == 2 ? 1 : 0); // chroma plane row of shared row 0
                int       fast_cols = 0;
                if (fh == 2 && fv == 2)
                {
                    // 4:2:0 fast path: one thread = 8 x 2 output pixels (4 chroma samples of one chroma row).
                    // The last column group of a row and partial groups take the generic path below.
                    const int groups   = W >> 3;                       // full 8-pixel groups per row
                    const int interior = min(groups, (cw - 1) >> 2);   // groups whose chroma columns cx0..cx0+4 all exist
                    const int pairs    = (rows + 1) >> 1;
                    for (int i = tid; i < pairs * interior; i += JPG_THREADS)
                    {
                        const int k   = i / interior;                  // chroma row inside the MCU row
                        const int j   = i - k * interior;
                        const int x0  = j << 3, cx0 = j << 2;
                        const int cy  = mrow * 8 + k;
                        const int cr  = cy - crow_base;
                        const int up  = cy > 0 ? cr - 1 : cr;
                        const int dn  = cy + 1 < chh ? cr + 1 : cr;
                        const int lft = max(cx0 - 1, 0);
                        int       sb_t[6], sb_b[6], sr_t[6], sr_b[6];  // vertical sums for columns cx0-1 .. cx0+4
#pragma unroll
                        for (int comp = 0; comp < 2; ++comp)
                        {
                            const uint8_t* pl = comp == 0 ? cbplane : crplane;
                            int            cu[6], cm[6], cd[6];
                            const uint32_t wu = *reinterpret_cast<const uint32_t*>(pl + up * cwp + cx0);
                            const uint32_t wm = *reinterpret_cast<const uint32_t*>(pl + cr * cwp + cx0);
                            const uint32_t wd = *reinterpret_cast<const uint32_t*>(pl + dn * cwp + cx0);
                            cu[0] = pl[up * cwp + lft];
                            cm[0] = pl[cr * cwp + lft];
                            cd[0] = pl[dn * cwp + lft];
                            cu[5] = pl[up * cwp + cx0 + 4];
                            cm[5] = pl[cr * cwp + cx0 + 4];
                            cd[5] = pl[dn * cwp + cx0 + 4];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                            {
                                cu[q + 1] = (wu >> (8 * q)) & 0xFF;
                                cm[q + 1] = (wm >> (8 * q)) & 0xFF;
                                cd[q + 1] = (wd >> (8 * q)) & 0xFF;
                            }
#pragma unroll
                            for (int q = 0; q < 6; ++q)
                            {
                                const int t = 3 * cm[q];
                                if (comp == 0)
                                {
                                    sb_t[q] = t + cu[q];
                                    sb_b[q] = t + cd[q];
                                }
                                else
                                {
                                    sr_t[q] = t + cu[q];
                                    sr_b[q] = t + cd[q];
                                }
                            }
                        }
#pragma unroll
                        for (int half = 0; half < 2; ++half)
                        {
                            const int y = y0 + 2 * k + half;
                            if (y >= H)
                                break;
                            const int* sb = half ? sb_b : sb_t;
                            const int* sr = half ? sr_b : sr_t;
                            const uint2 yy = *reinterpret_cast<const uint2*>(yplane + (2 * k + half) * yw + x0);
                            uint32_t    px[8];
#pragma unroll
                            for (int p = 0; p < 8; ++p)
                            {
                                const int c  = (p >> 1) + 1;
                                const int u  = (((p & 1) ? 3 * sb[c] + sb[c + 1] + 7 : 3 * sb[c] + sb[c - 1] + 8) >> 4) - 128;
                                const int v  = (((p & 1) ? 3 * sr[c] + sr[c + 1] + 7 : 3 * sr[c] + sr[c - 1] + 8) >> 4) - 128;
                                const int yv = ((p < 4 ? yy.x : yy.y) >> (8 * (p & 3))) & 0xFF;
                                const int r  = yv + ((91881 * v + 32768) >> 16);
                                const int g  = yv + ((-22554 * u - 46802 * v + 32768) >> 16);
                                const int b  = yv + ((116130 * u + 32768) >> 16);
                                px[p]        = pack_sat_u8(b, g, r, 0);
                            }
                            uint8_t* out = d.dst + (size_t)y * d.dst_pitch + (size_t)x0 * pix;
                            if (pix == 4)
                            {
                                reinterpret_cast<uint4*>(out)[0] = make_uint4(px[0], px[1], px[2], px[3]);
                                reinterpret_cast<uint4*>(out)[1] = make_uint4(px[4], px[5], px[6], px[7]);
                            }
                            else
                            {
                                uint2* o2 = reinterpret_cast<uint2*>(out); // 24 bytes, 8-byte aligned (x0 is a multiple of 8)
                                o2[0] = make_uint2((px[0] & 0xFFFFFF) | (px[1] << 24), ((px[1] >> 8) & 0xFFFF) | (px[2] << 16));
                                o2[1] = make_uint2(((px[2] >> 16) & 0xFF) | (px[3] << 8), (px[4] & 0xFFFFFF) | (px[5] << 24));
                                o2[2] = make_uint2(((px[5] >> 8) & 0xFFFF) | (px[6] << 16), ((px[6] >> 16) & 0xFF) | (px[7] << 8));
                            }
                        }
                    }
                    fast_cols = interior << 3; // pixels [0, fast_cols) of every row are done
                }
                // generic path: one thread = 4 pixels of one row (all sampling modes, and the right edge of 4:2:0)
                const int quad0  = fast_cols >> 2;
                const int nquads = quads - quad0;
                for (int i = tid; i < rows * nquads; i += JPG_THREADS)
                {
                    const int ry = i / nquads;
                    const int x0 = (quad0 + i - ry * nquads) * 4;
                    const int y  = y0 + ry;
                    const int n  = min(4, W - x0);
                    int       b[4], g[4], r[4];
                    const uint32_t yy = *reinterpret_cast<const uint32_t*>(yplane + ry * yw + x0);
                    if (ncomp == 1)
                    {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            b[k] = g[k] = r[k] = (yy >> (8 * k)) & 0xFF;
                    }
                    else
                    {
                        int cb[4], cr[4];
                        if (fh == 1 && fv == 2)
                        {
                            // 4:4:0: libjpeg's vertical triangle filter alone (3 near + 1 far, bias 1 upper / 2 lower row)
                            const int cy   = y >> 1;
                            const int far  = ((y & 1) ? min(cy + 1, chh - 1) : max(cy - 1, 0)) - crow_base;
                            const int near = cy - crow_base, bias = (y & 1) ? 2 : 1;
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                            {
                                cb[k] = (3 * cbplane[near * cwp + x0 + k] + cbplane[far * cwp + x0 + k] + bias) >> 2;
                                cr[k] = (3 * crplane[near * cwp + x0 + k] + crplane[far * cwp + x0 + k] + bias) >> 2;
                            }
                        }
                        else if (fh == 4)
                        {
                            // 4:1:1: four pixels share one chroma sample (libjpeg replicates when the factor is not 2)
                            const int cy = y - crow_base;
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                            {
                                cb[k] = cbplane[cy * cwp + (x0 >> 2)];
                                cr[k] = crplane[cy * cwp + (x0 >> 2)];
                            }
                        }
                        else if (fh == 1)
                        {
                            const int cy = y - crow_base;
                            const uint32_t u = *reinterpret_cast<const uint32_t*>(cbplane + cy * cwp + x0);
                            const uint32_t v = *reinterpret_cast<const uint32_t*>(crplane + cy * cwp + x0);
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                            {
                                cb[k] = (u >> (8 * k)) & 0xFF;
                                cr[k] = (v >> (8 * k)) & 0xFF;
                            }
                        }
                        else
                        {
                            // chroma columns x0/2-1 .. x0/2+2 (clamped) of the near and far rows
                            const int cx0 = x0 >> 1;
                            int       col[4];
                            col[0] = max(cx0 - 1, 0);
                            col[1] = min(cx0, cw - 1);
                            col[2] = min(cx0 + 1, cw - 1);
                            col[3] = min(cx0 + 2, cw - 1);
                            int near_row, far_row;
                            if (fv == 2)
                            {
                                const int cy = y >> 1;
                                near_row     = cy;
                                far_row      = (y & 1) ? min(cy + 1, chh - 1) : max(cy - 1, 0);
                            }
                            else
                            {
                                near_row = far_row = y;
                            }
                            near_row -= crow_base;
                            far_row -= crow_base;
                            int sb[4], sr[4]; // column sums (vertical filter already applied)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                            {
                                const int nb = cbplane[near_row * cwp + col[k]], nr = crplane[near_row * cwp + col[k]];
                                if (fv == 2)
                                {
                                    sb[k] = 3 * nb + cbplane[far_row * cwp + col[k]];
                                    sr[k] = 3 * nr + crplane[far_row * cwp + col[k]];
                                }
                                else
                                {
                                    sb[k] = nb;
                                    sr[k] = nr;
                                }
                            }
                            if (fv == 2)
                            {
                                cb[0] = (3 * sb[1] + sb[0] + 8) >> 4;
                                cb[1] = (3 * sb[1] + sb[2] + 7) >> 4;
                                cb[2] = (3 * sb[2] + sb[1] + 8) >> 4;
                                cb[3] = (3 * sb[2] + sb[3] + 7) >> 4;
                                cr[0] = (3 * sr[1] + sr[0] + 8) >> 4;
                                cr[1] = (3 * sr[1] + sr[2] + 7) >> 4;
                                cr[2] = (3 * sr[2] + sr[1] + 8) >> 4;
                                cr[3] = (3 * sr[2] + sr[3] + 7) >> 4;
                            }
                            else
                            {
                                cb[0] = (3 * sb[1] + sb[0] + 1) >> 2;
                                cb[1] = (3 * sb[1] + sb[2] + 2) >> 2;
                                cb[2] = (3 * sb[2] + sb[1] + 1) >> 2;
                                cb[3] = (3 * sb[2] + sb[3] + 2) >> 2;
                                cr[0] = (3 * sr[1] + sr[0] + 1) >> 2;
                                cr[1] = (3 * sr[1] + sr[2] + 2) >> 2;
                                cr[2] = (3 * sr[2] + sr[1] + 1) >> 2;
                                cr[3] = (3 * sr[2] + sr[3] + 2) >> 2;
                            }
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                        {
                            const int yv = (yy >> (8 * k)) & 0xFF;
                            const int u = cb[k] - 128, v = cr[k] - 128;
                            r[k] = clamp255(yv + ((91881 * v + 32768) >> 16));
                            g[k] = clamp255(yv + ((-22554 * u - 46802 * v + 32768) >> 16));
                            b[k] = clamp255(yv + ((116130 * u + 32768) >> 16));
                        }
                    }
                    store_bgr4(d.dst + (size_t)y * d.dst_pitch + (size_t)x0 * pix, pix, b, g, r, n);
                }
            }
        }
    }

    cudaError_t launch_jpeg_backend(const aeonb_jpeg_desc* descs_dev, const int2* work_dev, int n_work, size_t smem,
                                    cudaStream_t stream)
    {
        if (n_work <= 0)
            return cudaSuccess;
        cudaError_t err = cudaFuncSetAttribute(jpeg_backend_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess)
            return err;
        jpeg_launch L{descs_dev, work_dev};
        jpeg_backend_kernel<<<n_work, JPG_THREADS, smem, stream>>>(L);
        return cudaGetLastError();
    }

    int jpeg_backend_strip() { return JPG_STRIP; }

    // Shared memory one CTA needs for a record.
    size_t jpeg_backend_smem(const aeonb_jpeg_desc& d)
    {
        const int yrows = JPG_STRIP * d.vs[0] * 8;
        const int fv    = d.ncomp == 3 ? d.vs[0] : 1;
        const int crows = JPG_STRIP * 8 + (fv == 2 ? 2 : 0);
        const size_t planes = (size_t)yrows * d.blocks_w[0] * 8 + (d.ncomp == 3 ? (size_t)2 * crows * d.blocks_w[1] * 8 : 0);
        const size_t blocks = (size_t)JPG_STRIP * d.vs[0] * d.blocks_w[0] +
                              (d.ncomp == 3 ? (size_t)2 * (JPG_STRIP + (fv == 2 ? 2 : 0)) * d.blocks_w[1] : 0);
        return ((planes + 127) & ~(size_t)127) + blocks * 128;
    }
}
