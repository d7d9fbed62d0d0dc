// Device-side JPEG entropy decoding for sm_100a: the Huffman stage of cv::imdecode (src/etl_image.cpp:90).
//
// Huffman decoding of a baseline scan is a serial chain -- every code starts where the previous one ended --
// and on the host it was the end-to-end bottleneck of the record path.  Two kernels take it over:
//
//  * jpeg_entropy_parallel_kernel, one thread block per stream, for scans without restart markers (the
//    common case).  The stream is cut into one segment per thread; every thread decodes its segment from a
//    guessed state, and because Huffman streams re-synchronise, most guesses leave their segment in the
//    true state.  Rounds in which each thread restarts from its left neighbour's exit state settle the rest
//    (details at the kernel).  Coefficients are stored in a last pass once every entry state is known.
//  * jpeg_entropy_kernel, one warp per stream, walks the stream serially (lane 0 decodes, all lanes build
//    tables, prefetch the stream into a shared-memory window and flush each block with one 128-byte store).
//    It takes streams with restart markers and callers that give no work area.
//
// Both produce what the host decoder produces (ITU-T T.81 F.2.2; same column-major coefficient planes,
// optionally restricted to a rectangle of MCUs), bit for bit.  Every loop is bounded by the stream length,
// the block count or the segment count; a malformed stream sets the record's status word and the block
// returns, it never spins.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdlib>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    namespace
    {
        constexpr int LOOK   = 10;
        constexpr int WINDOW = 1024; // bytes of the stream kept in shared memory (two halves of 512)

        struct huff_table
        {
            uint16_t lookup[1 << LOOK];  // (length << 8) | symbol for codes up to LOOK bits, else 0
            int16_t  fast_ac[1 << LOOK]; // (value << 8) | (run << 4) | total bits for short AC codes, else 0
            int      maxcode[18];        // exclusive upper bound of the codes of each length, left-justified to 16 bits
            int      valoff[17];
            int      first[17];          // first code of each length
            int      count[17];
            uint8_t  vals[256];
        };

        struct warp_state
        {
            huff_table    dc[2], ac[2];
            alignas(16) uint8_t window[WINDOW];
            alignas(16) int16_t block[64];
        };

        // zig-zag position -> index inside a column-major block
        __constant__ uint8_t k_zz_colmajor[64] = {
            0, 8, 1, 2, 9, 16, 24, 17, 10, 3, 4, 11, 18, 25, 32, 40, 33, 26, 19, 12, 5, 6, 13, 20, 27, 34, 41, 48, 56, 49, 42, 35,
            28, 21, 14, 7, 15, 22, 29, 36, 43, 50, 57, 58, 51, 44, 37, 30, 23, 31, 38, 45, 52, 59, 60, 53, 46, 39, 47, 54, 61, 62,
            55, 63};

        // All 32 lanes build one table from the DHT form (16 counts + up to 256 values).
        __device__ void build_table(huff_table& t, const uint8_t* __restrict__ dht, bool is_ac, int lane, int* bad)
        {
            if (lane == 0)
            {
                int code = 0, k = 0;
                for (int len = 1; len <= 16; ++len)
                {
                    const int n   = dht[len - 1];
                    t.first[len]  = code;
                    t.count[len]  = n;
                    t.valoff[len] = k - code;
                    code += n;
                    k += n;
                    if (code > (1 << len) || k > 256)
                        *bad = 1;
                    t.maxcode[len] = n ? (code << (16 - len)) : -1;
                    code <<= 1;
                }
                t.maxcode[17] = 0x7fffffff;
            }
            for (int i = lane; i < 256; i += 32)
                t.vals[i] = dht[16 + i];
            __syncwarp();
            for (int i = lane; i < (1 << LOOK); i += 32)
            {
                uint16_t e = 0;
                for (int len = 1; len <= LOOK; ++len)
                {
                    const int prefix = i >> (LOOK - len);
                    const int idx    = prefix - t.first[len];
                    if (idx >= 0 && idx < t.count[len])
                    {
                        e = (uint16_t)((len << 8) | t.vals[(prefix + t.valoff[len]) & 255]);
                        break;
                    }
                }
                t.lookup[i] = e;
                int16_t f   = 0;
                if (is_ac && e)
                {
                    const int len = e >> 8, rs = e & 255, run = rs >> 4, mag = rs & 15;
                    if (mag && len + mag <= LOOK)
                    {
                        int v = (i >> (LOOK - len - mag)) & ((1 << mag) - 1);
                        if (v < (1 << (mag - 1)))
                            v -= (1 << mag) - 1;
                        if (v >= -128 && v <= 127)
                            f = (int16_t)((v * 256) | (run << 4) | (len + mag));
                    }
                }
                t.fast_ac[i] = f;
            }
            __syncwarp();
        }

        // Bit reader of lane 0 over the shared-memory window.  `pos` counts bytes of the scan consumed.
        struct bit_reader
        {
            const uint8_t* window;
            uint32_t       pos, size; // next byte to take / scan length
            uint64_t       acc;       // bits are consumed from the top
            int            n;
            bool           at_marker;

            __device__ __forceinline__ uint8_t byte_at(uint32_t p) const { return window[p & (WINDOW - 1)]; }
            // Tops the accumulator up to at least 32 bits, byte by byte: removes stuffed zeros, stops at markers.
            __device__ __forceinline__ void refill(uint32_t limit)
            {
                if (n > 32)
                    return;
                if (pos + 4 <= limit && !at_marker)
                {
                    // four bytes at once when none of them is 0xFF (no stuffing, no marker)
                    const uint32_t* w32 = reinterpret_cast<const uint32_t*>(window);
                    const uint32_t  i   = (pos >> 2) & (WINDOW / 4 - 1);
                    const uint32_t  k   = pos & 3;
                    const uint32_t  be  = __byte_perm(w32[i], w32[(i + 1) & (WINDOW / 4 - 1)],
                                                      (k + 3) | ((k + 2) << 4) | ((k + 1) << 8) | (k << 12));
                    const uint32_t  inv = ~be;
                    if (!((inv - 0x01010101u) & ~inv & 0x80808080u))
                    {
                        acc |= (uint64_t)be << (32 - n);
                        n += 32;
                        pos += 4;
                        return;
                    }
                }
                while (n <= 32)
                {
                    uint64_t b = 0;
                    if (pos < limit && !at_marker)
                    {
                        b = byte_at(pos);
                        if (b == 0xFF)
                        {
                            const uint8_t nx = pos + 1 < size ? byte_at(pos + 1) : 0xD9;
                            if (nx == 0)
                                pos += 2;
                            else
                            {
                                b         = 0;
                                at_marker = true; // a marker: feed zero bits and stay put
                            }
                        }
                        else
                            ++pos;
                    }
                    acc |= b << (56 - n);
                    n += 8;
                }
            }
            __device__ __forceinline__ uint32_t peek(int k) const { return (uint32_t)(acc >> (64 - k)); }
            __device__ __forceinline__ void     skip(int k)
            {
                acc <<= k;
                n -= k;
            }
            __device__ __forceinline__ int receive_extend(int s)
            {
                const uint32_t v = peek(s);
                skip(s);
                return (int)v - (int)(((v >> (s - 1)) ^ 1u)) * ((1 << s) - 1);
            }
            __device__ __forceinline__ int decode(const huff_table& t, int* bad)
            {
                const uint16_t e = t.lookup[peek(LOOK)];
                if (e)
                {
                    skip(e >> 8);
                    return e & 255;
                }
                const int c16 = (int)peek(16);
                int       len = LOOK + 1;
                while (len <= 16 && (t.maxcode[len] < 0 || c16 >= t.maxcode[len]))
                    ++len;
                if (len > 16)
                {
                    *bad = 1;
                    return 0;
                }
                skip(len);
                return t.vals[((c16 >> (16 - len)) + t.valoff[len]) & 255];
            }
        };

        __global__ void __launch_bounds__(32) jpeg_entropy_kernel(const aeonb_entropy_desc* __restrict__ descs)
        {
            extern __shared__ __align__(16) unsigned char smem_raw[];
            warp_state&              S    = *reinterpret_cast<warp_state*>(smem_raw);
            const int                lane = threadIdx.x;
            __shared__ aeonb_entropy_desc d; // in shared memory: its arrays are indexed by loop variables
            __shared__ int           pred[3];
            __shared__ int           bad;
            __shared__ uint32_t      fetched; // bytes of the scan loaded into the window so far
            static_assert(sizeof(aeonb_entropy_desc) % 4 == 0, "descriptor is copied word by word");
            for (int i = lane; i < (int)(sizeof(aeonb_entropy_desc) / 4); i += 32)
                reinterpret_cast<uint32_t*>(&d)[i] = reinterpret_cast<const uint32_t*>(descs + blockIdx.x)[i];
            if (lane == 0)
            {
                bad     = 0;
                fetched = 0;
                pred[0] = pred[1] = pred[2] = 0;
            }
            __syncwarp();
            if (d.scratch && d.restart_interval == 0)
                return; // the block-parallel kernel's stream
            const bool shape_ok = d.ncomp >= 1 && d.ncomp <= 3 && d.mcux > 0 && d.mcuy > 0 && d.scan && d.tables;
            if (!shape_ok)
            {
                if (lane == 0 && d.status)
                    *d.status = 1;
                return;
            }
            build_table(S.dc[0], d.tables + 0 * 272, false, lane, &bad);
            build_table(S.dc[1], d.tables + 1 * 272, false, lane, &bad);
            build_table(S.ac[0], d.tables + 2 * 272, true, lane, &bad);
            build_table(S.ac[1], d.tables + 3 * 272, true, lane, &bad);
            for (int i = lane; i < 64; i += 32)
                S.block[i] = 0;

            // window loader: all lanes copy the next half window (512 bytes) with 16-byte loads where aligned
            auto load_half = [&](uint32_t from) {
                for (uint32_t i = lane; i < WINDOW / 2; i += 32)
                {
                    const uint32_t p = from + i;
                    S.window[p & (WINDOW - 1)] = p < d.scan_size ? __ldg(d.scan + p) : 0;
                }
                __syncwarp();
            };
            load_half(0);
            load_half(WINDOW / 2);
            if (lane == 0)
                fetched = WINDOW;
            __syncwarp();

            bit_reader br;
            br.window    = S.window;
            br.pos       = 0;
            br.size      = d.scan_size;
            br.acc       = 0;
            br.n         = 0;
            br.at_marker = false;
            int until_restart  = d.restart_interval ? d.restart_interval : -1;
            const int mx0 = max(d.roi[0], 0), my0 = max(d.roi[1], 0), mx1 = min(d.roi[2], d.mcux), my1 = min(d.roi[3], d.mcuy);

            for (int my = 0; my < my1; ++my)
            {
                for (int mx = 0; mx < d.mcux; ++mx)
                {
                    const bool keep = my >= my0 && mx >= mx0 && mx < mx1;
                    if (lane == 0)
                    {
                        if (until_restart == 0)
                        {
                            // restart marker: drop the remaining bits, step over FF Dx, reset the predictors
                            br.acc = 0;
                            br.n   = 0;
                            uint32_t guard = 0;
                            while (br.pos + 1 < br.size && guard < 64 &&
                                   !(br.byte_at(br.pos) == 0xFF && br.byte_at(br.pos + 1) >= 0xD0 && br.byte_at(br.pos + 1) <= 0xD7))
                            {
                                ++br.pos;
                                ++guard;
                            }
                            if (br.pos + 1 < br.size && guard < 64)
                                br.pos += 2;
                            else
                                bad = 1;
                            br.at_marker = false;
                            pred[0] = pred[1] = pred[2] = 0;
                            until_restart               = d.restart_interval;
                        }
                        if (until_restart > 0)
                            --until_restart;
                    }
                    for (int c = 0; c < d.ncomp; ++c)
                    {
                        const int nblk = d.hs[c] * d.vs[c];
                        for (int b = 0; b < nblk; ++b)
                        {
                            // ---- lane 0 decodes one block into shared memory
                            if (lane == 0 && !bad)
                            {
                                const huff_table& dt = S.dc[d.dc_table[c] & 1];
                                const huff_table& at = S.ac[d.ac_table[c] & 1];
                                const uint32_t    limit = min(fetched, br.size);
                                br.refill(limit);
                                const int t = br.decode(dt, &bad);
                                if (t > 15)
                                    bad = 1;
                                else if (t)
                                {
                                    br.refill(limit);
                                    pred[c] += br.receive_extend(t);
                                }
                                S.block[0] = (int16_t)pred[c];
                                int k      = 1;
                                while (k < 64 && !bad)
                                {
                                    br.refill(limit);
                                    const int16_t fa = at.fast_ac[br.peek(LOOK)];
                                    if (fa)
                                    {
                                        k += (fa >> 4) & 15;
                                        if (k > 63)
                                        {
                                            bad = 1;
                                            break;
                                        }
                                        br.skip(fa & 15);
                                        S.block[k_zz_colmajor[k++]] = (int16_t)(fa >> 8);
                                        continue;
                                    }
                                    const int rs = br.decode(at, &bad);
                                    const int r = rs >> 4, s = rs & 15;
                                    if (s == 0)
                                    {
                                        if (r != 15)
                                            break;
                                        k += 16;
                                        continue;
                                    }
                                    k += r;
                                    if (k > 63)
                                    {
                                        bad = 1;
                                        break;
                                    }
                                    S.block[k_zz_colmajor[k++]] = (int16_t)br.receive_extend(s);
                                }
                            }
                            __syncwarp();
                            // ---- all lanes: flush the block (one 128-byte store), clear it, keep the window ahead of the reader
                            if (keep)
                            {
                                const int by = b / d.hs[c], bx = b - by * d.hs[c];
                                int16_t*  out = d.coef[c] + ((size_t)((my - my0) * d.vs[c] + by) * ((mx1 - mx0) * d.hs[c]) +
                                                            ((mx - mx0) * d.hs[c] + bx)) * 64;
                                reinterpret_cast<uint32_t*>(out)[lane] = reinterpret_cast<const uint32_t*>(S.block)[lane];
                            }
                            __syncwarp();
                            reinterpret_cast<uint32_t*>(S.block)[lane] = 0;
                            // the reader may touch at most one block's worth of bytes (< 256) before the next check:
                            // refill the half of the window it has left behind
                            const uint32_t pos = __shfl_sync(0xffffffffu, br.pos, 0);
                            if (fetched < d.scan_size && pos + WINDOW / 2 >= fetched)
                            {
                                load_half(fetched);
                                if (lane == 0)
                                    fetched += WINDOW / 2;
                            }
                            __syncwarp();
                        }
                    }
                    if (bad) // uniform: `bad` lives in shared memory and every lane reads it after the barrier above
                    {
                        if (lane == 0 && d.status)
                            *d.status = 1;
                        return;
                    }
                }
            }
            if (lane == 0 && d.status)
                *d.status = 0;
        }
    

        // ------------------------------------------------------------------------------------------------
        // Block-parallel decoder for streams without restart markers.
        //
        // One thread block per stream.  The stream is first copied without its stuffed zero bytes (so bit
        // positions are plain offsets), then cut into one segment per thread.  Every thread decodes its
        // segment starting from a guessed state (block 0 of an MCU, DC coefficient next) and records the
        // state in which it leaves the segment: the bit position of the first symbol that starts past the
        // segment's end, the block's index inside the MCU and the zig-zag index.  At three evenly spaced
        // checkpoints inside the segment it also notes the state of the first symbol at or past the
        // checkpoint and the blocks completed so far.  Rounds follow in which every thread takes its left
        // neighbour's exit state as its entry state and, if that differs from the entry it used before,
        // decodes again -- but only until it arrives at a checkpoint in the state noted there, because from
        // there on it would repeat the earlier run and leave the segment in the same state.  Segment 0 always
        // starts in the true state, so after round r the first r+1 exits are true, and the rounds stop as
        // soon as nothing changes (at most one round per segment).  A prefix sum over the blocks each
        // segment completed gives every segment its first block number, and a last pass decodes each
        // segment once more from its now true entry state, this time storing the coefficients.  DC values
        // are stored as differences and summed up per component in a final scan.
        //
        // The threads of a warp sit in different segments, so the symbol loop is flat -- every pass of it
        // decodes one symbol in every lane, whatever kind (DC category, AC run/size, end of block, zero run),
        // with the block-end bookkeeping predicated.  With every warp of an SM decoding, the loop is bound by
        // trips through the L1 pipeline (a load by 32 lanes in 32 places of the stream takes one per cache
        // line), so the bits under the read position live in a 64-bit register and a lane loads one word when
        // it has used one up; the checkpoints live in shared memory, lane-major, for the same reason.
        //
        // Measured on a B200 with 256 streams of 25-85 KB (4:2:0, quality 90, crop regions stored): 0.61 ms per batch
        // with 512 threads per block and segments of at least 160 bytes (128-192 bytes within 3 %), against 20.9 ms
        // for the one-warp kernel and about 10 ms for 14 host threads.  A wrong guess falls into step with the true
        // decoder after about 10 blocks on average (the block's position inside the MCU has to match too), and not
        // at all inside flat regions, where every block looks the same: there a chain of segments is settled one
        // round per segment, which is what the slowest streams of a batch spend their time on (6.4 rounds on
        // average, 11 at most in that batch).  Tried and no faster: warming up on the tail of the left neighbour's
        // segment before the guess, a per-lane ring of stream words in shared memory topped up by asynchronous
        // copies, reading the two words under the bit position afresh for every symbol.
        constexpr int PLOOK = 12; // bits of the lookup window: AC tables
        constexpr int DLOOK = 9;  //                            DC tables (few, short codes)
        // One 16-bit lookup gives everything the symbol loop needs:
        //   bits 0-4  total bits the symbol takes (code + value bits)     bits 5-8  number of value bits (AC size / DC category)
        //   bits 9-15 advance of the zig-zag index: run + 1, 16 for ZRL, 64 for end of block, 1 for a DC category,
        //             127 for an invalid code (which still takes bits and ends the block, so that a decoder in a wrong state moves on)
        // 0 = the code is longer than the window.
        __device__ __forceinline__ uint32_t pack_symbol(int len, int sym, bool is_ac)
        {
            const int s = sym & 15, r = sym >> 4;
            const int kinc = is_ac ? (s ? r + 1 : (r == 15 ? 16 : 64)) : (r == 0 ? 1 : 127);
            return (uint32_t)(len + s) | (uint32_t)s << 5 | (uint32_t)kinc << 9;
        }
        constexpr uint32_t k_invalid_symbol = 16u | 127u << 9;

        struct par_table
        {
            uint16_t lookup[1 << PLOOK];
            int      limit[17]; // limit[len]: exclusive upper bound of the codes of length <= len, left-justified to 16 bits
            int      valoff[17];
            uint8_t  vals[256];
            int      is_ac;
            int      window; // bits of the lookup window in use
        };

        // One thread fills the canonical-code limits of a table from the DHT form (16 counts); the values are copied by the caller.
        __device__ void build_par_table_head(par_table& T, const uint8_t* __restrict__ dht, bool is_ac, int* bad)
        {
            int code = 0, k = 0;
            T.limit[0] = 0;
            T.is_ac    = is_ac;
            T.window   = is_ac ? PLOOK : DLOOK;
            for (int len = 1; len <= 16; ++len)
            {
                const int n   = dht[len - 1];
                T.valoff[len] = k - code;
                code += n;
                k += n;
                if (code > (1 << len) || k > 256)
                    *bad = 1;
                T.limit[len] = code << (16 - len);
                code <<= 1;
            }
        }
        // `nth` threads (index `t`) fill the lookup window once limits and values are in place.
        __device__ void build_par_table_body(par_table& T, int t, int nth)
        {
            const int bits = T.window;
            for (int i = t; i < (1 << bits); i += nth)
            {
                const int i16 = i << (16 - bits);
                int       len = 1;
#pragma unroll
                for (int l = 1; l < PLOOK; ++l)
                    len += l < bits && i16 >= T.limit[l];
                uint32_t e = 0;
                if (i16 < T.limit[len])
                    e = pack_symbol(len, T.vals[((i >> (bits - len)) + T.valoff[len]) & 255], T.is_ac != 0);
                T.lookup[i] = (uint16_t)e;
            }
        }
        // A code longer than the window, or an invalid one.
        __device__ __noinline__ uint32_t long_symbol(const par_table& T, uint32_t h)
        {
            const int c16 = (int)(h >> 16);
            if (c16 >= T.limit[16])
                return k_invalid_symbol;
            int len = T.window + 1;
#pragma unroll
            for (int l = DLOOK + 1; l < 16; ++l)
                len += l > T.window && c16 >= T.limit[l];
            return pack_symbol(len, T.vals[((c16 >> (16 - len)) + T.valoff[len]) & 255], T.is_ac != 0);
        }

        constexpr int PAR_THREADS = 512;  // most threads (= segments) a stream can have; the launch picks the actual number
        constexpr int NCHECK      = 3;    // checkpoints inside a segment (7 measured the same; 3 leaves room for a third kernel's CTA on the SM)

        struct par_state
        {
            par_table  tab[4]; // DC slot 0, DC slot 1, AC slot 0, AC slot 1
            uint32_t   ent_p[PAR_THREADS], ext_p[PAR_THREADS], cnt[PAR_THREADS];
            uint16_t   ent_bk[PAR_THREADS], ext_bk[PAR_THREADS];
            uint32_t   warp_sums[3][32];
            uint8_t    zz[64];
            uint8_t    comp[16], bx[16], by[16]; // per block of an MCU: component and position inside the MCU,
            const par_table* dct_of[16];         //                       its DC / AC table,
            const par_table* act_of[16];
            uint32_t   dc_look[16], ac_look[16]; //                       the shared-memory addresses of their lookup windows,
            int16_t*   blk_base[16];             //                       where its coefficients go: blk_base + (mcu row - first row) * blk_dy
            int64_t    blk_dy[16];               //                                                           + (mcu column - first column) * blk_dx
            int        blk_dx[16];
            aeonb_entropy_desc d;
            int        bpm;                      // blocks per MCU
            uint32_t   total_blocks;
            int        bad;
            uint32_t   marker_at;                // first marker byte in the raw scan (or its size)
        };

        __device__ __forceinline__ uint32_t lds_u16(uint32_t addr)
        {
            uint16_t v;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
            return v;
        }

        // Where block `b` of MCU (mx, my) lives in the compact coefficient planes, or NULL outside the region.
        __device__ __forceinline__ int16_t* block_home(const par_state& S, int mx, int my, int b)
        {
            const aeonb_entropy_desc& d = S.d;
            if (my < d.roi[1] || my >= d.roi[3] || mx < d.roi[0] || mx >= d.roi[2])
                return nullptr;
            return S.blk_base[b] + (my - d.roi[1]) * S.blk_dy[b] + (mx - d.roi[0]) * S.blk_dx[b];
        }

        struct seg_result
        {
            uint32_t p;      // exit state: bit position of the first symbol past the segment,
            int      b, k;   //             block inside the MCU, zig-zag index
            uint32_t blocks; // blocks completed
            int      bad;
            bool     merged; // the run fell into step with the remembered run: the exit state is that run's (p, b, k unset)
        };

        // Decodes symbols from bit position p in state (b, k) until the first symbol that starts at or past pend.  The copy of the
        // stream holds big-endian words, so the 32 bits under p are one funnel shift of two words.
        // WRITE: stores coefficients and DC differences, `g` being the number of the block in progress.
        // Otherwise the state at the checkpoints (first one at bit check_at, then every check_step bits) goes to chk[0],
        // chk[check_stride], ... and the blocks completed by then NCHECK rows further on; with `compare`, the run stops at the
        // first checkpoint that an earlier run over this segment (old_blocks blocks in all) passed in the same state, and the
        // block counts from there on are renumbered for this run.
        template <bool WRITE>
        __device__ __forceinline__ seg_result run_segment(const par_state& S, const uint32_t* __restrict__ words, uint32_t p, int b, int k,
                                                          uint32_t pend, uint32_t g, int16_t* __restrict__ dcdiff, uint32_t* chk,
                                                          uint32_t check_stride, uint32_t check_at, uint32_t check_step, bool compare,
                                                          uint32_t old_blocks)
        {
            seg_result R;
            R.merged         = false;
            uint32_t  blocks = 0;
            int       bad    = 0;
            const int bpm    = S.bpm;
            int       mx = 0, my = 0;
            int16_t*  out = nullptr;
            if (WRITE)
            {
                const uint32_t mcu = g / (uint32_t)bpm;
                my                 = (int)(mcu / (uint32_t)S.d.mcux);
                mx                 = (int)(mcu - (uint32_t)my * S.d.mcux);
                if (my >= S.d.roi[3])
                    pend = 0; // nothing of this segment is wanted
                else
                    out = block_home(S, mx, my, b);
            }
            uint32_t dc_look = S.dc_look[b], ac_look = S.ac_look[b];
            // checkpoints: `slot` walks down this thread's column (state; the blocks so far NCHECK rows further on); `old_key` is
            // the state an earlier run noted at the next checkpoint (no state has all bits set)
            const uint32_t rows    = NCHECK * check_stride;
            uint32_t*      slot    = chk;
            uint32_t       old_key = !WRITE && compare ? chk[0] : 0xffffffffu;
            // A checkpoint at or past the segment's end is never taken: a run can step over it with its last symbol or stop short
            // of it, so what is noted there could be left from an older run than the one whose block count goes with it.
            if (WRITE || check_at >= pend)
                check_at = 0xffffffffu;
            // The bits under p: `n` of them (33 to 64) at the top of `acc`; `next` is word `wp` of the copy, loaded a pass ahead.
            uint32_t wp   = (p >> 5) + 2;
            uint64_t acc  = ((uint64_t)words[wp - 2] << 32 | words[wp - 1]) << (p & 31);
            int      n    = 64 - (int)(p & 31);
            uint32_t next = words[wp];
            while (p < pend)
            {
                const uint32_t h = (uint32_t)(acc >> 32); // 32 valid bits; a symbol takes at most 31
                const bool     dc = k == 0;
                uint32_t       e  = lds_u16((dc ? dc_look : ac_look) + ((h >> (dc ? 32 - DLOOK : 32 - PLOOK)) << 1));
                if (!e)
                    e = long_symbol(dc ? *S.dct_of[b] : *S.act_of[b], h);
                const int tot = e & 31, kinc = e >> 9;
                if (WRITE)
                {
                    const int sz  = (e >> 5) & 15;
                    const int raw = sz ? (int)((h << (tot - sz)) >> (32 - sz)) : 0;
                    const int v   = raw - (sz && raw < ((1 << sz) >> 1) ? (1 << sz) - 1 : 0);
                    if (kinc == 127)
                        bad = 1; // invalid code, or a DC symbol that is no category
                    if (dc)
                    {
                        if (g < S.total_blocks) // always true for a well-formed stream
                            dcdiff[g] = (int16_t)v;
                    }
                    else if (sz)
                    {
                        const int kk = k + kinc - 1; // position of this coefficient
                        if (kk > 63)
                            bad = 1; // the run leaves the block
                        else if (out)
                            out[S.zz[kk]] = (int16_t)v;
                    }
                }
                p += tot;
                k += kinc;
                acc <<= tot;
                n -= tot;
                if (n <= 32)
                {
                    // only lanes that took the word ask for the next one: few trips through the L1 pipeline per pass, and a
                    // pass is longer than a hit takes, so `next` has arrived when a lane wants it
                    acc |= (uint64_t)next << (32 - n);
                    n += 32;
                    next = words[++wp];
                }
                if (k >= 64)
                {
                    k = 0;
                    ++blocks;
                    b       = b + 1 == bpm ? 0 : b + 1;
                    dc_look = S.dc_look[b];
                    ac_look = S.ac_look[b];
                    if (WRITE)
                    {
                        ++g;
                        if (b == 0 && ++mx == S.d.mcux)
                        {
                            mx = 0;
                            ++my;
                            if (my >= S.d.roi[3])
                                break;
                        }
                        out = block_home(S, mx, my, b);
                    }
                }
                if (!WRITE && p >= check_at)
                {
                    const uint32_t key = (p - check_at) << 10 | (uint32_t)b << 6 | (uint32_t)k; // p - check_at <= 30
                    if (key == old_key)
                    {
                        // in step with the earlier run: its blocks from here on are this run's too
                        const uint32_t was = slot[rows];
                        for (uint32_t* later = slot; later < chk + rows; later += check_stride)
                            later[rows] += blocks - was;
                        blocks += old_blocks - was;
                        R.merged = true;
                        break;
                    }
                    slot[0]    = key;
                    slot[rows] = blocks;
                    slot += check_stride;
                    const bool more = slot < chk + rows && check_at + check_step < pend;
                    check_at        = more ? check_at + check_step : 0xffffffffu;     // past the last checkpoint: none left
                    old_key         = more && compare ? slot[0] : 0xffffffffu;        // fetched now, wanted at the next checkpoint
                }
            }
            R.p      = p;
            R.b      = b;
            R.k      = k;
            R.blocks = blocks;
            R.bad    = bad;
            return R;
        }

        // Exclusive prefix sum over the block's threads; `total` receives the sum.  `sums` is 32 words of shared memory.
        __device__ __forceinline__ uint32_t cta_exclusive_scan(uint32_t v, uint32_t* sums, uint32_t& total)
        {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            uint32_t  incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1)
            {
                const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o)
                    incl += up;
            }
            __syncthreads(); // `sums` may still be read from an earlier scan
            if (lane == 31)
                sums[warp] = incl;
            __syncthreads();
            uint32_t  before = 0, all = 0;
            const int nwarps = (int)(blockDim.x >> 5);
            for (int w = 0; w < nwarps; ++w)
            {
                const uint32_t s = sums[w];
                if (w < warp)
                    before += s;
                all += s;
            }
            total = all;
            return before + incl - v;
        }

        __global__ void __launch_bounds__(PAR_THREADS) jpeg_entropy_parallel_kernel(const aeonb_entropy_desc* __restrict__ descs, int min_segment)
        {
            const uint32_t T = blockDim.x; // threads = most segments of this launch
            extern __shared__ __align__(16) unsigned char smem_raw[];
            par_state&      S       = *reinterpret_cast<par_state*>(smem_raw);
            uint32_t* const chk_all = reinterpret_cast<uint32_t*>(smem_raw + sizeof(par_state)); // 2 x NCHECK rows of T words
            const int       tid     = threadIdx.x;
            for (int i = tid; i < (int)(sizeof(aeonb_entropy_desc) / 4); i += T)
                reinterpret_cast<uint32_t*>(&S.d)[i] = reinterpret_cast<const uint32_t*>(descs + blockIdx.x)[i];
            if (tid < 64)
                S.zz[tid] = k_zz_colmajor[tid];
            if (tid == 0)
                S.bad = 0;
            __syncthreads();
            const aeonb_entropy_desc& d = S.d;
            if (!d.scratch || d.restart_interval != 0)
                return; // the serial kernel's stream
            int bpm = 0;
            for (int c = 0; c < 3; ++c)
                if (c < d.ncomp)
                    bpm += d.hs[c] * d.vs[c];
            const uint64_t total_blocks64 = (uint64_t)d.mcux * d.mcuy * bpm;
            const uint64_t clean_room     = ((uint64_t)d.scan_size + 32 + 15) & ~15ull;
            const uint64_t dc_room        = (total_blocks64 * 2 + 15) & ~15ull;
            const bool     shape_ok = d.ncomp >= 1 && d.ncomp <= 3 && d.mcux > 0 && d.mcuy > 0 && d.scan && d.tables && bpm <= 16 &&
                                  d.scan_size < (1u << 27) && total_blocks64 < (1ull << 30) && d.scratch_bytes >= clean_room + dc_room &&
                                  (reinterpret_cast<uintptr_t>(d.scratch) & 3) == 0;
            if (!shape_ok)
            {
                if (tid == 0 && d.status)
                    *d.status = 1;
                return;
            }
            if (tid == 0)
            {
                int b = 0;
                for (int c = 0; c < d.ncomp; ++c)
                {
                    const int64_t row_blocks = (int64_t)(d.roi[2] - d.roi[0]) * d.hs[c]; // blocks in a row of the compact plane
                    for (int y = 0; y < d.vs[c]; ++y)
                        for (int x = 0; x < d.hs[c]; ++x, ++b)
                        {
                            S.comp[b]     = (uint8_t)c;
                            S.bx[b]       = (uint8_t)x;
                            S.by[b]       = (uint8_t)y;
                            S.dct_of[b]   = &S.tab[d.dc_table[c] & 1];
                            S.act_of[b]   = &S.tab[2 + (d.ac_table[c] & 1)];
                            S.dc_look[b]  = (uint32_t)__cvta_generic_to_shared(S.dct_of[b]->lookup);
                            S.ac_look[b]  = (uint32_t)__cvta_generic_to_shared(S.act_of[b]->lookup);
                            S.blk_base[b] = d.coef[c] + (y * row_blocks + x) * 64;
                            S.blk_dy[b]   = d.vs[c] * row_blocks * 64;
                            S.blk_dx[b]   = d.hs[c] * 64;
                        }
                }
                S.bpm          = b;
                S.total_blocks = (uint32_t)total_blocks64;
                S.marker_at    = d.scan_size;
            }
            // ---- tables: a quarter of the threads builds each
            if (tid < 4)
                build_par_table_head(S.tab[tid], d.tables + tid * 272, tid >= 2, &S.bad);
            for (int i = tid; i < 4 * 256; i += T)
                S.tab[i >> 8].vals[i & 255] = d.tables[(i >> 8) * 272 + 16 + (i & 255)];
            __syncthreads();
            {
                const int quarter = (int)T / 4;
                build_par_table_body(S.tab[min(tid / quarter, 3)], tid % quarter, quarter);
            }
            __syncthreads();

            // ---- copy without stuffed bytes, as big-endian 32-bit words (byte i of the stream is byte i ^ 3 of the copy)
            uint8_t* const  clean  = static_cast<uint8_t*>(d.scratch);
            int16_t* const  dcdiff = reinterpret_cast<int16_t*>(clean + clean_room);
            const uint32_t  N      = d.scan_size;
            // The raw scan is read as 16-byte vectors from the aligned address below it; `lead` bytes precede it there.
            const uint32_t     lead = (uint32_t)(reinterpret_cast<uintptr_t>(d.scan) & 15);
            const uint4* const vec  = reinterpret_cast<const uint4*>(d.scan - lead);
            const uint32_t     nv   = (lead + N + 15) >> 4;
            // For vector i: bit b of `stuffed` = byte b is a zero that follows 0xFF, of `marker` = byte b is non-zero and
            // follows 0xFF; only bytes at stream offsets [0, limit) count, and the byte before the stream is not 0xFF.
            auto classify = [&](uint32_t i, uint32_t limit, uint32_t (&w)[4], uint32_t& valid, uint32_t& stuffed, uint32_t& marker) {
                const uint4 x = __ldg(vec + i);
                w[0] = x.x, w[1] = x.y, w[2] = x.z, w[3] = x.w;
                uint32_t prev = i > 0 ? (uint32_t)__ldg(reinterpret_cast<const uint8_t*>(vec) + 16 * i - 1) : 0;
                valid = stuffed = marker = 0;
                // Nearly every vector lies inside the stream and has no 0xFF in front of any of its bytes: all 16 are kept.
                const bool inside = 16 * i >= lead && 16 * i + 16 - lead <= limit && 16 * i != lead;
                const bool no_ff  = prev != 0xFF && !__vcmpeq4(w[0], 0xFFFFFFFFu) && !__vcmpeq4(w[1], 0xFFFFFFFFu) &&
                                   !__vcmpeq4(w[2], 0xFFFFFFFFu) && !(__vcmpeq4(w[3], 0xFFFFFFFFu) & 0x00FFFFFFu);
                if (inside && no_ff)
                {
                    valid = 0xFFFF;
                    return;
                }
#pragma unroll
                for (int b = 0; b < 16; ++b)
                {
                    const uint32_t v   = (w[b >> 2] >> (8 * (b & 3))) & 255;
                    const uint32_t pos = 16 * i + b; // offset from the aligned address
                    if (pos == lead)
                        prev = 0;
                    const bool in = pos >= lead && pos - lead < limit;
                    valid |= (uint32_t)in << b;
                    stuffed |= (uint32_t)(in && prev == 0xFF && v == 0) << b;
                    marker |= (uint32_t)(in && prev == 0xFF && v != 0) << b;
                    prev = v;
                }
            };
            {
                // a marker (0xFF followed by anything but 0x00, or 0xFF as the last byte) ends the entropy-coded data
                uint32_t first_marker = N;
                for (uint32_t i = tid; i < nv; i += T)
                {
                    uint32_t w[4], valid, stuffed, marker;
                    classify(i, N, w, valid, stuffed, marker);
                    if (marker)
                        first_marker = min(first_marker, 16 * i + (uint32_t)__ffs(marker) - 1 - lead - 1); // the 0xFF before it
                }
                if (tid == 0 && N > 0 && __ldg(d.scan + N - 1) == 0xFF)
                    first_marker = min(first_marker, N - 1);
                if (first_marker < N)
                    atomicMin(&S.marker_at, first_marker);
            }
            __syncthreads();
            const uint32_t raw_end    = S.marker_at;
            uint32_t       clean_size = 0; // bytes written so far (the same in every thread)
            for (uint32_t tile = 0; tile < nv; tile += T)
            {
                const uint32_t i = tile + tid;
                uint32_t       w[4] = {0, 0, 0, 0}, keep = 0;
                if (i < nv)
                {
                    uint32_t valid, stuffed, marker;
                    classify(i, raw_end, w, valid, stuffed, marker);
                    keep = valid & ~stuffed;
                }
                uint32_t       tile_total;
                uint32_t       o = clean_size + cta_exclusive_scan((uint32_t)__popc(keep), S.warp_sums[0], tile_total);
#pragma unroll
                for (int b = 0; b < 16; ++b)
                    if (keep >> b & 1)
                        clean[o++ ^ 3] = (uint8_t)(w[b >> 2] >> (8 * (b & 3)));
                clean_size += tile_total;
            }
            {
                if (tid < 32)
                    clean[(clean_size + tid) ^ 3] = 0; // padding the readers may run into
            }
            __syncthreads();
            const uint32_t* words = reinterpret_cast<const uint32_t*>(clean);

            // ---- clear the coefficient planes now: the stores drain while the segments are being decoded, and the
            // barriers between here and the storing pass order them before that pass's stores
            for (int c = 0; c < d.ncomp; ++c)
            {
                const size_t n16 = (size_t)(d.roi[2] - d.roi[0]) * d.hs[c] * (d.roi[3] - d.roi[1]) * d.vs[c] * 8; // 16-byte units
                uint4*       p   = reinterpret_cast<uint4*>(d.coef[c]);
                for (size_t i = tid; i < n16; i += T)
                    p[i] = make_uint4(0, 0, 0, 0);
            }
            // ---- segments: one per thread, a multiple of 4 bytes, at least min_segment bytes
            uint32_t seg = (clean_size + T - 1) / T;
            seg          = max((seg + 3u) & ~3u, (uint32_t)max(min_segment, 64) & ~3u);
            const uint32_t nseg      = (clean_size + seg - 1) / seg; // <= T
            const uint32_t total_bit = clean_size * 8;
            const bool     mine      = (uint32_t)tid < nseg;
            const uint32_t pbeg = (uint32_t)tid * seg * 8, pend = min(total_bit, pbeg + seg * 8);
            // checkpoints of this thread's segment, evenly spaced (at least 64 bits apart; a symbol is shorter, so it passes at most one)
            const uint32_t  step       = seg * 8 / (NCHECK + 1); // bits between checkpoints (seg is a multiple of 4 bytes)
            uint32_t* const chk        = chk_all + tid;
            uint32_t        run_blocks = 0; // blocks of this thread's latest run
            // first decoding pass: guessed entry states (segment 0: the true one)
            if (mine)
            {
                const seg_result r = run_segment<false>(S, words, pbeg, 0, 0, pend, 0, nullptr, chk, T, pbeg + step, step, false, 0);
                S.ent_p[tid]  = pbeg;
                S.ent_bk[tid] = 0;
                S.ext_p[tid]  = r.p;
                S.ext_bk[tid] = (uint16_t)((r.b << 8) | r.k);
                S.cnt[tid]    = r.blocks;
                run_blocks    = r.blocks;
            }
            else
                S.cnt[tid] = 0;
            __syncthreads();
            for (uint32_t round = 1; round < nseg; ++round)
            {
                uint32_t cand_p  = 0;
                uint16_t cand_bk = 0;
                bool     redo    = false;
                if (mine && tid > 0)
                {
                    cand_p  = S.ext_p[tid - 1];
                    cand_bk = S.ext_bk[tid - 1];
                    redo    = cand_p != S.ent_p[tid] || cand_bk != S.ent_bk[tid];
                }
                __syncthreads(); // every candidate has been read before any exit state changes
                if (redo)
                {
                    const seg_result r =
                        run_segment<false>(S, words, cand_p, cand_bk >> 8, cand_bk & 255, pend, 0, nullptr, chk, T, pbeg + step, step, true, run_blocks);
                    S.ent_p[tid]  = cand_p;
                    S.ent_bk[tid] = cand_bk;
                    S.cnt[tid]    = r.blocks;
                    run_blocks    = r.blocks;
                    if (!r.merged)
                    {
                        S.ext_p[tid]  = r.p;
                        S.ext_bk[tid] = (uint16_t)((r.b << 8) | r.k);
                    }
                }
                if (!__syncthreads_or(redo))
                    break;
            }

            // ---- first block number of every segment
            uint32_t       counted;
            const uint32_t g0            = cta_exclusive_scan(S.cnt[tid], S.warp_sums[0], counted);
            const uint32_t needed_mcus   = (uint32_t)min(d.roi[3], d.mcuy) * d.mcux;
            const uint32_t needed_blocks = needed_mcus * bpm;
            if (tid == 0 && counted < needed_blocks)
                S.bad = 1;

            // ---- decode once more from the true entry states, storing (the planes were cleared above).  The checkpoints now
            // describe every segment's final run, so each segment falls into NCHECK + 1 pieces with known entry states and block
            // numbers, and the pieces -- not the segments -- are dealt out to the threads: streams with fewer segments than
            // threads keep every warp busy, and neighbouring lanes work on neighbouring pieces.
            S.ext_p[tid] = g0; // the exit states have served
            __syncthreads();
            for (uint32_t q = tid; q < nseg * (NCHECK + 1); q += T)
            {
                const uint32_t t = q / (NCHECK + 1), piece = q % (NCHECK + 1);
                const uint32_t seg_beg = t * seg * 8, seg_end = min(total_bit, seg_beg + seg * 8);
                const uint32_t at = seg_beg + piece * step; // the checkpoint this piece starts from
                if (at >= seg_end)
                    continue;
                uint32_t p0 = S.ent_p[t], bk = S.ent_bk[t], before = 0;
                if (piece > 0)
                {
                    const uint32_t key = chk_all[(piece - 1) * T + t];
                    p0                 = at + (key >> 10);
                    bk                 = (key >> 6 & 15) << 8 | (key & 63);
                    before             = chk_all[(NCHECK + piece - 1) * T + t];
                }
                const seg_result r = run_segment<true>(S, words, p0, bk >> 8, bk & 255, min(seg_end, at + step), S.ext_p[t] + before, dcdiff,
                                                       nullptr, 0, 0, 0, false, 0);
                if (r.bad)
                    S.bad = 1;
            }
            __syncthreads();

            // ---- DC: sum the differences per component in scan order.  Thread t owns MCUs [m0, m1).
            const uint32_t mchunk = (needed_mcus + T - 1) / T;
            const uint32_t m0 = min(needed_mcus, tid * mchunk), m1 = min(needed_mcus, m0 + mchunk);
            int            sum[3] = {0, 0, 0};
            for (uint32_t m = m0; m < m1; ++m)
                for (int b = 0; b < bpm; ++b)
                {
                    const int v = dcdiff[(size_t)m * bpm + b];
                    const int c = S.comp[b];
                    sum[0] += c == 0 ? v : 0;
                    sum[1] += c == 1 ? v : 0;
                    sum[2] += c == 2 ? v : 0;
                }
            int pred[3];
#pragma unroll
            for (int c = 0; c < 3; ++c)
            {
                uint32_t total;
                pred[c] = (int)cta_exclusive_scan((uint32_t)sum[c], S.warp_sums[c], total);
            }
            if (m0 < m1)
            {
                int my = (int)(m0 / (uint32_t)d.mcux), mx = (int)(m0 - (uint32_t)my * d.mcux);
                for (uint32_t m = m0; m < m1; ++m)
                {
                    for (int b = 0; b < bpm; ++b)
                    {
                        const int v = dcdiff[(size_t)m * bpm + b];
                        const int c = S.comp[b];
                        int       now;
                        if (c == 0)
                            now = pred[0] += v;
                        else if (c == 1)
                            now = pred[1] += v;
                        else
                            now = pred[2] += v;
                        int16_t* out = block_home(S, mx, my, b);
                        if (out)
                            out[0] = (int16_t)now;
                    }
                    if (++mx == d.mcux)
                    {
                        mx = 0;
                        ++my;
                    }
                }
            }
            __syncthreads();
            if (tid == 0 && d.status)
                *d.status = S.bad ? 1 : 0;
        }
    }

    int jpeg_entropy_min_segment()
    {
        static const int value = [] {
            int v = 160;
            if (const char* e = std::getenv("AEONB_ENTROPY_SEGMENT"))
                v = std::atoi(e);
            return v < 64 ? 64 : v > (1 << 20) ? (1 << 20) : v;
        }();
        return value;
    }

    int jpeg_entropy_threads()
    {
        static const int value = [] {
            int v = 512;
            if (const char* e = std::getenv("AEONB_ENTROPY_THREADS"))
                v = std::atoi(e);
            v = v < 64 ? 64 : v > PAR_THREADS ? PAR_THREADS : v;
            return v & ~31;
        }();
        return value;
    }

    int64_t jpeg_entropy_scratch_bytes(const aeonb_entropy_desc& d)
    {
        int64_t bpm = 0;
        for (int c = 0; c < d.ncomp && c < 3; ++c)
            bpm += (int64_t)d.hs[c] * d.vs[c];
        const int64_t blocks = (int64_t)d.mcux * d.mcuy * bpm;
        return (((int64_t)d.scan_size + 32 + 15) & ~15ll) + ((blocks * 2 + 15) & ~15ll);
    }

    cudaError_t launch_jpeg_entropy(const aeonb_entropy_desc* descs_dev, int n, bool any_parallel, bool any_serial, int min_segment,
                                    int threads, cudaStream_t stream)
    {
        if (n <= 0)
            return cudaSuccess;
        if (any_parallel)
        {
            threads           = std::min(std::max(threads, 64), jpeg_entropy_threads()) & ~31;
            const size_t smem = sizeof(par_state) + (size_t)2 * NCHECK * threads * sizeof(uint32_t);
            cudaError_t  err  = cudaFuncSetAttribute(jpeg_entropy_parallel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess)
                return err;
            jpeg_entropy_parallel_kernel<<<n, threads, smem, stream>>>(descs_dev, min_segment);
            err = cudaGetLastError();
            if (err != cudaSuccess)
                return err;
        }
        if (any_serial)
        {
            const size_t smem = sizeof(warp_state);
            cudaError_t  err  = cudaFuncSetAttribute(jpeg_entropy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess)
                return err;
            jpeg_entropy_kernel<<<n, 32, smem, stream>>>(descs_dev);
            return cudaGetLastError();
        }
        return cudaSuccess;
    }
}
