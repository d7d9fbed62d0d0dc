// Device-side JPEG entropy decoding for sm_100a: one warp per JPEG stream.
//
// Huffman decoding of a baseline scan without restart markers is a serial chain -- every code
// starts where the previous one ended -- so a single stream cannot be spread over threads.  A
// batch, however, holds hundreds of independent streams, and a B200 has 592 warp schedulers:
// giving every stream its own warp (one warp per CTA, so the CTAs spread over all SMs) decodes
// the whole batch in the time one stream takes, and removes the host CPU -- the end-to-end
// bottleneck of the host path -- from the per-record work.  Within a warp lane 0 walks the bit
// stream; all 32 lanes build the lookup tables, prefetch the stream into a shared-memory window
// with coalesced loads, and flush each finished 8x8 block with one coalesced 128-byte store.
//
// The decoder is the same algorithm as the host one (ITU-T T.81 F.2.2: table lookup on a 10-bit
// window with a combined run/size/value table for short AC codes, canonical-code search for long
// codes, DC prediction per component, restart handling) and produces the same column-major
// coefficient planes, optionally restricted to a rectangle of MCUs.  Every loop is bounded by the
// stream length or by the block count; a malformed stream sets the record's status word and the
// warp stops, it never spins.
#include <cuda_runtime.h>
#include <stdint.h>

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
        // segment's end, the block's index inside the MCU and the zig-zag index.  Huffman streams
        // re-synchronise: a decoder started in a wrong state soon falls into step with the true one, so
        // most guesses leave their segment in the true state.  Rounds follow in which every thread takes
        // its left neighbour's exit state as its entry state and decodes again if that entry differs from
        // the one it used before; segment 0 always starts in the true state, so after round r the first
        // r+1 exits are true, and the rounds stop as soon as nothing changes (at most one round per
        // segment).  A prefix sum over the blocks each segment completed gives every segment its first
        // block number, and a last pass decodes each segment once more from its now true entry state,
        // this time storing the coefficients.  DC values are stored as differences and summed up per
        // component in a final scan.
        constexpr int PAR_THREADS = 256;

        struct par_state
        {
            huff_table dc[2], ac[2];
            uint32_t   ent_p[PAR_THREADS], ext_p[PAR_THREADS], cnt[PAR_THREADS];
            uint16_t   ent_bk[PAR_THREADS], ext_bk[PAR_THREADS];
            uint32_t   warp_sums[3][PAR_THREADS / 32];
            uint8_t    zz[64];
            uint8_t    comp[16], bx[16], by[16]; // per block of an MCU: component and position inside the MCU
            aeonb_entropy_desc d;
            int        bpm;                      // blocks per MCU
            uint32_t   total_blocks;
            int        bad;
            uint32_t   marker_at;                // first marker byte in the raw scan (or its size)
        };

        // Bit reader over the copy without stuffed bytes; reads 32-bit words (the copy is padded with zeros).
        struct clean_reader
        {
            const uint32_t* words;
            uint64_t        acc;
            int             n;
            uint32_t        wp;

            __device__ __forceinline__ uint32_t load_be(uint32_t i) const { return __byte_perm(words[i], 0, 0x0123); } // plain load: this block wrote the copy
            __device__ __forceinline__ void     start(const uint32_t* w, uint32_t bitpos)
            {
                words = w;
                wp    = bitpos >> 5;
                acc   = (uint64_t)load_be(wp) << 32;
                ++wp;
                const int r = bitpos & 31;
                acc <<= r;
                n = 32 - r;
            }
            __device__ __forceinline__ void refill()
            {
                if (n <= 32)
                {
                    acc |= (uint64_t)load_be(wp) << (32 - n);
                    n += 32;
                    ++wp;
                }
            }
            __device__ __forceinline__ uint32_t pos() const { return wp * 32u - (uint32_t)n; }
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
            // An invalid code still consumes bits, so that a decoder in a wrong state always moves on.
            __device__ __forceinline__ int decode(const huff_table& t, int& bad)
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
                    bad = 1;
                    skip(16);
                    return 0;
                }
                skip(len);
                return t.vals[((c16 >> (16 - len)) + t.valoff[len]) & 255];
            }
        };

        // Where block `b` of MCU (mx, my) lives in the compact coefficient planes, or NULL outside the region.
        __device__ __forceinline__ int16_t* locate_block(const par_state& S, int mx, int my, int b)
        {
            const aeonb_entropy_desc& d = S.d;
            if (my < d.roi[1] || my >= d.roi[3] || mx < d.roi[0] || mx >= d.roi[2])
                return nullptr;
            const int c = S.comp[b];
            return d.coef[c] + ((size_t)((my - d.roi[1]) * d.vs[c] + S.by[b]) * ((d.roi[2] - d.roi[0]) * d.hs[c]) +
                                ((mx - d.roi[0]) * d.hs[c] + S.bx[b])) * 64;
        }

        // Decodes symbols from bit position p0 in state (b, k) until the first symbol that starts at or past pend.
        // WRITE: also stores coefficients and DC differences, `g` being the number of the block in progress.
        template <bool WRITE>
        __device__ __forceinline__ void run_segment(const par_state& S, const uint32_t* words, uint32_t p0, int b, int k, uint32_t pend,
                                                    uint32_t& p_out, int& b_out, int& k_out, uint32_t& blocks_out, uint32_t g,
                                                    int16_t* __restrict__ dcdiff, int& bad_out)
        {
            clean_reader br;
            br.start(words, p0);
            uint32_t          blocks = 0;
            int               bad    = 0;
            const int         bpm    = S.bpm;
            int               mx = 0, my = 0;
            int16_t*          out = nullptr;
            if (WRITE)
            {
                const uint32_t mcu = g / (uint32_t)bpm;
                my                 = (int)(mcu / (uint32_t)S.d.mcux);
                mx                 = (int)(mcu - (uint32_t)my * S.d.mcux);
                if (my >= S.d.roi[3])
                    pend = 0; // nothing of this segment is wanted
                else
                    out = locate_block(S, mx, my, b);
            }
            const huff_table* dct = &S.dc[S.d.dc_table[S.comp[b]] & 1];
            const huff_table* act = &S.ac[S.d.ac_table[S.comp[b]] & 1];
            while (br.pos() < pend)
            {
                br.refill();
                if (k == 0)
                {
                    int t = br.decode(*dct, bad);
                    if (t > 15)
                    {
                        bad = 1;
                        t   = 0;
                    }
                    const int diff = t ? br.receive_extend(t) : 0;
                    if (WRITE && g < S.total_blocks) // always true for a well-formed stream
                        dcdiff[g] = (int16_t)diff;
                    k = 1;
                }
                else
                {
                    const int16_t fa = act->fast_ac[br.peek(LOOK)];
                    if (fa)
                    {
                        k += (fa >> 4) & 15;
                        br.skip(fa & 15);
                        if (k > 63)
                        {
                            bad = 1;
                            k   = 64;
                        }
                        else
                        {
                            if (WRITE && out)
                                out[S.zz[k]] = (int16_t)(fa >> 8);
                            ++k;
                        }
                    }
                    else
                    {
                        const int rs = br.decode(*act, bad);
                        const int r = rs >> 4, s = rs & 15;
                        if (s == 0)
                            k = r == 15 ? k + 16 : 64;
                        else
                        {
                            k += r;
                            const int v = br.receive_extend(s);
                            if (k > 63)
                            {
                                bad = 1;
                                k   = 64;
                            }
                            else
                            {
                                if (WRITE && out)
                                    out[S.zz[k]] = (int16_t)v;
                                ++k;
                            }
                        }
                    }
                }
                if (k >= 64)
                {
                    k = 0;
                    ++blocks;
                    if (++b == bpm)
                    {
                        b = 0;
                        if (WRITE && ++mx == S.d.mcux)
                        {
                            mx = 0;
                            ++my;
                        }
                    }
                    dct = &S.dc[S.d.dc_table[S.comp[b]] & 1];
                    act = &S.ac[S.d.ac_table[S.comp[b]] & 1];
                    if (WRITE)
                    {
                        ++g;
                        if (my >= S.d.roi[3])
                            break;
                        out = locate_block(S, mx, my, b);
                    }
                }
            }
            p_out      = br.pos();
            b_out      = b;
            k_out      = k;
            blocks_out = blocks;
            bad_out    = bad;
        }

        // Exclusive prefix sum over the block's threads; `total` receives the sum.  `sums` is PAR_THREADS/32 words of shared memory.
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
            uint32_t before = 0, all = 0;
#pragma unroll
            for (int w = 0; w < PAR_THREADS / 32; ++w)
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
            extern __shared__ __align__(16) unsigned char smem_raw[];
            par_state& S    = *reinterpret_cast<par_state*>(smem_raw);
            const int  tid  = threadIdx.x;
            const int  lane = tid & 31, warp = tid >> 5;
            for (int i = tid; i < (int)(sizeof(aeonb_entropy_desc) / 4); i += PAR_THREADS)
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
            const bool     shape_ok = d.ncomp >= 1 && d.ncomp <= 3 && d.mcux > 0 && d.mcuy > 0 && d.scan && d.tables && bpm <= 16 &&
                                  d.scan_size < (1u << 28) && total_blocks64 < (1ull << 30) &&
                                  d.scratch_bytes >= clean_room + ((total_blocks64 * 2 + 15) & ~15ull);
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
                    for (int y = 0; y < d.vs[c]; ++y)
                        for (int x = 0; x < d.hs[c]; ++x, ++b)
                        {
                            S.comp[b] = (uint8_t)c;
                            S.bx[b]   = (uint8_t)x;
                            S.by[b]   = (uint8_t)y;
                        }
                S.bpm          = b;
                S.total_blocks = (uint32_t)total_blocks64;
                S.marker_at    = d.scan_size;
            }
            // ---- tables: warps 0..3 build one each
            if (warp < 4)
                build_table(warp == 0 ? S.dc[0] : warp == 1 ? S.dc[1] : warp == 2 ? S.ac[0] : S.ac[1], d.tables + warp * 272, warp >= 2,
                            lane, &S.bad);
            __syncthreads();

            // ---- copy without stuffed bytes.  Thread t owns raw bytes [c0, c1).
            uint8_t* const  clean  = static_cast<uint8_t*>(d.scratch);
            int16_t* const  dcdiff = reinterpret_cast<int16_t*>(clean + clean_room);
            const uint32_t  N      = d.scan_size;
            const uint32_t  chunk  = (N + PAR_THREADS - 1) / PAR_THREADS;
            const uint32_t  c0 = min(N, tid * chunk), c1 = min(N, c0 + chunk);
            {
                // a marker (0xFF followed by anything but 0x00) ends the entropy-coded data
                uint32_t first_marker = N;
                uint8_t  prev         = c0 > 0 ? __ldg(d.scan + c0 - 1) : 0;
                for (uint32_t i = c0; i < c1; ++i)
                {
                    const uint8_t v = __ldg(d.scan + i);
                    if (prev == 0xFF && v != 0 && first_marker == N)
                        first_marker = i - 1;
                    prev = v;
                }
                if (c1 == N && c1 > c0 && prev == 0xFF && first_marker == N)
                    first_marker = N - 1;
                if (first_marker < N)
                    atomicMin(&S.marker_at, first_marker);
            }
            __syncthreads();
            const uint32_t raw_end = S.marker_at;
            uint32_t       stuffed = 0;
            {
                uint8_t prev = c0 > 0 ? __ldg(d.scan + c0 - 1) : 0;
                for (uint32_t i = c0; i < min(c1, raw_end); ++i)
                {
                    const uint8_t v = __ldg(d.scan + i);
                    stuffed += (prev == 0xFF && v == 0);
                    prev = v;
                }
            }
            uint32_t       stuffed_total;
            const uint32_t stuffed_before = cta_exclusive_scan(stuffed, S.warp_sums[0], stuffed_total);
            const uint32_t clean_size     = raw_end - stuffed_total;
            {
                uint32_t o    = c0 - stuffed_before;
                uint8_t  prev = c0 > 0 ? __ldg(d.scan + c0 - 1) : 0;
                for (uint32_t i = c0; i < min(c1, raw_end); ++i)
                {
                    const uint8_t v = __ldg(d.scan + i);
                    if (!(prev == 0xFF && v == 0))
                        clean[o++] = v;
                    prev = v;
                }
                if (tid < 32)
                    clean[clean_size + tid] = 0; // padding the readers may run into
            }
            __syncthreads();
            const uint32_t* words = reinterpret_cast<const uint32_t*>(clean);

            // ---- segments: one per thread, a multiple of 4 bytes, at least min_segment bytes
            uint32_t seg = (clean_size + PAR_THREADS - 1) / PAR_THREADS;
            seg          = max((seg + 3u) & ~3u, (uint32_t)max(min_segment, 16) & ~3u);
            const uint32_t nseg      = (clean_size + seg - 1) / seg; // <= PAR_THREADS
            const uint32_t total_bit = clean_size * 8;
            const bool     mine      = (uint32_t)tid < nseg;
            const uint32_t pbeg = (uint32_t)tid * seg * 8, pend = min(total_bit, pbeg + seg * 8);
            int            unused_bad;
            // round 0: guessed entry states (segment 0: the true one)
            if (mine)
            {
                uint32_t p, blocks;
                int      b, k;
                run_segment<false>(S, words, pbeg, 0, 0, pend, p, b, k, blocks, 0, nullptr, unused_bad);
                S.ent_p[tid]  = pbeg;
                S.ent_bk[tid] = 0;
                S.ext_p[tid]  = p;
                S.ext_bk[tid] = (uint16_t)((b << 8) | k);
                S.cnt[tid]    = blocks;
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
                    uint32_t p, blocks;
                    int      b, k;
                    run_segment<false>(S, words, cand_p, cand_bk >> 8, cand_bk & 255, pend, p, b, k, blocks, 0, nullptr, unused_bad);
                    S.ent_p[tid]  = cand_p;
                    S.ent_bk[tid] = cand_bk;
                    S.ext_p[tid]  = p;
                    S.ext_bk[tid] = (uint16_t)((b << 8) | k);
                    S.cnt[tid]    = blocks;
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

            // ---- clear the planes, then decode once more from the true entry states, storing
            for (int c = 0; c < d.ncomp; ++c)
            {
                const size_t n16 = (size_t)(d.roi[2] - d.roi[0]) * d.hs[c] * (d.roi[3] - d.roi[1]) * d.vs[c] * 8; // 16-byte units
                uint4*       p   = reinterpret_cast<uint4*>(d.coef[c]);
                for (size_t i = tid; i < n16; i += PAR_THREADS)
                    p[i] = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
            if (mine)
            {
                uint32_t p, blocks;
                int      b, k, bad;
                run_segment<true>(S, words, S.ent_p[tid], S.ent_bk[tid] >> 8, S.ent_bk[tid] & 255, pend, p, b, k, blocks, g0, dcdiff, bad);
                if (bad)
                    S.bad = 1;
            }
            __syncthreads();

            // ---- DC: sum the differences per component in scan order.  Thread t owns MCUs [m0, m1).
            const uint32_t mchunk = (needed_mcus + PAR_THREADS - 1) / PAR_THREADS;
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
                        int16_t* out = locate_block(S, mx, my, b);
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
            int v = 384;
            if (const char* e = std::getenv("AEONB_ENTROPY_SEGMENT"))
                v = std::atoi(e);
            return v < 64 ? 64 : v > (1 << 20) ? (1 << 20) : v;
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
                                    cudaStream_t stream)
    {
        if (n <= 0)
            return cudaSuccess;
        if (any_parallel)
        {
            const size_t smem = sizeof(par_state);
            cudaError_t  err  = cudaFuncSetAttribute(jpeg_entropy_parallel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess)
                return err;
            jpeg_entropy_parallel_kernel<<<n, PAR_THREADS, smem, stream>>>(descs_dev, min_segment);
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
