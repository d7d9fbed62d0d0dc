#include "jpeg_host.hpp"

#include <algorithm>
#include <cstring>
#include <vector>

#include "../context.hpp"

namespace aeonb
{
    namespace
    {
        const char* const k_bad_image = "Decoding image failed due to invalid data in the image file.";

        [[noreturn]] void bad(const char* detail)
        {
            throw error(AEONB_ERR_DECODE, std::string(k_bad_image) + " (" + detail + ")");
        }

        // zig-zag position -> natural (row-major) index, ITU-T T.81 figure A.6
        const uint8_t k_zigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                                      41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                                      30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

        // zig-zag position -> index inside a column-major block
        struct zz_t
        {
            uint8_t v[64];
            zz_t()
            {
                for (int i = 0; i < 64; ++i)
                    v[i] = static_cast<uint8_t>(((k_zigzag[i] & 7) << 3) | (k_zigzag[i] >> 3));
            }
        };
        const zz_t k_zz_colmajor;

        // ITU-T T.81 Annex K.3 typical tables (used when a stream carries no DHT, as MJPEG frames may).
        const uint8_t k_std_dc_luma_bits[16]   = {0, 1, 5, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0};
        const uint8_t k_std_dc_chroma_bits[16] = {0, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0};
        const uint8_t k_std_dc_vals[12]        = {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11};
        const uint8_t k_std_ac_luma_bits[16]   = {0, 2, 1, 3, 3, 2, 4, 3, 5, 5, 4, 4, 0, 0, 1, 0x7d};
        const uint8_t k_std_ac_luma_vals[162]  = {
            0x01, 0x02, 0x03, 0x00, 0x04, 0x11, 0x05, 0x12, 0x21, 0x31, 0x41, 0x06, 0x13, 0x51, 0x61, 0x07, 0x22, 0x71,
            0x14, 0x32, 0x81, 0x91, 0xa1, 0x08, 0x23, 0x42, 0xb1, 0xc1, 0x15, 0x52, 0xd1, 0xf0, 0x24, 0x33, 0x62, 0x72,
            0x82, 0x09, 0x0a, 0x16, 0x17, 0x18, 0x19, 0x1a, 0x25, 0x26, 0x27, 0x28, 0x29, 0x2a, 0x34, 0x35, 0x36, 0x37,
            0x38, 0x39, 0x3a, 0x43, 0x44, 0x45, 0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58, 0x59,
            0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68, 0x69, 0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a, 0x83,
            0x84, 0x85, 0x86, 0x87, 0x88, 0x89, 0x8a, 0x92, 0x93, 0x94, 0x95, 0x96, 0x97, 0x98, 0x99, 0x9a, 0xa2, 0xa3,
            0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4, 0xb5, 0xb6, 0xb7, 0xb8, 0xb9, 0xba, 0xc2, 0xc3,
            0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6, 0xd7, 0xd8, 0xd9, 0xda, 0xe1, 0xe2,
            0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf1, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8, 0xf9, 0xfa};
        const uint8_t k_std_ac_chroma_bits[16] = {0, 2, 1, 2, 4, 4, 3, 4, 7, 5, 4, 4, 0, 1, 2, 0x77};
        const uint8_t k_std_ac_chroma_vals[162] = {
            0x00, 0x01, 0x02, 0x03, 0x11, 0x04, 0x05, 0x21, 0x31, 0x06, 0x12, 0x41, 0x51, 0x07, 0x61, 0x71, 0x13, 0x22,
            0x32, 0x81, 0x08, 0x14, 0x42, 0x91, 0xa1, 0xb1, 0xc1, 0x09, 0x23, 0x33, 0x52, 0xf0, 0x15, 0x62, 0x72, 0xd1,
            0x0a, 0x16, 0x24, 0x34, 0xe1, 0x25, 0xf1, 0x17, 0x18, 0x19, 0x1a, 0x26, 0x27, 0x28, 0x29, 0x2a, 0x35, 0x36,
            0x37, 0x38, 0x39, 0x3a, 0x43, 0x44, 0x45, 0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58,
            0x59, 0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68, 0x69, 0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a,
            0x82, 0x83, 0x84, 0x85, 0x86, 0x87, 0x88, 0x89, 0x8a, 0x92, 0x93, 0x94, 0x95, 0x96, 0x97, 0x98, 0x99, 0x9a,
            0xa2, 0xa3, 0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4, 0xb5, 0xb6, 0xb7, 0xb8, 0xb9, 0xba,
            0xc2, 0xc3, 0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6, 0xd7, 0xd8, 0xd9, 0xda,
            0xe2, 0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8, 0xf9, 0xfa};

        void set_std(jpeg_frame::huff& h, const uint8_t* bits, const uint8_t* vals, int n)
        {
            h.present = true;
            h.bits[0] = 0;
            std::memcpy(h.bits + 1, bits, 16);
            std::memcpy(h.vals, vals, n);
        }

        constexpr int LOOK = 10;

        struct decode_table
        {
            // lookup[peek]: (code length << 8) | symbol for codes of at most LOOK bits, 0 otherwise
            uint16_t lookup[1 << LOOK];
            // fast_ac[peek]: for AC tables, whole (run, size, value) when code + value bits fit in LOOK bits:
            // (value << 8) | (run << 4) | total bits; 0 when not available
            int16_t fast_ac[1 << LOOK];
            int32_t maxcode[18]; // maxcode[len] = largest code of this length, left-justified to 16 bits (+1), or -1
            int32_t valoff[17];
            uint8_t vals[256];

            void build(const jpeg_frame::huff& h, bool is_ac)
            {
                if (!h.present)
                    bad("missing Huffman table");
                std::memset(lookup, 0, sizeof lookup);
                std::memset(fast_ac, 0, sizeof fast_ac);
                std::memcpy(vals, h.vals, 256);
                int code = 0, k = 0;
                for (int len = 1; len <= 16; ++len)
                {
                    valoff[len] = k - code;
                    for (int i = 0; i < h.bits[len]; ++i, ++k, ++code)
                    {
                        if (len <= LOOK)
                        {
                            const int first = code << (LOOK - len);
                            for (int j = 0; j < (1 << (LOOK - len)); ++j)
                                lookup[first + j] = static_cast<uint16_t>((len << 8) | h.vals[k]);
                        }
                    }
                    if (code > (1 << len))
                        bad("invalid Huffman table");
                    maxcode[len] = h.bits[len] ? (code << (16 - len)) : -1; // exclusive upper bound, left-justified
                    code <<= 1;
                }
                maxcode[17] = 0x7fffffff;
                if (!is_ac)
                    return;
                for (int i = 0; i < (1 << LOOK); ++i)
                {
                    const uint16_t e = lookup[i];
                    if (!e)
                        continue;
                    const int len = e >> 8, rs = e & 255, run = rs >> 4, mag = rs & 15;
                    if (mag && len + mag <= LOOK)
                    {
                        int v = (i >> (LOOK - len - mag)) & ((1 << mag) - 1);
                        if (v < (1 << (mag - 1)))
                            v -= (1 << mag) - 1;
                        if (v >= -128 && v <= 127)
                            fast_ac[i] = static_cast<int16_t>((v * 256) | (run << 4) | (len + mag));
                    }
                }
            }
        };

        struct bit_reader
        {
            const uint8_t* p;
            const uint8_t* end;
            uint64_t       acc = 0; // bits are consumed from the top
            int            n   = 0;

            bit_reader(const uint8_t* b, const uint8_t* e) : p(b), end(e) {}

            // Tops the accumulator up to more than 32 valid bits (a code plus its value bits need at most 31).
            // Fast path: four bytes at once when none of
            // them is 0xFF (no stuffing, no marker) -- true for almost every refill of natural images.
            inline void refill()
            {
                if (n > 32)
                    return;
                if (end - p >= 4)
                {
                    uint32_t w;
                    std::memcpy(&w, p, 4);
                    // any byte equal to 0xFF?  (classic zero-byte test on the complement)
                    const uint32_t inv = ~w;
                    if (!((inv - 0x01010101u) & ~inv & 0x80808080u))
                    {
                        const uint64_t be = __builtin_bswap32(w);
                        acc |= be << (32 - n);
                        n += 32;
                        p += 4;
                        return;
                    }
                }
                while (n <= 56)
                {
                    uint64_t b = 0;
                    if (p < end)
                    {
                        b = *p;
                        if (b == 0xFF)
                        {
                            if (p + 1 < end && p[1] == 0)
                                p += 2;
                            else
                                b = 0; // a marker: the segment is over, feed zero bits and stay put
                        }
                        else
                            ++p;
                    }
                    acc |= b << (56 - n);
                    n += 8;
                }
            }
            inline uint32_t peek(int k) const { return static_cast<uint32_t>(acc >> (64 - k)); }
            inline void     skip(int k)
            {
                acc <<= k;
                n -= k;
            }
            // value of `s` magnitude bits with the JPEG sign extension (T.81 F.2.2.1)
            inline int receive_extend(int s)
            {
                const uint32_t v = peek(s);
                skip(s);
                return static_cast<int>(v) - (static_cast<int>(((v >> (s - 1)) ^ 1u)) * ((1 << s) - 1));
            }
            inline int decode(const decode_table& t)
            {
                const uint16_t e = t.lookup[peek(LOOK)];
                if (e)
                {
                    skip(e >> 8);
                    return e & 255;
                }
                const int32_t c16 = static_cast<int32_t>(peek(16));
                int           len = LOOK + 1;
                while (len <= 16 && (t.maxcode[len] < 0 || c16 >= t.maxcode[len]))
                    ++len;
                if (len > 16)
                    bad("bad Huffman code");
                skip(len);
                return t.vals[(c16 >> (16 - len)) + t.valoff[len]];
            }
            void restart()
            {
                acc = 0;
                n   = 0;
                while (p + 1 < end && !(p[0] == 0xFF && p[1] >= 0xD0 && p[1] <= 0xD7))
                    ++p;
                if (p + 1 < end)
                    p += 2;
            }
        };

        inline unsigned be16(const uint8_t* p) { return (unsigned(p[0]) << 8) | p[1]; }
    }

    namespace
    {
        // EXIF orientation (tag 0x0112 of IFD0) from the payload of an APP1 segment; 1 when absent or malformed.
        int exif_orientation(const uint8_t* s, const uint8_t* send)
        {
            if (send - s < 14 || std::memcmp(s, "Exif\0\0", 6) != 0)
                return 1;
            const uint8_t* t  = s + 6; // TIFF header
            const bool     le = t[0] == 'I' && t[1] == 'I';
            if (!le && !(t[0] == 'M' && t[1] == 'M'))
                return 1;
            auto u16 = [&](const uint8_t* q) { return le ? unsigned(q[0]) | unsigned(q[1]) << 8 : unsigned(q[0]) << 8 | q[1]; };
            auto u32 = [&](const uint8_t* q) {
                return le ? unsigned(q[0]) | unsigned(q[1]) << 8 | unsigned(q[2]) << 16 | unsigned(q[3]) << 24
                          : unsigned(q[0]) << 24 | unsigned(q[1]) << 16 | unsigned(q[2]) << 8 | q[3];
            };
            if (u16(t + 2) != 0x002A)
                return 1;
            const size_t room = static_cast<size_t>(send - t);
            const size_t ifd  = u32(t + 4);
            if (ifd + 2 > room)
                return 1;
            const unsigned count = u16(t + ifd);
            for (unsigned i = 0; i < count; ++i)
            {
                const size_t e = ifd + 2 + 12 * static_cast<size_t>(i);
                if (e + 12 > room)
                    break;
                if (u16(t + e) == 0x0112)
                {
                    const unsigned v = u16(t + e + 8);
                    return v >= 1 && v <= 8 ? static_cast<int>(v) : 1;
                }
            }
            return 1;
        }
    }

    void jpeg_parse(const void* data, size_t size, jpeg_frame& f)
    {
        const uint8_t* d   = static_cast<const uint8_t*>(data);
        const uint8_t* end = d + size;
        if (size < 4 || d[0] != 0xFF || d[1] != 0xD8)
            bad("not a JPEG stream");
        f                  = jpeg_frame();
        f.info.orientation = 1;
        set_std(f.dc[0], k_std_dc_luma_bits, k_std_dc_vals, 12);
        set_std(f.dc[1], k_std_dc_chroma_bits, k_std_dc_vals, 12);
        set_std(f.ac[0], k_std_ac_luma_bits, k_std_ac_luma_vals, 162);
        set_std(f.ac[1], k_std_ac_chroma_bits, k_std_ac_chroma_vals, 162);
        uint16_t qt[4][64];
        bool     qt_present[4] = {false, false, false, false};
        int      comp_id[3] = {0, 0, 0}, comp_tq[3] = {0, 0, 0};
        bool     have_sof = false;
        const uint8_t* p  = d + 2;
        for (;;)
        {
            while (p < end && *p != 0xFF)
                ++p;
            while (p < end && *p == 0xFF)
                ++p;
            if (p >= end)
                bad("no image data");
            const int m = *p++;
            if (m == 0xD9)
                bad("no image data");
            if ((m >= 0xD0 && m <= 0xD7) || m == 0x01)
                continue;
            if (p + 2 > end)
                bad("truncated header");
            const unsigned len = be16(p);
            if (len < 2 || p + len > end)
                bad("truncated header");
            const uint8_t* s    = p + 2;
            const uint8_t* send = p + len;
            switch (m)
            {
            case 0xDB:
                while (s < send)
                {
                    const int pq = *s >> 4, tq = *s & 15;
                    ++s;
                    if (tq > 3 || s + (pq ? 128 : 64) > send)
                        bad("bad quantisation table");
                    for (int i = 0; i < 64; ++i)
                    {
                        unsigned v = pq ? be16(s) : *s;
                        s += pq ? 2 : 1;
                        qt[tq][k_zz_colmajor.v[i]] = static_cast<uint16_t>(v);
                    }
                    qt_present[tq] = true;
                }
                break;
            case 0xC0:
            case 0xC1:
            case 0xC2:
            {
                f.progressive = m == 0xC2;
                if (send - s < 6 || s[0] != 8)
                    bad("only 8-bit JPEG is supported");
                f.info.height = be16(s + 1);
                f.info.width  = be16(s + 3);
                f.info.ncomp  = s[5];
                if ((f.info.ncomp != 1 && f.info.ncomp != 3) || send - s < 6 + 3 * f.info.ncomp)
                    bad("unsupported number of components");
                if (f.info.width <= 0 || f.info.height <= 0)
                    bad("empty image");
                for (int i = 0; i < f.info.ncomp; ++i)
                {
                    comp_id[i]   = s[6 + 3 * i];
                    f.comp_id[i] = comp_id[i];
                    f.info.hs[i] = s[7 + 3 * i] >> 4;
                    f.info.vs[i] = s[7 + 3 * i] & 15;
                    comp_tq[i]   = s[8 + 3 * i];
                    if (comp_tq[i] > 3 || f.info.hs[i] < 1 || f.info.vs[i] < 1)
                        bad("bad frame header");
                }
                have_sof = true;
                break;
            }
            case 0xC3: case 0xC5: case 0xC6: case 0xC7: case 0xC9: case 0xCA: case 0xCB: case 0xCD: case 0xCE: case 0xCF:
                bad("only baseline sequential and progressive Huffman JPEG are supported");
            case 0xC4:
                while (s < send)
                {
                    const int tc = *s >> 4, th = *s & 15;
                    ++s;
                    if (tc > 1 || th > 3 || s + 16 > send)
                        bad("bad Huffman table");
                    jpeg_frame::huff& h = tc ? f.ac[th] : f.dc[th];
                    h.present           = true;
                    h.bits[0]           = 0;
                    int n               = 0;
                    for (int i = 1; i <= 16; ++i)
                        n += (h.bits[i] = s[i - 1]);
                    s += 16;
                    if (n > 256 || s + n > send)
                        bad("bad Huffman table");
                    std::memset(h.vals, 0, 256);
                    std::memcpy(h.vals, s, n);
                    s += n;
                }
                break;
            case 0xDD:
                if (send - s < 2)
                    bad("bad restart interval");
                f.restart_interval = be16(s);
                break;
            case 0xE1:
                if (f.info.orientation == 1)
                    f.info.orientation = exif_orientation(s, send);
                break;
            case 0xDA:
            {
                if (!have_sof)
                    bad("scan before frame header");
                if (send - s < 1)
                    bad("bad scan header");
                const int ns = s[0];
                if (send - s < 1 + 2 * ns + 3) // component selectors, then Ss, Se, Ah/Al
                    bad("bad scan header");
                if (!f.progressive && ns != f.info.ncomp)
                    bad("non-interleaved scans are not supported");
                f.first_sos  = p - 2;
                f.stream_end = end;
                for (int i = 0; i < ns && !f.progressive; ++i)
                {
                    int c = -1;
                    for (int j = 0; j < f.info.ncomp; ++j)
                        if (comp_id[j] == s[1 + 2 * i])
                            c = j;
                    if (c < 0)
                        bad("bad scan header");
                    f.dc_table[c] = s[2 + 2 * i] >> 4;
                    f.ac_table[c] = s[2 + 2 * i] & 15;
                    if (f.dc_table[c] > 3 || f.ac_table[c] > 3)
                        bad("bad scan header");
                }
                f.scan      = send;
                f.scan_size = static_cast<size_t>(end - send);
                // finalise geometry
                aeonb_jpeg_info& in = f.info;
                if (in.ncomp == 1)
                    in.hs[0] = in.vs[0] = 1;
                int hmax = 1, vmax = 1;
                for (int i = 0; i < in.ncomp; ++i)
                {
                    hmax = std::max(hmax, in.hs[i]);
                    vmax = std::max(vmax, in.vs[i]);
                }
                const int mcux = (in.width + 8 * hmax - 1) / (8 * hmax);
                const int mcuy = (in.height + 8 * vmax - 1) / (8 * vmax);
                for (int i = 0; i < in.ncomp; ++i)
                {
                    if (!qt_present[comp_tq[i]])
                        bad("missing quantisation table");
                    std::memcpy(f.quant[i], qt[comp_tq[i]], sizeof f.quant[i]);
                    in.blocks_w[i]   = mcux * in.hs[i];
                    in.blocks_h[i]   = mcuy * in.vs[i];
                    in.coef_count[i] = static_cast<int64_t>(in.blocks_w[i]) * in.blocks_h[i] * 64;
                }
                if (in.ncomp == 3)
                {
                    const bool chroma_ok = in.hs[1] == 1 && in.vs[1] == 1 && in.hs[2] == 1 && in.vs[2] == 1;
                    const bool luma_ok   = (in.hs[0] == 1 && in.vs[0] == 1) || (in.hs[0] == 2 && in.vs[0] == 1) ||
                                         (in.hs[0] == 2 && in.vs[0] == 2) || (in.hs[0] == 1 && in.vs[0] == 2) ||
                                         (in.hs[0] == 4 && in.vs[0] == 1);
                    if (!chroma_ok || !luma_ok)
                        bad("unsupported chroma subsampling (supported: 4:4:4, 4:2:2, 4:2:0, 4:4:0, 4:1:1)");
                }
                return;
            }
            default: break; // APPn, COM, ...: skipped
            }
            p += len;
        }
    }

    jpeg_roi jpeg_roi_for_box(const aeonb_jpeg_info& in, int x0, int y0, int x1, int y1)
    {
        const int mw = 8 * in.hs[0], mh = 8 * in.vs[0];
        const int mcux = in.blocks_w[0] / in.hs[0], mcuy = in.blocks_h[0] / in.vs[0];
        x0 = std::max(x0, 0);
        y0 = std::max(y0, 0);
        x1 = std::min(x1, in.width);
        y1 = std::min(y1, in.height);
        if (x1 <= x0 || y1 <= y0)
            return jpeg_roi{0, 0, 1, 1};
        jpeg_roi r;
        r.mx0 = std::max(x0 - 2, 0) / mw;
        r.my0 = std::max(y0 - 2, 0) / mh;
        r.mx1 = std::min(mcux, (x1 + 2 + mw - 1) / mw);
        r.my1 = std::min(mcuy, (y1 + 2 + mh - 1) / mh);
        return r;
    }

    namespace
    {
        // One scan of a progressive stream (ITU-T T.81 annex G): a band Ss..Se of the zig-zag sequence at bit position
        // Al, either the first pass over it (Ah == 0) or a refinement that adds one bit (Ah == Al + 1).
        struct progressive_scan
        {
            int ncomp = 0, comp[3]{}, dc_tab[3]{}, ac_tab[3]{};
            int ss = 0, se = 0, ah = 0, al = 0;
        };

        inline int get_bits(bit_reader& br, int n)
        {
            br.refill();
            const int v = static_cast<int>(br.peek(n));
            br.skip(n);
            return v;
        }

        // Refinement of the already non-zero coefficients from k on, until `zeros` still-zero positions have been
        // passed (zeros < 0: to the end of the band): each gets one correction bit (figure G.7).
        inline int refine_nonzeros(bit_reader& br, int16_t* blk, const uint8_t* zz, int k, int se, int zeros, int p1, int m1)
        {
            for (; k <= se; ++k)
            {
                int16_t& c = blk[zz[k]];
                if (c != 0)
                {
                    if (get_bits(br, 1) && (c & p1) == 0)
                        c = static_cast<int16_t>(c + (c >= 0 ? p1 : m1));
                }
                else if (zeros >= 0 && --zeros < 0)
                    break;
            }
            return k;
        }

        void decode_progressive_scan(const jpeg_frame& f, const progressive_scan& sc, const jpeg_frame::huff* dc_tabs,
                                     const jpeg_frame::huff* ac_tabs, int restart_interval, bit_reader& br, int16_t* const coef[3])
        {
            const aeonb_jpeg_info& in = f.info;
            const uint8_t*         zz = k_zz_colmajor.v;
            int hmax = 1, vmax = 1;
            for (int c = 0; c < in.ncomp; ++c)
            {
                hmax = std::max(hmax, in.hs[c]);
                vmax = std::max(vmax, in.vs[c]);
            }
            decode_table dct[3], act[3];
            for (int i = 0; i < sc.ncomp; ++i)
            {
                if (sc.ss == 0 && sc.ah == 0)
                    dct[i].build(dc_tabs[sc.dc_tab[i]], false);
                if (sc.ss > 0)
                    act[i].build(ac_tabs[sc.ac_tab[i]], true);
            }
            int       pred[3]       = {0, 0, 0};
            int       eobrun        = 0;
            int       until_restart = restart_interval ? restart_interval : -1;
            const int p1 = 1 << sc.al, m1 = -(1 << sc.al);
            auto restart_check = [&]() {
                if (until_restart == 0)
                {
                    br.restart();
                    pred[0] = pred[1] = pred[2] = 0;
                    eobrun                      = 0;
                    until_restart               = restart_interval;
                }
                if (until_restart > 0)
                    --until_restart;
            };
            auto block_at = [&](int c, int bx, int by) { return coef[c] + (static_cast<size_t>(by) * in.blocks_w[c] + bx) * 64; };
            auto decode_block = [&](int i, int16_t* blk) {
                const int c = sc.comp[i];
                if (sc.ss == 0)
                {
                    if (sc.ah == 0)
                    {
                        br.refill();
                        const int t = br.decode(dct[i]);
                        if (t > 15)
                            bad("bad DC coefficient");
                        if (t)
                        {
                            br.refill();
                            pred[c] += br.receive_extend(t);
                        }
                        blk[0] = static_cast<int16_t>(pred[c] * (1 << sc.al));
                    }
                    else if (get_bits(br, 1))
                        blk[0] = static_cast<int16_t>(blk[0] | p1);
                    return;
                }
                if (sc.ah == 0)
                {
                    if (eobrun > 0)
                    {
                        --eobrun;
                        return;
                    }
                    for (int k = sc.ss; k <= sc.se; ++k)
                    {
                        br.refill();
                        const int rs = br.decode(act[i]);
                        const int r = rs >> 4, s = rs & 15;
                        if (s)
                        {
                            k += r;
                            if (k > 63)
                                bad("corrupt coefficient run");
                            br.refill();
                            blk[zz[k]] = static_cast<int16_t>(br.receive_extend(s) * (1 << sc.al));
                        }
                        else if (r == 15)
                            k += 15;
                        else
                        {
                            eobrun = 1 << r;
                            if (r)
                                eobrun += get_bits(br, r);
                            --eobrun;
                            break;
                        }
                    }
                    return;
                }
                // refinement of an AC band
                int k = sc.ss;
                if (eobrun == 0)
                {
                    for (; k <= sc.se; ++k)
                    {
                        br.refill();
                        const int rs = br.decode(act[i]);
                        int       r = rs >> 4, s = rs & 15;
                        int       value = 0;
                        if (s)
                            value = get_bits(br, 1) ? p1 : m1; // a newly non-zero coefficient has magnitude 1 at this bit
                        else if (r != 15)
                        {
                            eobrun = 1 << r;
                            if (r)
                                eobrun += get_bits(br, r);
                            break;
                        }
                        k = refine_nonzeros(br, blk, zz, k, sc.se, r, p1, m1);
                        if (k > 63)
                            bad("corrupt coefficient run");
                        if (s)
                            blk[zz[k]] = static_cast<int16_t>(value);
                    }
                }
                if (eobrun > 0)
                {
                    refine_nonzeros(br, blk, zz, k, sc.se, -1, p1, m1);
                    --eobrun;
                }
            };
            if (sc.ncomp > 1)
            {
                // interleaved (DC scans only): MCU order, all hs x vs blocks of every component
                const int mcux = in.blocks_w[0] / in.hs[0], mcuy = in.blocks_h[0] / in.vs[0];
                for (int my = 0; my < mcuy; ++my)
                    for (int mx = 0; mx < mcux; ++mx)
                    {
                        restart_check();
                        for (int i = 0; i < sc.ncomp; ++i)
                        {
                            const int c = sc.comp[i];
                            for (int by = 0; by < in.vs[c]; ++by)
                                for (int bx = 0; bx < in.hs[c]; ++bx)
                                    decode_block(i, block_at(c, mx * in.hs[c] + bx, my * in.vs[c] + by));
                        }
                    }
            }
            else
            {
                // non-interleaved: the component's own blocks in raster order, only those that hold picture samples
                const int c  = sc.comp[0];
                const int cw = (in.width * in.hs[c] + hmax - 1) / hmax, ch = (in.height * in.vs[c] + vmax - 1) / vmax;
                const int bw = (cw + 7) / 8, bh = (ch + 7) / 8;
                for (int by = 0; by < bh; ++by)
                    for (int bx = 0; bx < bw; ++bx)
                    {
                        restart_check();
                        decode_block(0, block_at(c, bx, by));
                    }
            }
        }

        // All scans of a progressive stream into whole-picture planes (zeroed here).
        void jpeg_progressive_decode(const jpeg_frame& f, int16_t* const coef[3])
        {
            const aeonb_jpeg_info& in = f.info;
            for (int c = 0; c < in.ncomp; ++c)
                std::memset(coef[c], 0, static_cast<size_t>(in.coef_count[c]) * sizeof(int16_t));
            jpeg_frame::huff dc[4], ac[4];
            for (int i = 0; i < 4; ++i)
            {
                dc[i] = f.dc[i];
                ac[i] = f.ac[i];
            }
            int            restart_interval = f.restart_interval;
            const uint8_t* p   = f.first_sos;
            const uint8_t* end = f.stream_end;
            int            scans = 0;
            while (p && p + 4 <= end)
            {
                // p stands on a marker (0xFF, code)
                while (p < end && *p != 0xFF)
                    ++p;
                while (p < end && *p == 0xFF)
                    ++p;
                if (p >= end)
                    break;
                const int m = *p++;
                if (m == 0xD9)
                    break;
                if ((m >= 0xD0 && m <= 0xD7) || m == 0x01 || m == 0x00)
                    continue;
                if (p + 2 > end)
                    bad("truncated header");
                const unsigned len = be16(p);
                if (len < 2 || p + len > end)
                    bad("truncated header");
                const uint8_t* s    = p + 2;
                const uint8_t* send = p + len;
                p                   = send;
                if (m == 0xC4)
                {
                    while (s < send)
                    {
                        const int tc = *s >> 4, th = *s & 15;
                        ++s;
                        if (tc > 1 || th > 3 || s + 16 > send)
                            bad("bad Huffman table");
                        jpeg_frame::huff& h = tc ? ac[th] : dc[th];
                        h.present           = true;
                        h.bits[0]           = 0;
                        int n               = 0;
                        for (int i = 1; i <= 16; ++i)
                            n += (h.bits[i] = s[i - 1]);
                        s += 16;
                        if (n > 256 || s + n > send)
                            bad("bad Huffman table");
                        std::memset(h.vals, 0, 256);
                        std::memcpy(h.vals, s, n);
                        s += n;
                    }
                }
                else if (m == 0xDD)
                {
                    if (send - s < 2)
                        bad("bad restart interval");
                    restart_interval = be16(s);
                }
                else if (m == 0xDA)
                {
                    progressive_scan sc;
                    sc.ncomp = s[0];
                    if (sc.ncomp < 1 || sc.ncomp > in.ncomp || send - s < 4 + 2 * sc.ncomp)
                        bad("bad scan header");
                    for (int i = 0; i < sc.ncomp; ++i)
                    {
                        int c = -1;
                        for (int j = 0; j < in.ncomp; ++j)
                            if (f.comp_id[j] == s[1 + 2 * i])
                                c = j;
                        if (c < 0)
                            bad("bad scan header");
                        sc.comp[i]   = c;
                        sc.dc_tab[i] = s[2 + 2 * i] >> 4;
                        sc.ac_tab[i] = s[2 + 2 * i] & 15;
                        if (sc.dc_tab[i] > 3 || sc.ac_tab[i] > 3)
                            bad("bad scan header");
                    }
                    const uint8_t* t = s + 1 + 2 * sc.ncomp;
                    sc.ss = t[0];
                    sc.se = t[1];
                    sc.ah = t[2] >> 4;
                    sc.al = t[2] & 15;
                    const bool band_ok = sc.ss == 0 ? sc.se == 0 : (sc.ss <= sc.se && sc.se <= 63 && sc.ncomp == 1);
                    if (!band_ok || sc.al > 13 || (sc.ah != 0 && sc.ah != sc.al + 1))
                        bad("bad progressive scan parameters");
                    bit_reader br(send, end);
                    decode_progressive_scan(f, sc, dc, ac, restart_interval, br, coef);
                    p = br.p; // at or before the marker that ends the scan's data
                    // skip what is left of the entropy-coded segment: to the next marker that is not a restart marker
                    while (p + 1 < end && !(p[0] == 0xFF && p[1] != 0x00 && p[1] != 0xFF && !(p[1] >= 0xD0 && p[1] <= 0xD7)))
                        ++p;
                    if (++scans > 1000)
                        bad("too many scans");
                }
            }
            if (scans == 0)
                bad("no image data");
        }
    }

    void jpeg_entropy_decode(const jpeg_frame& f, int16_t* const coef[3], const jpeg_roi* roi)
    {
        if (f.progressive)
        {
            const aeonb_jpeg_info& pin = f.info;
            if (!roi)
            {
                jpeg_progressive_decode(f, coef);
                return;
            }
            // the scans cover the whole picture: decode all of it, then keep the region's blocks
            std::vector<int16_t> whole[3];
            int16_t*             planes[3] = {nullptr, nullptr, nullptr};
            for (int c = 0; c < pin.ncomp; ++c)
            {
                whole[c].resize(static_cast<size_t>(pin.coef_count[c]));
                planes[c] = whole[c].data();
            }
            jpeg_progressive_decode(f, planes);
            const int pmcux = pin.blocks_w[0] / pin.hs[0], pmcuy = pin.blocks_h[0] / pin.vs[0];
            const int x0 = std::max(roi->mx0, 0), x1 = std::min(roi->mx1, pmcux), y0 = std::max(roi->my0, 0), y1 = std::min(roi->my1, pmcuy);
            for (int c = 0; c < pin.ncomp; ++c)
            {
                const int bw = (x1 - x0) * pin.hs[c];
                for (int by = 0; by < (y1 - y0) * pin.vs[c]; ++by)
                    std::memcpy(coef[c] + static_cast<size_t>(by) * bw * 64,
                                planes[c] + (static_cast<size_t>(y0 * pin.vs[c] + by) * pin.blocks_w[c] + x0 * pin.hs[c]) * 64,
                                static_cast<size_t>(bw) * 64 * sizeof(int16_t));
            }
            return;
        }
        const aeonb_jpeg_info& in = f.info;
        decode_table           dct[3], act[3];
        for (int c = 0; c < in.ncomp; ++c)
        {
            dct[c].build(f.dc[f.dc_table[c]], false);
            act[c].build(f.ac[f.ac_table[c]], true);
        }
        const int mcux = in.blocks_w[0] / in.hs[0];
        const int mcuy = in.blocks_h[0] / in.vs[0];
        const int mx0 = roi ? std::max(roi->mx0, 0) : 0, mx1 = roi ? std::min(roi->mx1, mcux) : mcux;
        const int my0 = roi ? std::max(roi->my0, 0) : 0, my1 = roi ? std::min(roi->my1, mcuy) : mcuy;
        int16_t    outside[64]; // blocks outside the region are decoded into this and dropped
        bit_reader br(f.scan, f.scan + f.scan_size);
        int        pred[3] = {0, 0, 0};
        int        until_restart = f.restart_interval ? f.restart_interval : -1;
        const uint8_t* zz = k_zz_colmajor.v;
        for (int my = 0; my < my1; ++my)
        {
            for (int mx = 0; mx < mcux; ++mx)
            {
                const bool keep = my >= my0 && mx >= mx0 && mx < mx1;
                if (until_restart == 0)
                {
                    br.restart();
                    pred[0] = pred[1] = pred[2] = 0;
                    until_restart               = f.restart_interval;
                }
                if (until_restart > 0)
                    --until_restart;
                for (int c = 0; c < in.ncomp; ++c)
                {
                    const decode_table& dt = dct[c];
                    const decode_table& at = act[c];
                    for (int by = 0; by < in.vs[c]; ++by)
                    {
                        for (int bx = 0; bx < in.hs[c]; ++bx)
                        {
                            int16_t* blk = keep ? coef[c] + (static_cast<size_t>((my - my0) * in.vs[c] + by) * ((mx1 - mx0) * in.hs[c]) +
                                                             ((mx - mx0) * in.hs[c] + bx)) * 64
                                                : outside;
                            std::memset(blk, 0, 64 * sizeof(int16_t));
                            br.refill();
                            const int t = br.decode(dt);
                            if (t > 15)
                                bad("bad DC coefficient");
                            if (t)
                            {
                                br.refill();
                                pred[c] += br.receive_extend(t);
                            }
                            blk[0] = static_cast<int16_t>(pred[c]);
                            int k  = 1;
                            while (k < 64)
                            {
                                br.refill();
                                const int16_t fa = at.fast_ac[br.peek(LOOK)];
                                if (fa)
                                {
                                    k += (fa >> 4) & 15;
                                    if (k > 63)
                                        bad("corrupt coefficient run");
                                    br.skip(fa & 15);
                                    blk[zz[k++]] = static_cast<int16_t>(fa >> 8);
                                    continue;
                                }
                                const int rs = br.decode(at);
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
                                    bad("corrupt coefficient run");
                                blk[zz[k++]] = static_cast<int16_t>(br.receive_extend(s));
                            }
                        }
                    }
                }
            }
        }
    }

    bool jpeg_entropy_prepare(const jpeg_frame& f, uint8_t tables[4 * 272], aeonb_entropy_desc& d)
    {
        std::memset(tables, 0, 4 * 272);
        d                     = aeonb_entropy_desc{};
        if (f.progressive)
            return false; // several scans over the same coefficients: decoded on the host
        const aeonb_jpeg_info& in = f.info;
        int dc_ids[2] = {-1, -1}, ac_ids[2] = {-1, -1};
        auto slot_of = [](int ids[2], int id) {
            for (int s = 0; s < 2; ++s)
            {
                if (ids[s] == id)
                    return s;
                if (ids[s] < 0)
                {
                    ids[s] = id;
                    return s;
                }
            }
            return -1;
        };
        for (int c = 0; c < in.ncomp; ++c)
        {
            const int ds = slot_of(dc_ids, f.dc_table[c]), as = slot_of(ac_ids, f.ac_table[c]);
            if (ds < 0 || as < 0)
                return false;
            d.dc_table[c] = ds;
            d.ac_table[c] = as;
            d.hs[c]       = in.hs[c];
            d.vs[c]       = in.vs[c];
        }
        for (int s = 0; s < 2; ++s)
        {
            if (dc_ids[s] >= 0)
            {
                std::memcpy(tables + s * 272, f.dc[dc_ids[s]].bits + 1, 16);
                std::memcpy(tables + s * 272 + 16, f.dc[dc_ids[s]].vals, 256);
            }
            if (ac_ids[s] >= 0)
            {
                std::memcpy(tables + (2 + s) * 272, f.ac[ac_ids[s]].bits + 1, 16);
                std::memcpy(tables + (2 + s) * 272 + 16, f.ac[ac_ids[s]].vals, 256);
            }
        }
        d.ncomp            = in.ncomp;
        d.scan_size        = static_cast<uint32_t>(f.scan_size);
        d.mcux             = in.blocks_w[0] / in.hs[0];
        d.mcuy             = in.blocks_h[0] / in.vs[0];
        d.roi[0]           = 0;
        d.roi[1]           = 0;
        d.roi[2]           = d.mcux;
        d.roi[3]           = d.mcuy;
        d.restart_interval = f.restart_interval;
        return true;
    }
}

using namespace aeonb;

extern "C" {

int aeonb_jpeg_parse(const void* data, size_t size, aeonb_jpeg_info* info)
{
    return guarded([&]() {
        if (!data || !info)
            throw std::invalid_argument("aeonb_jpeg_parse: NULL argument");
        jpeg_frame f;
        jpeg_parse(data, size, f);
        *info = f.info;
        return AEONB_OK;
    });
}

int aeonb_jpeg_roi_for_crop(const aeonb_jpeg_info* info, int crop_x, int crop_y, int crop_w, int crop_h, int32_t roi[4])
{
    return guarded([&]() {
        if (!info || !roi)
            throw std::invalid_argument("aeonb_jpeg_roi_for_crop: NULL argument");
        const jpeg_roi r = jpeg_roi_for_box(*info, crop_x, crop_y, crop_x + crop_w, crop_y + crop_h);
        roi[0] = r.mx0;
        roi[1] = r.my0;
        roi[2] = r.mx1;
        roi[3] = r.my1;
        return AEONB_OK;
    });
}

int aeonb_jpeg_entropy_decode_roi(const void* data, size_t size, const int32_t roi[4], int16_t* coef[3], uint16_t* quant[3])
{
    return guarded([&]() {
        if (!data || !coef || !quant || !roi)
            throw std::invalid_argument("aeonb_jpeg_entropy_decode_roi: NULL argument");
        jpeg_frame f;
        jpeg_parse(data, size, f);
        const int mcux = f.info.blocks_w[0] / f.info.hs[0], mcuy = f.info.blocks_h[0] / f.info.vs[0];
        if (roi[0] < 0 || roi[1] < 0 || roi[2] > mcux || roi[3] > mcuy || roi[0] >= roi[2] || roi[1] >= roi[3])
            throw std::invalid_argument("aeonb_jpeg_entropy_decode_roi: region outside the picture");
        for (int c = 0; c < f.info.ncomp; ++c)
        {
            if (!coef[c] || !quant[c])
                throw std::invalid_argument("aeonb_jpeg_entropy_decode_roi: NULL plane");
            std::memcpy(quant[c], f.quant[c], sizeof f.quant[c]);
        }
        jpeg_roi r{roi[0], roi[1], roi[2], roi[3]};
        jpeg_entropy_decode(f, coef, &r);
        return AEONB_OK;
    });
}

int aeonb_jpeg_entropy_prepare(const void* data, size_t size, aeonb_jpeg_info* info, uint16_t quant[192], uint8_t tables[1088],
                               aeonb_entropy_desc* desc, size_t* scan_offset)
{
    return guarded([&]() {
        if (!data || !info || !quant || !tables || !desc || !scan_offset)
            throw std::invalid_argument("aeonb_jpeg_entropy_prepare: NULL argument");
        jpeg_frame f;
        jpeg_parse(data, size, f);
        if (!jpeg_entropy_prepare(f, tables, *desc))
            throw error(AEONB_ERR_UNSUPPORTED, "progressive stream, or a scan with more than two DC or two AC Huffman tables: use aeonb_jpeg_entropy_decode");
        *info = f.info;
        std::memcpy(quant, f.quant, sizeof f.quant);
        *scan_offset = static_cast<size_t>(f.scan - static_cast<const uint8_t*>(data));
        return AEONB_OK;
    });
}

int aeonb_jpeg_entropy_decode(const void* data, size_t size, int16_t* coef[3], uint16_t* quant[3])
{
    return guarded([&]() {
        if (!data || !coef || !quant)
            throw std::invalid_argument("aeonb_jpeg_entropy_decode: NULL argument");
        jpeg_frame f;
        jpeg_parse(data, size, f);
        for (int c = 0; c < f.info.ncomp; ++c)
        {
            if (!coef[c] || !quant[c])
                throw std::invalid_argument("aeonb_jpeg_entropy_decode: NULL plane");
            std::memcpy(quant[c], f.quant[c], sizeof f.quant[c]);
        }
        jpeg_entropy_decode(f, coef);
        return AEONB_OK;
    });
}

} // extern "C"
