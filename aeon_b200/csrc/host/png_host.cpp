#include "png_host.hpp"

#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "../context.hpp"

namespace aeonb
{
    namespace
    {
        const char* const k_bad_image = "Decoding image failed due to invalid data in the image file.";

        [[noreturn]] void bad(const char* detail)
        {
            throw error(AEONB_ERR_DECODE, std::string(k_bad_image) + " (PNG: " + detail + ")");
        }

        const uint8_t k_signature[8] = {0x89, 'P', 'N', 'G', 0x0D, 0x0A, 0x1A, 0x0A};

        inline uint32_t be32(const uint8_t* p) { return uint32_t(p[0]) << 24 | uint32_t(p[1]) << 16 | uint32_t(p[2]) << 8 | p[3]; }

        // ---- inflate (RFC 1951) inside a zlib stream (RFC 1950)

        // Canonical Huffman code of deflate: codes are sent most significant bit first inside a stream that is read
        // least significant bit first, so the lookup table is indexed by the next FAST stream bits with the code reversed.
        struct deflate_code
        {
            static constexpr int FAST = 10;
            uint16_t fast[1 << FAST]; // (length << 9) | symbol, 0 = longer code
            uint16_t count[16];
            uint16_t symbol[288 + 32];

            void build(const uint8_t* lengths, int n)
            {
                std::memset(fast, 0, sizeof fast);
                std::memset(count, 0, sizeof count);
                for (int i = 0; i < n; ++i)
                    ++count[lengths[i]];
                count[0] = 0;
                int left = 1;
                for (int len = 1; len <= 15; ++len)
                {
                    left = (left << 1) - count[len];
                    if (left < 0)
                        bad("over-subscribed Huffman code");
                }
                uint16_t offs[16];
                offs[1] = 0;
                for (int len = 1; len < 15; ++len)
                    offs[len + 1] = static_cast<uint16_t>(offs[len] + count[len]);
                for (int i = 0; i < n; ++i)
                    if (lengths[i])
                        symbol[offs[lengths[i]]++] = static_cast<uint16_t>(i);
                // fast table from the canonical codes
                int code = 0, index = 0;
                for (int len = 1; len <= FAST; ++len)
                {
                    for (int k = 0; k < count[len]; ++k, ++code, ++index)
                    {
                        int rev = 0;
                        for (int b = 0; b < len; ++b)
                            rev |= ((code >> b) & 1) << (len - 1 - b);
                        for (int i = rev; i < (1 << FAST); i += 1 << len)
                            fast[i] = static_cast<uint16_t>((len << 9) | symbol[index]);
                    }
                    code <<= 1;
                }
            }
        };

        struct inflater
        {
            const uint8_t* p;
            const uint8_t* end;
            uint64_t       acc = 0; // bits are consumed from the bottom
            int            n   = 0;

            inflater(const uint8_t* b, const uint8_t* e) : p(b), end(e) {}
            int            over = 0; // bytes made up past the end of the data
            inline void refill()
            {
                while (n <= 56)
                {
                    uint64_t b = 0;
                    if (p < end)
                        b = *p++;
                    else if (++over > 64) // a few zero bytes let the last code finish; more means the stream was cut short
                        bad("truncated data");
                    acc |= b << n;
                    n += 8;
                }
            }
            inline uint32_t bits(int k)
            {
                if (n < k)
                    refill();
                const uint32_t v = static_cast<uint32_t>(acc & ((1ull << k) - 1));
                acc >>= k;
                n -= k;
                return v;
            }
            inline int decode(const deflate_code& h)
            {
                if (n < 16)
                    refill();
                const uint16_t e = h.fast[acc & ((1 << deflate_code::FAST) - 1)];
                if (e)
                {
                    acc >>= e >> 9;
                    n -= e >> 9;
                    return e & 511;
                }
                int code = 0, first = 0, index = 0;
                for (int len = 1; len <= 15; ++len)
                {
                    code |= static_cast<int>((acc >> (len - 1)) & 1);
                    const int cnt = h.count[len];
                    if (code - cnt < first)
                    {
                        acc >>= len;
                        n -= len;
                        return h.symbol[index + (code - first)];
                    }
                    index += cnt;
                    first += cnt;
                    first <<= 1;
                    code <<= 1;
                }
                bad("invalid Huffman code");
            }
        };

        const uint16_t k_len_base[29]  = {3, 4, 5, 6, 7, 8, 9, 10, 11, 13, 15, 17, 19, 23, 27, 31, 35, 43, 51, 59, 67, 83, 99, 115, 131, 163, 195, 227, 258};
        const uint8_t  k_len_extra[29] = {0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3, 4, 4, 4, 4, 5, 5, 5, 5, 0};
        const uint16_t k_dist_base[30] = {1,   2,   3,   4,   5,   7,    9,    13,   17,   25,   33,   49,   65,    97,    129,
                                          193, 257, 385, 513, 769, 1025, 1537, 2049, 3073, 4097, 6145, 8193, 12289, 16385, 24577};
        const uint8_t  k_dist_extra[30] = {0, 0, 0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7, 8, 8, 9, 9, 10, 10, 11, 11, 12, 12, 13, 13};

        // Inflates a zlib stream into exactly `want` bytes.
        void zlib_inflate(const uint8_t* src, size_t size, uint8_t* out, size_t want)
        {
            if (size < 2 || (src[0] & 15) != 8 || ((src[0] << 8) | src[1]) % 31 != 0 || (src[1] & 0x20))
                bad("not a zlib stream");
            inflater     in(src + 2, src + size);
            size_t       o = 0;
            deflate_code lit, dist;
            bool         last = false;
            while (!last)
            {
                last           = in.bits(1) != 0;
                const int type = static_cast<int>(in.bits(2));
                if (type == 0)
                {
                    // stored: back to a byte boundary, LEN, NLEN, bytes
                    in.bits(in.n & 7);
                    const uint32_t len = in.bits(16), nlen = in.bits(16);
                    if ((len ^ 0xFFFF) != nlen)
                        bad("stored block length");
                    for (uint32_t i = 0; i < len; ++i)
                    {
                        if (o >= want)
                            bad("too much data");
                        out[o++] = static_cast<uint8_t>(in.bits(8));
                    }
                    continue;
                }
                if (type == 3)
                    bad("invalid block type");
                if (type == 1)
                {
                    uint8_t l[288 + 30];
                    for (int i = 0; i < 288; ++i)
                        l[i] = i < 144 ? 8 : i < 256 ? 9 : i < 280 ? 7 : 8;
                    lit.build(l, 288);
                    for (int i = 0; i < 30; ++i)
                        l[i] = 5;
                    dist.build(l, 30);
                }
                else
                {
                    const int nlen = static_cast<int>(in.bits(5)) + 257, ndist = static_cast<int>(in.bits(5)) + 1,
                              ncode = static_cast<int>(in.bits(4)) + 4;
                    if (nlen > 286 || ndist > 30)
                        bad("too many codes");
                    static const uint8_t order[19] = {16, 17, 18, 0, 8, 7, 9, 6, 10, 5, 11, 4, 12, 3, 13, 2, 14, 1, 15};
                    uint8_t              cl[19]    = {0};
                    for (int i = 0; i < ncode; ++i)
                        cl[order[i]] = static_cast<uint8_t>(in.bits(3));
                    deflate_code clc;
                    clc.build(cl, 19);
                    uint8_t l[286 + 30];
                    int     i = 0;
                    while (i < nlen + ndist)
                    {
                        const int sym = in.decode(clc);
                        if (sym < 16)
                            l[i++] = static_cast<uint8_t>(sym);
                        else
                        {
                            int rep, val = 0;
                            if (sym == 16)
                            {
                                if (i == 0)
                                    bad("repeat without a previous length");
                                val = l[i - 1];
                                rep = 3 + static_cast<int>(in.bits(2));
                            }
                            else if (sym == 17)
                                rep = 3 + static_cast<int>(in.bits(3));
                            else
                                rep = 11 + static_cast<int>(in.bits(7));
                            if (i + rep > nlen + ndist)
                                bad("too many code lengths");
                            while (rep--)
                                l[i++] = static_cast<uint8_t>(val);
                        }
                    }
                    if (l[256] == 0)
                        bad("no end-of-block code");
                    lit.build(l, nlen);
                    dist.build(l + nlen, ndist);
                }
                for (;;)
                {
                    const int sym = in.decode(lit);
                    if (sym < 256)
                    {
                        if (o >= want)
                            bad("too much data");
                        out[o++] = static_cast<uint8_t>(sym);
                    }
                    else if (sym == 256)
                        break;
                    else
                    {
                        if (sym > 285)
                            bad("invalid length code");
                        const size_t len = k_len_base[sym - 257] + in.bits(k_len_extra[sym - 257]);
                        const int    ds  = in.decode(dist);
                        if (ds > 29)
                            bad("invalid distance code");
                        const size_t d = k_dist_base[ds] + in.bits(k_dist_extra[ds]);
                        if (d > o || o + len > want)
                            bad("distance too far back or too much data");
                        for (size_t i = 0; i < len; ++i, ++o) // the ranges may overlap: byte by byte
                            out[o] = out[o - d];
                    }
                }
            }
            if (o != want)
                bad("not enough data");
        }

        inline int paeth(int a, int b, int c)
        {
            const int p = a + b - c, pa = std::abs(p - a), pb = std::abs(p - b), pc = std::abs(p - c);
            return pa <= pb && pa <= pc ? a : pb <= pc ? b : c;
        }

        struct chunks
        {
            std::vector<uint8_t> idat;
            uint8_t              palette[256][3] = {};
            int                  palette_size = 0;
        };

        // Walks the chunk list: IHDR (already parsed by the caller) ... IDAT+ ... IEND.
        void read_chunks(const uint8_t* d, size_t size, chunks& c)
        {
            size_t pos = 8;
            bool   end = false;
            while (!end && pos + 12 <= size)
            {
                const uint32_t len = be32(d + pos);
                if (len > size - pos - 12)
                    bad("truncated chunk");
                const uint8_t* type = d + pos + 4;
                const uint8_t* body = d + pos + 8;
                if (!std::memcmp(type, "IDAT", 4))
                    c.idat.insert(c.idat.end(), body, body + len);
                else if (!std::memcmp(type, "PLTE", 4))
                {
                    if (len % 3 || len > 768)
                        bad("bad palette");
                    c.palette_size = static_cast<int>(len / 3);
                    std::memcpy(c.palette, body, len);
                }
                else if (!std::memcmp(type, "IEND", 4))
                    end = true;
                pos += 12 + len;
            }
            if (c.idat.empty())
                bad("no image data");
        }
    }

    bool is_png(const void* data, size_t size) { return size >= 8 && !std::memcmp(data, k_signature, 8); }

    void png_parse(const void* data, size_t size, png_info& info)
    {
        const uint8_t* d = static_cast<const uint8_t*>(data);
        if (!is_png(data, size) || size < 8 + 25 || be32(d + 8) != 13 || std::memcmp(d + 12, "IHDR", 4))
            bad("no IHDR chunk");
        info.width      = static_cast<int>(be32(d + 16));
        info.height     = static_cast<int>(be32(d + 20));
        info.bit_depth  = d[24];
        info.color_type = d[25];
        if (info.width <= 0 || info.height <= 0 || info.width > (1 << 20) || info.height > (1 << 20) || d[26] != 0 || d[27] != 0)
            bad("bad IHDR chunk");
        const int  bd = info.bit_depth;
        const bool ok = (info.color_type == 0 && (bd == 1 || bd == 2 || bd == 4 || bd == 8 || bd == 16)) ||
                        (info.color_type == 3 && (bd == 1 || bd == 2 || bd == 4 || bd == 8)) ||
                        ((info.color_type == 2 || info.color_type == 4 || info.color_type == 6) && (bd == 8 || bd == 16));
        if (!ok)
            bad("bad colour type / bit depth");
        if (d[28] > 1)
            bad("bad interlace method");
        info.interlaced = d[28] == 1;
    }

    namespace
    {
        // Undoes the row filters of one image (or one interlace pass) in place: `rows` rows of a filter byte + `row` bytes.
        void unfilter(uint8_t* raw, size_t row, int rows, int bpp)
        {
            std::vector<uint8_t> zero(row, 0);
            const uint8_t*       prev = zero.data();
            for (int y = 0; y < rows; ++y)
            {
                uint8_t*  cur    = raw + static_cast<size_t>(y) * (row + 1) + 1;
                const int filter = cur[-1];
                switch (filter)
                {
                case 0: break;
                case 1:
                    for (size_t i = bpp; i < row; ++i)
                        cur[i] = static_cast<uint8_t>(cur[i] + cur[i - bpp]);
                    break;
                case 2:
                    for (size_t i = 0; i < row; ++i)
                        cur[i] = static_cast<uint8_t>(cur[i] + prev[i]);
                    break;
                case 3:
                    for (size_t i = 0; i < row; ++i)
                        cur[i] = static_cast<uint8_t>(cur[i] + (((i >= (size_t)bpp ? cur[i - bpp] : 0) + prev[i]) >> 1));
                    break;
                case 4:
                    for (size_t i = 0; i < row; ++i)
                        cur[i] = static_cast<uint8_t>(cur[i] + paeth(i >= (size_t)bpp ? cur[i - bpp] : 0, prev[i], i >= (size_t)bpp ? prev[i - bpp] : 0));
                    break;
                default: bad("bad filter type");
                }
                prev = cur;
            }
        }

        // libpng's colour -> grey weights as cv::imdecode sets them (png_set_rgb_to_gray(.., 0.299, 0.587)): 15-bit
        // integers, the blue weight being what is left of 32768.  8-bit samples are truncated, 16-bit samples rounded.
        constexpr int k_grey_r = 9797, k_grey_g = 19234, k_grey_b = 3737;

        // Writes `count` pixels of one unfiltered row to out[3 * (x0 + i * xstep)].
        void emit_row(const uint8_t* cur, int count, int x0, int xstep, const png_info& info, const chunks& c, int channels,
                      bool grey, uint8_t* out)
        {
            const int step = info.bit_depth == 16 ? 2 : 1; // 16-bit samples: the high byte comes first and is the one kept
            auto put = [&](int i, int b, int g, int r) {
                uint8_t* o = out + 3 * static_cast<size_t>(x0 + i * xstep);
                if (grey && !(b == g && g == r))
                    b = g = r = (k_grey_r * r + k_grey_g * g + k_grey_b * b) >> 15;
                o[0] = static_cast<uint8_t>(b);
                o[1] = static_cast<uint8_t>(g);
                o[2] = static_cast<uint8_t>(r);
            };
            auto put_index = [&](int i, int v) {
                if (v >= c.palette_size)
                    bad("palette index out of range");
                put(i, c.palette[v][2], c.palette[v][1], c.palette[v][0]);
            };
            if (info.color_type == 2 || info.color_type == 6)
            {
                for (int i = 0; i < count; ++i)
                {
                    const uint8_t* s = cur + static_cast<size_t>(i) * channels * step;
                    if (grey && step == 2)
                    {
                        // the conversion runs on the 16-bit samples; the high byte of its result is kept
                        const int r = s[0] << 8 | s[1], g = s[2] << 8 | s[3], b = s[4] << 8 | s[5];
                        const int v = (r == g && g == b) ? r : (int)(((int64_t)k_grey_r * r + (int64_t)k_grey_g * g + (int64_t)k_grey_b * b + 16384) >> 15);
                        uint8_t*  o = out + 3 * static_cast<size_t>(x0 + i * xstep);
                        o[0] = o[1] = o[2] = static_cast<uint8_t>(v >> 8);
                    }
                    else
                        put(i, s[2 * step], s[step], s[0]);
                }
            }
            else if (info.bit_depth >= 8) // grey, grey + alpha, or an 8-bit palette index
            {
                for (int i = 0; i < count; ++i)
                {
                    const uint8_t v = cur[static_cast<size_t>(i) * channels * step];
                    if (info.color_type == 3)
                        put_index(i, v);
                    else
                        put(i, v, v, v);
                }
            }
            else // 1, 2 or 4 bits per sample, most significant first: grey scaled to 0..255, or a palette index
            {
                const int bd = info.bit_depth, mask = (1 << bd) - 1, scale = 255 / mask;
                for (int i = 0; i < count; ++i)
                {
                    const int bit = i * bd;
                    const int v   = (cur[bit >> 3] >> (8 - bd - (bit & 7))) & mask;
                    if (info.color_type == 3)
                        put_index(i, v);
                    else
                        put(i, v * scale, v * scale, v * scale);
                }
            }
        }
    }

    void png_decode_bgr(const void* data, size_t size, const png_info& info, uint8_t* dst, size_t pitch, bool grey)
    {
        const uint8_t* d = static_cast<const uint8_t*>(data);
        chunks         c;
        read_chunks(d, size, c);
        static const int channels_of[7] = {1, 0, 3, 1, 2, 0, 4};
        const int        channels = channels_of[info.color_type];
        const int        bits_pp  = channels * info.bit_depth;            // bits per pixel
        const int        bpp      = std::max(1, bits_pp / 8);             // filter unit in bytes
        if (info.color_type == 3 && c.palette_size == 0)
            bad("palette image without a palette");
        // A plain file is one pass over every pixel; an interlaced (Adam7) file is seven reduced images one after the
        // other in the same zlib stream, each filtered on its own; empty passes take no bytes.
        struct pass
        {
            int x0, y0, dx, dy;
        };
        static const pass adam7[7] = {{0, 0, 8, 8}, {4, 0, 8, 8}, {0, 4, 4, 8}, {2, 0, 4, 4}, {0, 2, 2, 4}, {1, 0, 2, 2}, {0, 1, 1, 2}};
        static const pass whole[1] = {{0, 0, 1, 1}};
        const pass*       passes   = info.interlaced ? adam7 : whole;
        const int         npass    = info.interlaced ? 7 : 1;
        size_t            total    = 0;
        for (int p = 0; p < npass; ++p)
        {
            const int pw = (info.width - passes[p].x0 + passes[p].dx - 1) / passes[p].dx;
            const int ph = (info.height - passes[p].y0 + passes[p].dy - 1) / passes[p].dy;
            if (pw > 0 && ph > 0)
                total += ((static_cast<size_t>(pw) * bits_pp + 7) / 8 + 1) * ph;
        }
        std::vector<uint8_t> raw(total);
        zlib_inflate(c.idat.data(), c.idat.size(), raw.data(), raw.size());
        uint8_t* at = raw.data();
        for (int p = 0; p < npass; ++p)
        {
            const int pw = (info.width - passes[p].x0 + passes[p].dx - 1) / passes[p].dx;
            const int ph = (info.height - passes[p].y0 + passes[p].dy - 1) / passes[p].dy;
            if (pw <= 0 || ph <= 0)
                continue;
            const size_t row = (static_cast<size_t>(pw) * bits_pp + 7) / 8;
            unfilter(at, row, ph, bpp);
            for (int y = 0; y < ph; ++y)
                emit_row(at + static_cast<size_t>(y) * (row + 1) + 1, pw, passes[p].x0, passes[p].dx, info, c, channels, grey,
                         dst + static_cast<size_t>(passes[p].y0 + y * passes[p].dy) * pitch);
            at += (row + 1) * ph;
        }
    }
}

using namespace aeonb;

extern "C" {

int aeonb_png_info(const void* data, size_t size, int32_t* width, int32_t* height)
{
    return guarded([&]() {
        if (!data || !width || !height)
            throw std::invalid_argument("aeonb_png_info: NULL argument");
        png_info info;
        png_parse(data, size, info);
        *width  = info.width;
        *height = info.height;
        return AEONB_OK;
    });
}

int aeonb_png_decode_bgr(const void* data, size_t size, uint8_t* dst, size_t pitch)
{
    return guarded([&]() {
        if (!data || !dst)
            throw std::invalid_argument("aeonb_png_decode_bgr: NULL argument");
        png_info info;
        png_parse(data, size, info);
        if (pitch < (size_t)info.width * 3)
            throw std::invalid_argument("aeonb_png_decode_bgr: pitch smaller than a row");
        png_decode_bgr(data, size, info, dst, pitch);
        return AEONB_OK;
    });
}

int aeonb_png_decode_grey(const void* data, size_t size, uint8_t* dst, size_t pitch)
{
    return guarded([&]() {
        if (!data || !dst)
            throw std::invalid_argument("aeonb_png_decode_grey: NULL argument");
        png_info info;
        png_parse(data, size, info);
        if (pitch < (size_t)info.width)
            throw std::invalid_argument("aeonb_png_decode_grey: pitch smaller than a row");
        const size_t         wide = (size_t)info.width * 3;
        std::vector<uint8_t> bgr(wide * info.height);
        png_decode_bgr(data, size, info, bgr.data(), wide, true);
        for (int y = 0; y < info.height; ++y)
            for (int x = 0; x < info.width; ++x)
                dst[(size_t)y * pitch + x] = bgr[(size_t)y * wide + 3 * (size_t)x];
        return AEONB_OK;
    });
}

} // extern "C"
