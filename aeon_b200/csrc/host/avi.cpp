#include "avi.hpp"

#include <cstring>

namespace aeonb
{
    namespace
    {
        constexpr uint32_t cc(char a, char b, char c, char d)
        {
            return (uint32_t)(uint8_t)a | ((uint32_t)(uint8_t)b << 8) | ((uint32_t)(uint8_t)c << 16) | ((uint32_t)(uint8_t)d << 24);
        }
        struct reader
        {
            const uint8_t* p;
            size_t         n;
            bool     ok(size_t off, size_t len) const { return off <= n && len <= n - off; }
            uint32_t u32(size_t off) const
            {
                uint32_t v;
                std::memcpy(&v, p + off, 4);
                return v;
            }
        };

        uint32_t lower(uint32_t v)
        {
            uint32_t r = 0;
            for (int i = 0; i < 4; ++i)
            {
                uint32_t ch = (v >> (8 * i)) & 0xFF;
                if (ch >= 'A' && ch <= 'Z')
                    ch += 'a' - 'A';
                r |= ch << (8 * i);
            }
            return r;
        }

        // Walks the header list; returns the index of the MJPG video stream or -1.
        int find_mjpeg_stream(const reader& r, size_t begin, size_t end, bool& has_index, int& width, int& height)
        {
            int    stream = -1, found = -1;
            size_t pos = begin;
            while (pos + 8 <= end && r.ok(pos, 8))
            {
                const uint32_t id = r.u32(pos), sz = r.u32(pos + 4);
                const size_t   body = pos + 8;
                if (id == cc('a', 'v', 'i', 'h') && r.ok(body, 40))
                {
                    has_index = (r.u32(body + 12) & 0x10) != 0;
                    width     = (int)r.u32(body + 32);
                    height    = (int)r.u32(body + 36);
                }
                else if (id == cc('L', 'I', 'S', 'T') && r.ok(body, 4) && r.u32(body) == cc('s', 't', 'r', 'l'))
                {
                    ++stream;
                    const size_t sh = body + 4;
                    if (r.ok(sh, 8 + 8) && r.u32(sh) == cc('s', 't', 'r', 'h'))
                    {
                        const uint32_t type = r.u32(sh + 8), handler = r.u32(sh + 12);
                        if (type == cc('v', 'i', 'd', 's') && lower(handler) == cc('m', 'j', 'p', 'g') && found < 0)
                            found = stream;
                    }
                }
                pos = body + sz + (sz & 1);
            }
            return found;
        }
    }

    std::vector<avi_frame> avi_mjpeg_frames(const void* data, size_t size, int* width, int* height)
    {
        std::vector<avi_frame> frames;
        reader                 r{static_cast<const uint8_t*>(data), size};
        size_t                 riff = 0;
        int                    w = 0, h = 0;
        while (r.ok(riff, 12) && r.u32(riff) == cc('R', 'I', 'F', 'F') &&
               (r.u32(riff + 8) == cc('A', 'V', 'I', ' ') || r.u32(riff + 8) == cc('A', 'V', 'I', 'X')))
        {
            const size_t riff_end = std::min(size, riff + 8 + (size_t)r.u32(riff + 4));
            size_t       pos      = riff + 12;
            bool         has_index = false;
            int          stream    = -1;
            size_t       movi_start = 0, movi_end = 0;
            while (pos + 8 <= riff_end)
            {
                const uint32_t id = r.u32(pos), sz = r.u32(pos + 4);
                const size_t   body = pos + 8;
                if (id == cc('L', 'I', 'S', 'T') && r.ok(body, 4))
                {
                    const uint32_t kind = r.u32(body);
                    if (kind == cc('h', 'd', 'r', 'l'))
                        stream = find_mjpeg_stream(r, body + 4, std::min(riff_end, body + sz), has_index, w, h);
                    else if (kind == cc('m', 'o', 'v', 'i'))
                    {
                        movi_start = body; // offsets in idx1 count from the 'movi' tag
                        movi_end   = body + sz;
                    }
                }
                else if (id == cc('i', 'd', 'x', '1') && stream >= 0 && movi_start && has_index)
                {
                    const uint32_t want = cc('0' + (stream / 10) % 10, '0' + stream % 10, 'd', 'c');
                    const size_t   end  = std::min(riff_end, body + sz);
                    for (size_t e = body; e + 16 <= end; e += 16)
                    {
                        if (r.u32(e) != want)
                            continue;
                        const size_t at = movi_start + r.u32(e + 8);
                        if (at >= movi_end || !r.ok(at, 8))
                            continue;
                        const size_t len = r.u32(at + 4); // the chunk's own size field is what gets read
                        if (!r.ok(at + 8, len))
                            continue;
                        frames.push_back(avi_frame{r.p + at + 8, len});
                    }
                }
                pos = body + sz + (sz & 1);
            }
            riff = riff_end + (riff_end & 1);
        }
        if (width)
            *width = w;
        if (height)
            *height = h;
        return frames;
    }
}
