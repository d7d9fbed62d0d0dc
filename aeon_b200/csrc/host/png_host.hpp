// Host decoder for PNG records.
//
// aeon hands every image record to cv::imdecode (src/etl_image.cpp:83-99), which also reads PNG; the reference's
// own geometry tests feed losslessly coded PNG pictures (test/test_image.cpp:135,221-248,466,568,619).  Inflate is a
// serial bit stream, so a PNG is decoded on the worker pool straight into the pinned staging buffer as the
// B,G,R picture IMREAD_COLOR delivers, and the image kernel reads it from the device copy of that buffer.
#pragma once

#include <cstddef>
#include <cstdint>

namespace aeonb
{
    struct png_info
    {
        int width = 0, height = 0;
        int bit_depth = 0;  // 1, 2, 4, 8, 16
        int color_type = 0; // 0 grey, 2 RGB, 3 palette, 4 grey + alpha, 6 RGB + alpha
        bool interlaced = false; // Adam7
    };

    bool is_png(const void* data, size_t size);

    // Reads the IHDR chunk.  Throws aeonb::error(AEONB_ERR_DECODE) on a malformed file.
    void png_parse(const void* data, size_t size, png_info& info);

    // Decodes into dst (height rows of `pitch` bytes, 3 bytes per pixel, B,G,R): what cv::imdecode(IMREAD_COLOR) returns --
    // palette expanded, grey replicated, samples under 8 bits scaled to 8, 16-bit samples cut to their high byte, alpha dropped.
    // With `grey` the three bytes of a pixel all carry the grey value cv::imdecode(IMREAD_GRAYSCALE / IMREAD_ANYDEPTH)
    // returns: libpng's integer colour -> grey conversion (15-bit weights 9797, 19234, 3737 for R, G, B; truncated for 8-bit
    // samples; for 16-bit samples computed on the 16-bit values with rounding, then cut to the high byte).
    void png_decode_bgr(const void* data, size_t size, const png_info& info, uint8_t* dst, size_t pitch, bool grey = false);
}
