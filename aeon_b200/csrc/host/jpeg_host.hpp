// Host half of JPEG decoding: marker parsing (always), and a Huffman entropy decoder for baseline and
// progressive streams.
//
// aeon calls cv::imdecode per record (src/etl_image.cpp:83-99, src/cap_mjpeg_decoder.cpp:132-147).
// Baseline scans are normally Huffman-decoded on the GPU; this decoder takes progressive files (whose scans
// revisit the same coefficients), streams with more Huffman tables than the device decoder holds, and
// providers configured with "entropy_decode": "host".  It produces the same quantised
// DCT coefficient blocks, which the GPU back end turns into pixels.  Coefficients of a block
// are written in column-major order (element (row r, column c) at index c*8+r) so that a GPU
// thread that owns one block column reads its eight values with a single 128-bit load.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../../include/aeon_b200.h"

namespace aeonb
{
    struct jpeg_frame
    {
        aeonb_jpeg_info info{};
        uint16_t        quant[3][64]{}; // column-major, per component
        // scan description
        const uint8_t* scan          = nullptr; // first entropy-coded byte
        size_t         scan_size     = 0;
        int            restart_interval = 0;
        int            dc_table[3]{};
        int            ac_table[3]{};
        struct huff
        {
            bool     present = false;
            uint8_t  bits[17]{};
            uint8_t  vals[256]{};
        } dc[4], ac[4];
        // Progressive (SOF2) streams: several scans refine the coefficients; `first_sos` points at the first SOS
        // marker (0xFF 0xDA), the Huffman tables above are those defined before it, `stream_end` ends the file.
        bool           progressive = false;
        const uint8_t* first_sos   = nullptr;
        const uint8_t* stream_end  = nullptr;
        int            comp_id[3]{};
    };

    // Parses the headers up to the first start of scan.  Throws aeonb::error(AEONB_ERR_DECODE) with
    // aeon's message ("Decoding image failed due to invalid data in the image file.") on
    // anything that is not an 8-bit Huffman-coded JPEG (baseline sequential with one interleaved scan, or
    // progressive) with 1 or 3 components.
    void jpeg_parse(const void* data, size_t size, jpeg_frame& frame);

    // A rectangle of MCUs [mx0, mx1) x [my0, my1) to keep.  The bit stream is sequential, so everything
    // before the rectangle's last MCU row is still parsed, but only blocks inside it are stored (as a
    // compact plane of (mx1-mx0)*hs x (my1-my0)*vs blocks per component) and parsing stops after it.
    struct jpeg_roi
    {
        int mx0 = 0, my0 = 0, mx1 = 1 << 30, my1 = 1 << 30;
    };

    // The MCU rectangle covering the pixel box [x0,x1) x [y0,y1) of the picture plus one chroma sample of context.
    jpeg_roi jpeg_roi_for_box(const aeonb_jpeg_info& info, int x0, int y0, int x1, int y1);

    // Entropy-decodes the scan (all scans of a progressive stream: spectral selection and successive approximation,
    // ITU-T T.81 annex G).  Without a region coef[c] must hold info.coef_count[c] int16 values; with
    // one, the compact plane described above.  The planes are fully overwritten (absent coefficients are zero).
    void jpeg_entropy_decode(const jpeg_frame& frame, int16_t* const coef[3], const jpeg_roi* roi = nullptr);

    // Prepares a parsed frame for the device entropy decoder: writes the four Huffman tables the scan uses in
    // DHT form (4 x 272 bytes: DC slot 0, DC slot 1, AC slot 0, AC slot 1) and fills the shape fields of `desc`
    // (ncomp, sampling, table slots, MCU counts, restart interval, scan_size; roi = whole picture).  Pointers are
    // left NULL.  Returns false when the scan refers to more than two DC or two AC tables.
    bool jpeg_entropy_prepare(const jpeg_frame& frame, uint8_t tables[4 * 272], aeonb_entropy_desc& desc);
}
