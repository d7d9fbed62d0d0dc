// Motion-JPEG AVI container parsing (host).  Stands in for aeon's AviMjpegStream / MotionJpegCapture
// (src/avi.cpp:145-378, src/cap_mjpeg_decoder.cpp:102-227): the RIFF structure is walked, the video
// stream with an MJPG handler is located, and the `idx1` index yields the byte range of every frame.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

namespace aeonb
{
    struct avi_frame
    {
        const uint8_t* data; // JPEG bytes of the frame; size 0 marks a dropped frame (repeat the previous picture)
        size_t         size;
    };

    // Returns the frames in index order; empty when the buffer is not an indexed MJPEG AVI
    // (aeon then treats the record as undecodable).
    std::vector<avi_frame> avi_mjpeg_frames(const void* data, size_t size, int* width = nullptr, int* height = nullptr);
}
