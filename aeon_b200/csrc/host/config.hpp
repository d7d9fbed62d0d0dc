// ETL configuration blocks with aeon's keys, defaults and validation
// (image: src/etl_image.hpp:56-96, label: src/etl_label.hpp:39-63, video: src/etl_video.hpp:36-65,
// localization_ssd: src/etl_localization_ssd.hpp:49-70; key checking: src/interface.cpp:27-123).
#pragma once

#include <string>
#include <vector>

#include "../../../include/aeon_b200.h"
#include "json.hpp"

namespace aeonb
{
    // aeon output_type (src/typemap.hpp:43-52)
    struct output_type
    {
        std::string name = "uint8_t";
        int         dtype = AEONB_U8; // aeonb_dtype used for the bytes; uint32_t is stored as 32-bit integers
        size_t      size  = 1;
        static bool        is_valid(const std::string& s);
        static output_type from_name(const std::string& s); // throws "Unable to map output type <s>"
    };

    struct shape_type
    {
        std::vector<int64_t>     shape;
        std::vector<std::string> axis_names;
        output_type              otype;
        int64_t element_count() const
        {
            int64_t n = 1;
            for (auto d : shape)
                n *= d;
            return n;
        }
        int64_t byte_size() const { return element_count() * (int64_t)otype.size; }
    };

    // Throws std::invalid_argument("config element {key: value} is not understood[, did you mean 'x']")
    // for a key of `js` that is not in `known`.
    void verify_config(const std::string& location, const std::vector<std::string>& known, const json& js);

    struct image_config
    {
        int         height = 0, width = 0;
        int         channels      = 3;
        bool        channel_major = true;
        bool        bgr_to_rgb    = false;
        std::string output_type_name = "uint8_t";
        std::string name;
        shape_type  shape;
        image_config() = default;
        explicit image_config(json js); // `type` already removed
    };

    struct label_config
    {
        bool        binary = false;
        std::string output_type_name = "uint32_t";
        std::string name;
        shape_type  shape;
        label_config() = default;
        explicit label_config(json js);
    };

    // aeon blob::config (src/etl_blob.hpp:36-63): bytes copied as they are into a buffer of output_count elements
    struct blob_config
    {
        std::string output_type_name = "float";
        int         output_count     = 0;
        std::string name;
        shape_type  shape;
        blob_config() = default;
        explicit blob_config(json js);
    };

    struct video_config
    {
        int          max_frame_count = 0;
        image_config frame;
        std::string  name;
        shape_type   shape;
        video_config() = default;
        explicit video_config(json js);
    };

    struct ssd_config
    {
        int                      height = 0, width = 0;
        int                      max_gt_boxes = 64;
        std::vector<std::string> class_names;
        std::string              name;
        std::vector<shape_type>  shapes; // image_shape, gt_boxes, gt_box_count, gt_class_count, difficult_flag
        ssd_config() = default;
        explicit ssd_config(json js);
    };

    // boundingbox block (src/etl_boundingbox.hpp:39-66): the transformed boxes of a record as max_bbox_count rows of four
    // floats.  The reference declares the buffer as {max_bbox_count, 4 * sizeof(float)} elements of output_type and
    // fills the first max_bbox_count * 4 floats of it; the same shape is kept.
    struct bbox_config
    {
        int                      height = 0, width = 0;
        int                      max_bbox_count = 0;
        std::vector<std::string> class_names;
        std::string              output_type_name = "float";
        std::string              name;
        shape_type               shape;
        bbox_config() = default;
        explicit bbox_config(json js);
    };

    // Spectrogram block.  aeon's snapshot has the specgram routines (src/specgram.cpp) but no provider
    // wired to them; this block names their arguments.
    struct audio_config
    {
        int         frame_length   = 320;
        int         frame_stride   = 160;
        int         max_time_steps = 0; // derived from max_duration_samples when 0
        int         max_samples    = 0;
        int         num_filters    = 64;
        int         sample_rate    = 16000;
        std::string window_type    = "hann";
        std::string feature_type   = "mfsc"; // "specgram" (magnitudes), "mfsc" (log mel) or "mfcc" (DCT of log mel)
        int         num_cepstra    = 40;
        std::string name;
        shape_type  shape;
        audio_config() = default;
        explicit audio_config(json js);
        int window_code() const;
    };
}
