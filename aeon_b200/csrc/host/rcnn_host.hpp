// Host side of localization_rcnn (src/etl_localization_rcnn.cpp): configuration, anchor generation, and what follows
// the GPU labelling pass -- anchor sampling, the regression targets of the sampled anchors and the ten output buffers.
#pragma once

#include <cstdint>
#include <random>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/aeon_b200.h"
#include "config.hpp"
#include "params.hpp"

namespace aeonb
{
    struct rcnn_config // localization::rcnn::config (src/etl_localization_rcnn.hpp:96-150)
    {
        int                      rois_per_image = 256;
        int                      height = 0, width = 0;
        int                      base_size      = 16;
        float                    scaling_factor = 1.0f / 16.0f;
        std::vector<float>       ratios{0.5f, 1.f, 2.f};
        std::vector<float>       scales{8.f, 16.f, 32.f};
        float                    negative_overlap    = 0.3f;
        float                    positive_overlap    = 0.7f;
        float                    foreground_fraction = 0.5f;
        int                      max_gt_boxes        = 64;
        std::vector<std::string> class_names;
        std::string              name;
        bool                     deterministic_sampling = false; // params::debug_deterministic (src/augment_image.hpp:118)
        shape_type               shapes[10];
        rcnn_config() = default;
        explicit rcnn_config(json js);
        int total_anchors() const;
        aeonb_rcnn_config abi() const;
    };

    struct box4
    {
        float xmin, ymin, xmax, ymax;
    };

    // anchor::generate (src/etl_localization_rcnn.cpp:434-557)
    std::vector<box4> rcnn_generate_anchors(const aeonb_rcnn_config& cfg);

    // What transformer::transform leaves for the loader, per record.
    struct rcnn_record
    {
        std::vector<bbox> gt_boxes; // boundingbox::transformer::transform_box output
        float             image_scale = 1.f;
        int               im_width = 0, im_height = 0;
    };

    // transformer::sample_anchors (:218-263) on the labels of the GPU pass.  `engine` == nullptr: index order
    // (debug_deterministic); otherwise std::shuffle of the foreground and background lists with that engine.  (The
    // reference shuffles with a thread-local engine seeded from std::random_device, so its choice is not reproducible.)
    std::vector<int> rcnn_sample_anchors(const int8_t* labels, int n_anchors, int rois_per_image, float foreground_fraction,
                                         random_engine_t* engine);

    // loader::load (:340-432) into the ten buffers of one record; the regression targets (compute_targets, :265-300) are
    // formed here for the sampled anchors only, each against the box the GPU pass found best for it.
    void rcnn_load(const rcnn_config& cfg, const std::vector<box4>& anchors, const rcnn_record& rec, const int8_t* labels,
                   const int16_t* best_box, const std::vector<int>& sampled, void* const bufs[10]);
}
