// Host-side augmentation parameter factory.
//
// Mirrors aeon's augment::image::param_factory (src/augment_image.hpp:141-246,
// src/augment_image.cpp:27-331): it parses the "augmentation" JSON block with the
// same keys, defaults and checks, and draws the per-record random parameters from a
// std::minstd_rand0 engine with the same <random> distribution classes in the same
// order, so that a record gets the crop box, flip and photometric parameters the
// reference would give it for the same seed.  The draws stay on the host; only the
// resulting plain numbers travel to the GPU.
#pragma once

#include <cmath>
#include <limits>
#include <random>
#include <string>
#include <vector>

#include "json.hpp"

namespace aeonb
{
    using random_engine_t = std::minstd_rand0; // aeon src/util.hpp:146

    struct size2i
    {
        int width = 0, height = 0;
    };
    struct recti
    {
        int x = 0, y = 0, width = 0, height = 0;
    };

    // OpenCV's float->int conversion (cvRound): nearest, ties to even.
    inline int cv_round(float v) { return static_cast<int>(std::lrintf(v)); }
    inline int cv_round(double v) { return static_cast<int>(std::lrint(v)); }

    // aeon src/util.cpp:212-239
    int unbiased_round(float x);

    enum class emit_type
    {
        center,
        min_overlap,
        undefined
    };

    // Pixel-space box with inclusive max corner (aeon src/box.hpp, src/boundingbox.hpp).
    struct bbox
    {
        float xmin = 0, ymin = 0, xmax = -1, ymax = -1;
        int   label     = 0;
        bool  difficult = false;
        bool  truncated = false;
        float width() const { return xmax - xmin + 1; }
        float height() const { return ymax - ymin + 1; }
        float xcenter() const { return xmin + (xmax - xmin) / 2.; }
        float ycenter() const { return ymin + (ymax - ymin) / 2.; }
        float size() const { return (xmax < xmin || ymax < ymin) ? 0.0f : width() * height(); }
        recti rect() const
        {
            return recti{(int)std::round(xmin), (int)std::round(ymin), (int)std::round(width()), (int)std::round(height())};
        }
    };

    // Box in [0,1] coordinates with exclusive max corner (aeon src/normalized_box.hpp).
    struct nbox
    {
        float xmin = 0, ymin = 0, xmax = 0, ymax = 0;
        nbox() = default;
        nbox(float x0, float y0, float x1, float y1); // throws when not within [0,1] (with epsilon)
        float width() const { return xmax - xmin; }
        float height() const { return ymax - ymin; }
        float size() const { return (xmax < xmin || ymax < ymin) ? 0.0f : width() * height(); }
        nbox  intersect(const nbox& o) const;
        float jaccard_overlap(const nbox& o) const;
        float coverage(const nbox& o) const;
        bbox  unnormalize(float w, float h) const { return bbox{xmin * w, ymin * h, xmax * w - 1, ymax * h - 1}; }
    };

    // Field-for-field counterpart of aeon's augment::image::params (src/augment_image.hpp:69-123).
    struct image_params
    {
        float              expand_ratio = 1.0f;
        size2i             expand_offset;
        size2i             expand_size;
        emit_type          emit_constraint_type = emit_type::undefined;
        float              emit_min_overlap     = 0.f;
        recti              cropbox;
        int                resize_short_size    = 0;
        std::string        interpolation_method = "LINEAR";
        size2i             output_size;
        int                angle   = 0;
        bool               flip    = false;
        int                padding = 0;
        size2i             padding_crop_offset;
        std::vector<float> lighting;
        float              color_noise_std = 0;
        float              contrast        = 1.0f;
        float              brightness      = 1.0f;
        float              saturation      = 1.0f;
        int                hue             = 0;
    };

    class patch_sampler // aeon augment::image::sampler
    {
    public:
        patch_sampler() = default;
        explicit patch_sampler(const json& cfg);
        nbox sample_patch(random_engine_t& random) const;

    private:
        mutable std::uniform_real_distribution<float> m_scale{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> m_aspect_ratio{1.0f, 1.0f};
    };

    class sample_constraint
    {
    public:
        sample_constraint() = default;
        explicit sample_constraint(const json& cfg);
        bool satisfies(const nbox& sampled, const std::vector<nbox>& objects) const;

    private:
        static constexpr float unset = std::numeric_limits<float>::quiet_NaN();
        float min_jaccard_overlap = unset, max_jaccard_overlap = unset;
        float min_sample_coverage = unset, max_sample_coverage = unset;
        float min_object_coverage = unset, max_object_coverage = unset;
    };

    class batch_sampler
    {
    public:
        batch_sampler() = default;
        explicit batch_sampler(const json& cfg);
        void sample_patches(random_engine_t& random, const std::vector<nbox>& objects, std::vector<nbox>& out) const;

    private:
        int               m_max_sample = -1;
        unsigned          m_max_trials = 100;
        patch_sampler     m_sampler;
        sample_constraint m_constraint;
    };

    class param_factory
    {
    public:
        param_factory() = default;
        explicit param_factory(const json& cfg); // null => all defaults (aeon accepts a missing block)

        // src/augment_image.cpp:107-230.  `random` is the engine of the record's decode slot.
        image_params make_params(random_engine_t& random, size_t input_width, size_t input_height, size_t output_width,
                                 size_t output_height) const;
        // src/augment_image.cpp:232-310
        image_params make_ssd_params(random_engine_t& random, size_t input_width, size_t input_height, size_t output_width,
                                     size_t output_height, const std::vector<bbox>& object_bboxes) const;

        bool                do_area_scale        = false;
        bool                crop_enable          = true;
        bool                fixed_aspect_ratio   = false;
        std::vector<double> mean;
        std::vector<double> stddev;
        int                 resize_short_size    = 0;
        std::string         interpolation_method = "LINEAR";
        float               expand_probability   = 0.f;
        float               fixed_scaling_factor = -1;
        std::string         emit_constraint_type_name;
        float               emit_constraint_min_overlap = 0.f;
        int                 padding                     = 0;
        std::string         debug_output_directory;
        bool                flip_enable = false;
        bool                center      = true;
        emit_type           emit        = emit_type::undefined;

        // Distributions are mutable members exactly as in the reference: std::normal_distribution
        // keeps a saved second variate, so lighting draws carry over from one record to the next.
        mutable std::uniform_real_distribution<float> scale{1.0f, 1.0f};
        mutable std::uniform_int_distribution<int>    angle{0, 0};
        mutable std::normal_distribution<float>       lighting{0.0f, 0.0f};
        mutable std::uniform_real_distribution<float> horizontal_distortion{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> contrast{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> brightness{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> saturation{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> expand_ratio{1.0f, 1.0f};
        mutable std::uniform_real_distribution<float> expand_distribution{0.0f, 1.0f};
        mutable std::uniform_int_distribution<int>    hue{0, 0};
        mutable std::uniform_real_distribution<float> crop_offset{0.5f, 0.5f};
        mutable std::bernoulli_distribution           flip_distribution{0};
        mutable std::uniform_int_distribution<int>    padding_crop_offset_distribution{0, 0};

    private:
        nbox sample_patch(random_engine_t& random, const std::vector<nbox>& objects) const;
        std::vector<batch_sampler> m_batch_samplers;
    };

    // Crop-box helpers of aeon src/image.cpp:108-116,214-273 (all float32 arithmetic).
    size2i get_resized_short_size(size_t in_width, size_t in_height, size_t target_size);
    float  calculate_scale(int width, int height, int output_width, int output_height);
    void   cropbox_max_proportional(float in_w, float in_h, float out_w, float out_h, float& w, float& h);
    void   cropbox_area_scale(float in_w, float in_h, float& w, float& h, float scale);
    void   cropbox_shift(float in_w, float in_h, float crop_w, float crop_h, float xoff, float yoff, int& x, int& y);

    // Box transforms used by the SSD path (aeon src/boundingbox.cpp:78-163).
    bbox bbox_expand(const bbox& b, size2i offset, size2i size, float ratio);
    nbox bbox_normalize(const bbox& b, float width, float height);
    // aeon boundingbox::box::intersect / jaccard_overlap / coverage (src/boundingbox.cpp:105-148); an empty
    // intersection is the default box (0, 0, -1, -1)
    bbox  bbox_intersect(const bbox& a, const bbox& b);
    float bbox_jaccard(const bbox& a, const bbox& b);
    float bbox_coverage(const bbox& a, const bbox& b);
    // aeon boundingbox::transformer::transform_box for every box of a record (src/etl_boundingbox.cpp:146-261):
    // expand shift, emit constraint, clip to the crop box, flip, rescale to the output size
    std::vector<bbox> transform_boxes_for_ssd(const std::vector<bbox>& boxes, const image_params& p);
    // aeon localization::ssd::loader::load (src/etl_localization_ssd.cpp:116-149): the five buffers of one record
    void ssd_fill_buffers(const std::vector<bbox>& gt, int width, int height, int max_gt_boxes, int32_t* image_shape, float* gt_boxes,
                          int32_t* gt_box_count, int32_t* gt_class, int32_t* gt_difficult);
}
