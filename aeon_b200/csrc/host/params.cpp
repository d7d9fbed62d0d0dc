#include "params.hpp"

#include <algorithm>
#include <cctype>
#include <cfloat>
#include <sstream>
#include <stdexcept>

using namespace std;

namespace aeonb
{
    namespace
    {
        const float epsilon = 0.00001f; // aeon src/util.hpp:32

        // Config readers with the narrowing aeon applies (src/interface.hpp:131-161):
        // a distribution is a two-element array converted to the distribution's result type.
        template <typename T>
        void read_scalar(const json& js, const char* key, T& value)
        {
            const json* v = js.find(key);
            if (!v)
                return;
            if constexpr (is_same<T, bool>::value)
                value = v->as_bool();
            else if constexpr (is_same<T, string>::value)
                value = v->as_string();
            else if constexpr (is_floating_point<T>::value)
                value = static_cast<T>(v->as_double());
            else
                value = static_cast<T>(v->as_int());
        }

        void read_vector(const json& js, const char* key, vector<double>& value)
        {
            const json* v = js.find(key);
            if (!v)
                return;
            value.clear();
            for (const json& e : v->elements())
                value.push_back(e.as_double());
        }

        template <typename D>
        bool read_pair(const json& js, const char* key, typename D::result_type& a, typename D::result_type& b)
        {
            const json* v = js.find(key);
            if (!v)
                return false;
            const auto& e = v->elements();
            if (e.size() < 2)
                throw invalid_argument(string("distribution '") + key + "' needs two values");
            using R = typename D::result_type;
            if constexpr (is_floating_point<R>::value)
            {
                a = static_cast<R>(e[0].as_double());
                b = static_cast<R>(e[1].as_double());
            }
            else
            {
                a = static_cast<R>(e[0].as_int());
                b = static_cast<R>(e[1].as_int());
            }
            return true;
        }

        template <typename D, typename Check>
        void read_dist(const json& js, const char* key, D& dist, Check ok)
        {
            typename D::result_type a, b;
            if (!read_pair<D>(js, key, a, b))
                return;
            dist = D{a, b};
            if (!ok(dist))
            {
                stringstream ss;
                ss << "value for '" << key << "' out of range";
                throw invalid_argument(ss.str());
            }
        }

        bool in_unit_range(float x) { return x >= 0.0f - epsilon && x <= 1.0f + epsilon; }
    }

    int unbiased_round(float x)
    {
        float i;
        float fracpart = std::modf(x, &i);
        int   intpart  = int(i);
        int   rc;
        if (std::fabs(fracpart) == 0.5)
        {
            if (intpart % 2 == 0)
                rc = intpart;
            else
            {
                rc = std::fabs(x) + 0.5;
                rc = x < 0.0 ? -rc : rc;
            }
        }
        else
        {
            rc = std::floor(std::fabs(x) + 0.5);
            rc = x < 0.0 ? -rc : rc;
        }
        return rc;
    }

    // ------------------------------------------------------------------------------------------
    // boxes
    // ------------------------------------------------------------------------------------------

    nbox::nbox(float x0, float y0, float x1, float y1) : xmin(x0), ymin(y0), xmax(x1), ymax(y1)
    {
        if (!(in_unit_range(xmin) && in_unit_range(xmax) && in_unit_range(ymin) && in_unit_range(ymax)))
        {
            stringstream ss;
            ss << "bounding box '[" << xmax - xmin << " x " << ymax - ymin << " from (" << xmin << ", " << ymin
               << ")]' is not properly normalized";
            throw invalid_argument(ss.str());
        }
    }

    nbox nbox::intersect(const nbox& o) const
    {
        if (o.xmin > xmax || o.xmax < xmin || o.ymin > ymax || o.ymax < ymin)
            return nbox();
        return nbox(max(xmin, o.xmin), max(ymin, o.ymin), min(xmax, o.xmax), min(ymax, o.ymax));
    }

    float nbox::jaccard_overlap(const nbox& o) const
    {
        float inter = intersect(o).size();
        float a     = size();
        float b     = o.size();
        if (inter == 0.f)
            return 0.f;
        return inter / (a + b - inter);
    }

    float nbox::coverage(const nbox& o) const
    {
        float inter = intersect(o).size();
        if (inter > 0)
            return inter / size();
        return 0.;
    }

    bbox bbox_expand(const bbox& b, size2i offset, size2i size, float)
    {
        if (b.xmax + offset.width > size.width || b.ymax + offset.height > size.height)
        {
            stringstream ss;
            ss << "Invalid parameters to expand boundingbox: expand_offset (" << offset.width << "," << offset.height
               << ") expand_size (" << size.width << "," << size.height << ")";
            throw invalid_argument(ss.str());
        }
        bbox rc = b;
        rc.xmin += offset.width;
        rc.ymin += offset.height;
        rc.xmax += offset.width;
        rc.ymax += offset.height;
        return rc;
    }

    nbox bbox_normalize(const bbox& b, float width, float height)
    {
        return nbox(b.xmin / width, b.ymin / height, (b.xmax + 1) / width, (b.ymax + 1) / height);
    }

    bbox bbox_intersect(const bbox& a, const bbox& b)
    {
        if (b.xmin > a.xmax || b.xmax < a.xmin || b.ymin > a.ymax || b.ymax < a.ymin)
            return bbox();
        bbox i;
        i.xmin = max(a.xmin, b.xmin);
        i.ymin = max(a.ymin, b.ymin);
        i.xmax = min(a.xmax, b.xmax);
        i.ymax = min(a.ymax, b.ymax);
        return i;
    }

    float bbox_jaccard(const bbox& a, const bbox& b)
    {
        const float inter = bbox_intersect(a, b).size();
        if (inter == 0.f)
            return 0.f;
        return inter / (a.size() + b.size() - inter);
    }

    float bbox_coverage(const bbox& a, const bbox& b)
    {
        const float inter = bbox_intersect(a, b).size();
        return inter > 0 ? inter / a.size() : 0.f;
    }

    void ssd_fill_buffers(const vector<bbox>& gt, int width, int height, int max_gt_boxes, int32_t* image_shape, float* gt_boxes,
                          int32_t* gt_box_count, int32_t* gt_class, int32_t* gt_difficult)
    {
        image_shape[0] = width;
        image_shape[1] = height;
        *gt_box_count  = std::min<int>(max_gt_boxes, (int)gt.size());
        for (int i = 0; i < *gt_box_count; ++i)
        {
            const nbox nb = bbox_normalize(gt[i], width, height);
            gt_boxes[4 * i + 0] = nb.xmin;
            gt_boxes[4 * i + 1] = nb.ymin;
            gt_boxes[4 * i + 2] = nb.xmax;
            gt_boxes[4 * i + 3] = nb.ymax;
            gt_class[i]         = gt[i].label;
            gt_difficult[i]     = gt[i].difficult;
        }
    }

    // ------------------------------------------------------------------------------------------
    // crop-box helpers
    // ------------------------------------------------------------------------------------------

    size2i get_resized_short_size(size_t in_width, size_t in_height, size_t target_size)
    {
        auto percent = static_cast<float>(target_size) / min(in_height, in_width);
        return size2i{static_cast<int>(round(in_width * percent)), static_cast<int>(round(in_height * percent))};
    }

    float calculate_scale(int width, int height, int output_width, int output_height)
    {
        float im_scale = (float)output_width / (float)width;
        float h        = (float)height * im_scale;
        if (h > output_height)
            im_scale = (float)output_height / (float)height;
        return im_scale;
    }

    void cropbox_max_proportional(float in_w, float in_h, float out_w, float out_h, float& w, float& h)
    {
        float scale = in_w / out_w;
        w           = out_w * scale;
        h           = out_h * scale;
        if (h > in_h)
        {
            scale = in_h / h;
            w     = w * scale;
            h     = h * scale;
        }
    }

    void cropbox_area_scale(float in_w, float in_h, float& w, float& h, float scale)
    {
        float in_area    = in_w * in_h;
        float crop_area  = w * h;
        float size_ratio = crop_area / in_area;
        if (size_ratio > scale)
        {
            float crop_aspect_ratio = w / h;
            crop_area               = in_area * scale;
            float w2                = crop_area * crop_aspect_ratio;
            float width             = sqrt(w2);
            float height            = crop_area / width;
            w                       = width;
            h                       = height;
        }
    }

    void cropbox_shift(float in_w, float in_h, float crop_w, float crop_h, float xoff, float yoff, int& x, int& y)
    {
        x = (in_w - crop_w) * xoff;
        y = (in_h - crop_h) * yoff;
    }

    // ------------------------------------------------------------------------------------------
    // SSD patch sampling
    // ------------------------------------------------------------------------------------------

    patch_sampler::patch_sampler(const json& cfg)
    {
        if (cfg.is_null())
            return;
        read_dist(cfg, "scale", m_scale, [](decltype(m_scale) v) { return v.a() <= v.b() && v.a() > 0. && v.b() <= 1.; });
        read_dist(cfg, "aspect_ratio", m_aspect_ratio,
                  [](decltype(m_aspect_ratio) v) { return v.a() <= v.b() && v.a() > 0. && v.b() < FLT_MAX; });
    }

    nbox patch_sampler::sample_patch(random_engine_t& random) const
    {
        float scale            = m_scale(random);
        float min_aspect_ratio = max<float>(m_aspect_ratio.min(), pow(scale, 2.));
        float max_aspect_ratio = min<float>(m_aspect_ratio.max(), 1 / pow(scale, 2.));
        auto  local            = uniform_real_distribution<float>(min_aspect_ratio, max_aspect_ratio);
        float aspect_ratio     = local(random);

        float bbox_width  = scale * sqrt(aspect_ratio);
        float bbox_height = scale / sqrt(aspect_ratio);

        uniform_real_distribution<float> width_generator(0.f, 1.f - bbox_width);
        uniform_real_distribution<float> height_generator(0.f, 1.f - bbox_height);
        float                            w_off = width_generator(random);
        float                            h_off = height_generator(random);
        return nbox(w_off, h_off, w_off + bbox_width, h_off + bbox_height);
    }

    sample_constraint::sample_constraint(const json& cfg)
    {
        if (cfg.is_null())
            return;
        read_scalar(cfg, "min_jaccard_overlap", min_jaccard_overlap);
        read_scalar(cfg, "max_jaccard_overlap", max_jaccard_overlap);
        read_scalar(cfg, "min_sample_coverage", min_sample_coverage);
        read_scalar(cfg, "max_sample_coverage", max_sample_coverage);
        read_scalar(cfg, "min_object_coverage", min_object_coverage);
        read_scalar(cfg, "max_object_coverage", max_object_coverage);
    }

    bool sample_constraint::satisfies(const nbox& sampled, const vector<nbox>& objects) const
    {
        auto has = [](float v) { return !std::isnan(v); };
        bool has_jaccard = has(min_jaccard_overlap) || has(max_jaccard_overlap);
        bool has_sample  = has(min_sample_coverage) || has(max_sample_coverage);
        bool has_object  = has(min_object_coverage) || has(max_object_coverage);
        if (!has_jaccard && !has_sample && !has_object)
            return true;
        bool found = false;
        for (const nbox& object : objects)
        {
            if (has_jaccard)
            {
                const float v = sampled.jaccard_overlap(object);
                if (has(min_jaccard_overlap) && v < min_jaccard_overlap)
                    continue;
                if (has(max_jaccard_overlap) && v > max_jaccard_overlap)
                    continue;
                found = true;
            }
            if (has_sample)
            {
                const float v = sampled.coverage(object);
                if (has(min_sample_coverage) && v < min_sample_coverage)
                    continue;
                if (has(max_sample_coverage) && v > max_sample_coverage)
                    continue;
                found = true;
            }
            if (has_object)
            {
                const float v = object.coverage(sampled);
                if (has(min_object_coverage) && v < min_object_coverage)
                    continue;
                if (has(max_object_coverage) && v > max_object_coverage)
                    continue;
                found = true;
            }
            if (found)
                return true;
        }
        return found;
    }

    batch_sampler::batch_sampler(const json& cfg)
    {
        if (cfg.is_null())
            return;
        read_scalar(cfg, "max_sample", m_max_sample);
        if (cfg.contains("max_sample") && m_max_sample < 0)
            throw invalid_argument("value for 'max_sample' out of range");
        read_scalar(cfg, "max_trials", m_max_trials);
        if (const json* s = cfg.find("sampler"))
            if (!s->is_null())
                m_sampler = patch_sampler(*s);
        if (const json* c = cfg.find("sample_constraint"))
            if (!c->is_null())
                m_constraint = sample_constraint(*c);
    }

    void batch_sampler::sample_patches(random_engine_t& random, const vector<nbox>& objects, vector<nbox>& out) const
    {
        int found = 0;
        for (unsigned i = 0; i < m_max_trials; ++i)
        {
            if (m_max_sample != -1 && found >= m_max_sample)
                break;
            nbox sampled = m_sampler.sample_patch(random);
            if (m_constraint.satisfies(sampled, objects))
            {
                ++found;
                out.push_back(sampled);
            }
        }
    }

    // ------------------------------------------------------------------------------------------
    // param_factory
    // ------------------------------------------------------------------------------------------

    param_factory::param_factory(const json& cfg)
    {
        if (cfg.is_null())
            return;
        const json* type = cfg.find("type");
        if (!type)
            throw invalid_argument("augmentation missing 'type'");
        if (type->as_string() != "image")
            return; // the reference silently ignores other augmentation types (src/augment_image.cpp:44)

        // Unknown keys are accepted, as in the reference where the key check is disabled.
        read_dist(cfg, "scale", scale, [](const uniform_real_distribution<float>& v) {
            return v.a() >= 0 && v.a() <= 1 && v.b() >= 0 && v.b() <= 1 && v.a() <= v.b();
        });
        read_dist(cfg, "angle", angle, [](decltype(angle) v) { return v.a() <= v.b(); });
        {
            float a, b;
            if (read_pair<normal_distribution<float>>(cfg, "lighting", a, b))
                lighting = normal_distribution<float>{a, b};
        }
        read_dist(cfg, "horizontal_distortion", horizontal_distortion, [](decltype(horizontal_distortion) v) { return v.a() <= v.b(); });
        read_scalar(cfg, "flip_enable", flip_enable);
        read_scalar(cfg, "center", center);
        read_scalar(cfg, "resize_short_size", resize_short_size);
        read_scalar(cfg, "interpolation_method", interpolation_method);
        read_scalar(cfg, "do_area_scale", do_area_scale);
        read_scalar(cfg, "crop_enable", crop_enable);
        read_scalar(cfg, "expand_probability", expand_probability);
        read_scalar(cfg, "emit_constraint_type", emit_constraint_type_name);
        read_scalar(cfg, "emit_constraint_min_overlap", emit_constraint_min_overlap);
        read_scalar(cfg, "fixed_aspect_ratio", fixed_aspect_ratio);
        read_vector(cfg, "mean", mean);
        read_vector(cfg, "stddev", stddev);
        read_scalar(cfg, "fixed_scaling_factor", fixed_scaling_factor);
        read_scalar(cfg, "padding", padding);
        read_scalar(cfg, "debug_output_directory", debug_output_directory);
        read_dist(cfg, "contrast", contrast, [](decltype(contrast) v) { return v.a() <= v.b(); });
        read_dist(cfg, "brightness", brightness, [](decltype(brightness) v) { return v.a() <= v.b(); });
        read_dist(cfg, "saturation", saturation, [](decltype(saturation) v) { return v.a() <= v.b(); });
        read_dist(cfg, "expand_ratio", expand_ratio, [](decltype(expand_ratio) v) { return v.a() >= 1 && v.a() <= v.b(); });
        read_dist(cfg, "hue", hue, [](decltype(hue) v) { return v.a() <= v.b(); });

        if (const json* bs = cfg.find("batch_samplers"))
            for (const json& j : bs->elements())
                m_batch_samplers.push_back(j.is_null() ? batch_sampler() : batch_sampler(j));

        if (crop_enable && !m_batch_samplers.empty())
            throw invalid_argument("'Cannot use 'batch_samplers' with 'crop_enable'. Please use only one cropping method in augmentations.");

        if (flip_enable)
            flip_distribution = bernoulli_distribution{0.5};
        if (!center)
            crop_offset = uniform_real_distribution<float>{0.0f, 1.0f};
        if (padding > 0)
            padding_crop_offset_distribution = uniform_int_distribution<int>(0, padding * 2);

        string e = emit_constraint_type_name;
        transform(e.begin(), e.end(), e.begin(), ::tolower);
        if (e == "center")
            emit = emit_type::center;
        else if (e == "min_overlap")
            emit = emit_type::min_overlap;
        else if (e == "")
            emit = emit_type::undefined;
        else
            throw invalid_argument("Invalid emit constraint type");
    }

    image_params param_factory::make_params(random_engine_t& random, size_t input_width, size_t input_height,
                                            size_t output_width, size_t output_height) const
    {
        image_params settings;
        settings.output_size = size2i{(int)output_width, (int)output_height};

        // Draw order is part of the contract: angle, flip, hue, contrast, brightness, saturation.
        settings.angle                = angle(random);
        settings.flip                 = flip_distribution(random);
        settings.hue                  = hue(random);
        settings.contrast             = contrast(random);
        settings.brightness           = brightness(random);
        settings.saturation           = saturation(random);
        settings.padding              = padding;
        settings.resize_short_size    = resize_short_size;
        settings.interpolation_method = interpolation_method;

        float in_w = (float)(int)input_width;
        float in_h = (float)(int)input_height;

        if (!crop_enable)
        {
            int c_off_x                  = padding_crop_offset_distribution(random);
            int c_off_y                  = padding_crop_offset_distribution(random);
            settings.padding_crop_offset = size2i{c_off_x, c_off_y};
            settings.cropbox             = recti{0, 0, cv_round(in_w), cv_round(in_h)};

            float image_scale;
            if (fixed_scaling_factor > 0)
                image_scale = fixed_scaling_factor;
            else
                image_scale = calculate_scale(cv_round(in_w), cv_round(in_h), (int)output_width, (int)output_height);
            in_w = in_w * image_scale;
            in_h = in_h * image_scale;

            settings.output_size.width  = unbiased_round(in_w);
            settings.output_size.height = unbiased_round(in_h);
        }
        else if (do_area_scale)
        {
            float hd = horizontal_distortion(random);
            hd       = sqrt(hd);
            float out_w = hd, out_h = 1 / hd;

            float bound = min((float)input_width / input_height / (out_w * out_w),
                              (float)input_height / input_width / (out_h * out_h));

            float scale_max = std::min(scale.max(), bound);
            float scale_min = std::min(scale.min(), bound);

            std::uniform_real_distribution<float> scale2{scale_min, scale_max};

            float target_area = sqrt(input_height * input_width * scale2(random));
            out_w *= target_area;
            out_h *= target_area;

            float c_off_x = crop_offset(random);
            float c_off_y = crop_offset(random);

            int x, y;
            cropbox_shift(in_w, in_h, out_w, out_h, c_off_x, c_off_y, x, y);
            settings.cropbox = recti{x, y, cv_round(out_w), cv_round(out_h)};
        }
        else
        {
            if (padding > 0)
                throw invalid_argument("crop_enable should not be true: when padding is defined, crop is executed by "
                                       "default with cropbox size equal to intput image size");
            float image_scale = scale(random);
            float hd          = horizontal_distortion(random);
            float out_w = output_width * hd, out_h = output_height;

            if (resize_short_size > 0)
            {
                size2i s = get_resized_short_size(input_width, input_height, resize_short_size);
                in_w     = s.width;
                in_h     = s.height;
            }

            float cw, ch;
            cropbox_max_proportional(in_w, in_h, out_w, out_h, cw, ch);
            // do_area_scale is false on this branch, so the crop box scales linearly.
            cw = cw * image_scale;
            ch = ch * image_scale;

            float c_off_x = crop_offset(random);
            float c_off_y = crop_offset(random);

            int x, y;
            cropbox_shift(in_w, in_h, cw, ch, c_off_x, c_off_y, x, y);
            settings.cropbox = recti{x, y, cv_round(cw), cv_round(ch)};
        }

        if (lighting.stddev() != 0)
        {
            for (int i = 0; i < 3; i++)
                settings.lighting.push_back(lighting(random));
            settings.color_noise_std = lighting.stddev();
        }
        return settings;
    }

    image_params param_factory::make_ssd_params(random_engine_t& random, size_t input_width, size_t input_height,
                                                size_t output_width, size_t output_height,
                                                const vector<bbox>& object_bboxes) const
    {
        image_params settings         = make_params(random, input_width, input_height, output_width, output_height);
        settings.emit_min_overlap     = emit_constraint_min_overlap;
        settings.emit_constraint_type = emit;
        settings.output_size          = size2i{(int)output_width, (int)output_height}; // warp to the full output

        settings.expand_ratio = expand_ratio(random);
        bool expand_enabled   = expand_distribution(random) < expand_probability;

        if (settings.expand_ratio < 1.)
            throw invalid_argument("Expand ratio must be greater than 1.");
        if (expand_enabled)
        {
            float expand_width    = settings.expand_ratio * input_width;
            float expand_height   = settings.expand_ratio * input_height;
            settings.expand_size  = size2i{(int)floor(expand_width), (int)floor(expand_height)};
            float max_w_off       = expand_width - input_width;
            float max_h_off       = expand_height - input_height;
            float w_off           = expand_distribution(random) * max_w_off;
            float h_off           = expand_distribution(random) * max_h_off;
            settings.expand_offset = size2i{(int)floor(w_off), (int)floor(h_off)};
        }
        else
        {
            settings.expand_ratio  = 1.0;
            settings.expand_offset = size2i{0, 0};
            settings.expand_size   = size2i{(int)input_width, (int)input_height};
        }

        vector<nbox> normalized(object_bboxes.size());
        for (size_t i = 0; i < object_bboxes.size(); i++)
        {
            bbox e        = bbox_expand(object_bboxes[i], settings.expand_offset, settings.expand_size, settings.expand_ratio);
            normalized[i] = bbox_normalize(e, settings.expand_size.width, settings.expand_size.height);
        }
        if (!crop_enable)
        {
            nbox patch       = sample_patch(random, normalized);
            settings.cropbox = patch.unnormalize(settings.expand_size.width, settings.expand_size.height).rect();
        }
        return settings;
    }

    nbox param_factory::sample_patch(random_engine_t& random, const vector<nbox>& objects) const
    {
        vector<nbox> samples;
        for (const batch_sampler& s : m_batch_samplers)
            s.sample_patches(random, objects, samples);
        if (samples.empty())
            return nbox(0, 0, 1, 1);
        uniform_int_distribution<int> pick(0, samples.size() - 1);
        return samples[pick(random)];
    }
}
