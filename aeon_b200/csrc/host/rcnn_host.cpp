#include "rcnn_host.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

#include "../context.hpp"

namespace aeonb
{
    namespace
    {
        // box::width / height and xcenter / ycenter (src/box.hpp:51-52,92-93)
        float extent(float lo, float hi) { return hi - lo + 1; }
        float centre(float lo, float hi) { return lo + (hi - lo) / 2.; }

        // anchor::mkanchors (src/etl_localization_rcnn.cpp:508-522): the half extents are formed in double
        std::vector<box4> mkanchors(const std::vector<float>& ws, const std::vector<float>& hs, float x_ctr, float y_ctr)
        {
            std::vector<box4> rc;
            for (size_t i = 0; i < ws.size(); ++i)
                rc.push_back(box4{(float)(x_ctr - 0.5 * (ws[i] - 1)), (float)(y_ctr - 0.5 * (hs[i] - 1)), (float)(x_ctr + 0.5 * (ws[i] - 1)),
                                  (float)(y_ctr + 0.5 * (hs[i] - 1))});
            return rc;
        }

        // anchor::ratio_enum (:524-545): the area is cut to an int, widths and heights are rounded half away from zero
        std::vector<box4> ratio_enum(const box4& a, const float* ratios, int n)
        {
            const int          size = (int)(extent(a.xmin, a.xmax) * extent(a.ymin, a.ymax));
            std::vector<float> ws, hs;
            for (int i = 0; i < n; ++i)
                ws.push_back(std::round(std::sqrt((float)size / ratios[i])));
            for (int i = 0; i < n; ++i)
                hs.push_back(std::round(ws[i] * ratios[i]));
            return mkanchors(ws, hs, centre(a.xmin, a.xmax), centre(a.ymin, a.ymax));
        }

        // anchor::scale_enum (:547-557)
        std::vector<box4> scale_enum(const box4& a, const float* scales, int n)
        {
            std::vector<float> ws, hs;
            for (int i = 0; i < n; ++i)
            {
                ws.push_back(extent(a.xmin, a.xmax) * scales[i]);
                hs.push_back(extent(a.ymin, a.ymax) * scales[i]);
            }
            return mkanchors(ws, hs, centre(a.xmin, a.xmax), centre(a.ymin, a.ymax));
        }

        void check(const aeonb_rcnn_config& c)
        {
            if (c.width <= 0 || c.height <= 0 || c.base_size <= 0 || !(c.scaling_factor > 0) || c.n_ratios < 1 || c.n_ratios > 8 ||
                c.n_scales < 1 || c.n_scales > 8)
                throw std::invalid_argument("rcnn configuration: positive sizes and scaling factor, 1..8 ratios and scales");
        }
    }

    std::vector<box4> rcnn_generate_anchors(const aeonb_rcnn_config& c)
    {
        check(c);
        const int conv_x = (int)std::floor((float)c.width * c.scaling_factor);
        const int conv_y = (int)std::floor((float)c.height * c.scaling_factor);
        std::vector<box4> base;
        for (const box4& r : ratio_enum(box4{0.f, 0.f, (float)(c.base_size - 1), (float)(c.base_size - 1)}, c.ratios, c.n_ratios))
            for (const box4& b : scale_enum(r, c.scales, c.n_scales))
                base.push_back(b);
        // the feature stride 1 / scaling_factor, applied in double to a float index (:445-452)
        std::vector<float> sx, sy;
        for (float i = 0; i < conv_x; i++)
            sx.push_back((float)(i * 1. / c.scaling_factor));
        for (float i = 0; i < conv_y; i++)
            sy.push_back((float)(i * 1. / c.scaling_factor));
        std::vector<box4> all;
        all.reserve(base.size() * sx.size() * sy.size());
        for (const box4& a : base)
            for (float y : sy)
                for (float x : sx)
                    all.push_back(box4{x + a.xmin, y + a.ymin, x + a.xmax, y + a.ymax});
        return all;
    }

    std::vector<int> rcnn_sample_anchors(const int8_t* labels, int n_anchors, int rois_per_image, float foreground_fraction,
                                         random_engine_t* engine)
    {
        const int        num_fg = (int)(foreground_fraction * (float)rois_per_image);
        std::vector<int> fg, bg;
        for (int i = 0; i < n_anchors; ++i)
        {
            if (labels[i] >= 1)
                fg.push_back(i);
            else if (labels[i] == 0)
                bg.push_back(i);
        }
        if (engine)
        {
            std::shuffle(fg.begin(), fg.end(), *engine);
            std::shuffle(bg.begin(), bg.end(), *engine);
        }
        if ((int)fg.size() > num_fg)
            fg.resize(num_fg);
        const int remainder = rois_per_image - (int)fg.size();
        if ((int)bg.size() > remainder)
            bg.resize(remainder);
        fg.insert(fg.end(), bg.begin(), bg.end());
        return fg;
    }

    void rcnn_load(const rcnn_config& cfg, const std::vector<box4>& anchors, const rcnn_record& rec, const int8_t* labels,
                   const int16_t* best_box, const std::vector<int>& sampled, void* const bufs[10])
    {
        const size_t A = anchors.size();
        float*   bbtargets      = static_cast<float*>(bufs[0]);
        float*   bbtargets_mask = static_cast<float*>(bufs[1]);
        int32_t* labels_flat    = static_cast<int32_t*>(bufs[2]);
        int32_t* labels_mask    = static_cast<int32_t*>(bufs[3]);
        int32_t* im_shape       = static_cast<int32_t*>(bufs[4]);
        float*   gt_boxes       = static_cast<float*>(bufs[5]);
        int32_t* num_gt_boxes   = static_cast<int32_t*>(bufs[6]);
        int32_t* gt_classes     = static_cast<int32_t*>(bufs[7]);
        float*   im_scale       = static_cast<float*>(bufs[8]);
        int32_t* gt_difficult   = static_cast<int32_t*>(bufs[9]);
        std::memset(bbtargets, 0, 4 * A * sizeof(float));
        std::memset(bbtargets_mask, 0, 4 * A * sizeof(float));
        std::fill(labels_flat, labels_flat + A, 1);
        std::fill(labels_flat + A, labels_flat + 2 * A, 0);
        std::memset(labels_mask, 0, 2 * A * sizeof(int32_t));
        for (int index : sampled)
        {
            if (labels[index] == 1)
            {
                labels_flat[index]     = 0;
                labels_flat[index + A] = 1;
                for (int k = 0; k < 4; ++k)
                    bbtargets_mask[index + A * k] = 1.f;
            }
            labels_mask[index]     = 1;
            labels_mask[index + A] = 1;
            // compute_targets (:265-300) against the box this anchor overlaps most
            const bbox& gt = rec.gt_boxes[best_box[index]];
            const box4& rp = anchors[index];
            const float rw = extent(rp.xmin, rp.xmax), rh = extent(rp.ymin, rp.ymax);
            bbtargets[index + A * 0] = (centre(gt.xmin, gt.xmax) - centre(rp.xmin, rp.xmax)) / rw;
            bbtargets[index + A * 1] = (centre(gt.ymin, gt.ymax) - centre(rp.ymin, rp.ymax)) / rh;
            bbtargets[index + A * 2] = std::log(extent(gt.xmin, gt.xmax) / rw);
            bbtargets[index + A * 3] = std::log(extent(gt.ymin, gt.ymax) / rh);
        }
        im_shape[0]   = rec.im_width;
        im_shape[1]   = rec.im_height;
        *num_gt_boxes = std::min<int>(cfg.max_gt_boxes, (int)rec.gt_boxes.size());
        for (int i = 0; i < cfg.max_gt_boxes; ++i)
        {
            const bool  have = i < *num_gt_boxes;
            const bbox* gt   = have ? &rec.gt_boxes[i] : nullptr;
            gt_boxes[4 * i + 0] = have ? gt->xmin : 0.f;
            gt_boxes[4 * i + 1] = have ? gt->ymin : 0.f;
            gt_boxes[4 * i + 2] = have ? gt->xmax : 0.f;
            gt_boxes[4 * i + 3] = have ? gt->ymax : 0.f;
            gt_classes[i]       = have ? gt->label : 0;
            gt_difficult[i]     = have ? (int)gt->difficult : 0;
        }
        *im_scale = rec.image_scale;
    }
}

using namespace aeonb;

extern "C" {

int64_t aeonb_rcnn_anchor_count(const aeonb_rcnn_config* c)
{
    if (!c || c->width <= 0 || c->height <= 0 || !(c->scaling_factor > 0) || c->n_ratios < 1 || c->n_scales < 1)
        return 0;
    return (int64_t)c->n_ratios * c->n_scales * (int)std::floor((float)c->height * c->scaling_factor) *
           (int)std::floor((float)c->width * c->scaling_factor);
}

int aeonb_rcnn_anchors(const aeonb_rcnn_config* c, float* out)
{
    return guarded([&]() {
        if (!c || !out)
            throw std::invalid_argument("aeonb_rcnn_anchors: NULL argument");
        const std::vector<box4> all = rcnn_generate_anchors(*c);
        std::memcpy(out, all.data(), all.size() * sizeof(box4));
        return AEONB_OK;
    });
}

} // extern "C"
