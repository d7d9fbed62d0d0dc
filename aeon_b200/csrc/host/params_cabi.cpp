// C entry point exposing the seeded augmentation-parameter draws (used by callers that
// run the kernels themselves, and by the parity tests of the draw order).
#include <vector>

#include "../context.hpp"
#include "params.hpp"

using namespace aeonb;

namespace aeonb
{
    // aeon src/batch_decoder.cpp:47-54: one engine per decode slot, seeded from a master engine.
    std::vector<random_engine_t> make_slot_engines(uint32_t seed, int decode_size)
    {
        std::vector<random_engine_t> engines(decode_size);
        random_engine_t              master(seed);
        for (auto& e : engines)
            e.seed(master());
        return engines;
    }
}

namespace
{
    void write_params(const image_params& p, double* o)
    {
        o[0]  = p.cropbox.x;
        o[1]  = p.cropbox.y;
        o[2]  = p.cropbox.width;
        o[3]  = p.cropbox.height;
        o[4]  = p.output_size.width;
        o[5]  = p.output_size.height;
        o[6]  = p.flip;
        o[7]  = p.angle;
        o[8]  = p.hue;
        o[9]  = p.contrast;
        o[10] = p.brightness;
        o[11] = p.saturation;
        for (int k = 0; k < 3; ++k)
            o[12 + k] = k < (int)p.lighting.size() ? p.lighting[k] : 0.0;
        o[15] = p.color_noise_std;
        o[16] = p.padding_crop_offset.width;
        o[17] = p.padding_crop_offset.height;
        o[18] = p.expand_ratio;
        o[19] = p.expand_offset.width;
        o[20] = p.expand_offset.height;
        o[21] = p.expand_size.width;
        o[22] = p.expand_size.height;
        o[23] = 0;
    }
}

extern "C" int aeonb_draw_ssd_params(const char* augmentation_json, uint32_t seed, int decode_size, int n, const int32_t* in_w,
                                     const int32_t* in_h, int out_w, int out_h, const int32_t* box_counts, const float* boxes,
                                     double* out)
{
    return guarded([&]() {
        if (!in_w || !in_h || !out || !box_counts || decode_size <= 0 || n < 0)
            throw std::invalid_argument("aeonb_draw_ssd_params: bad argument");
        json cfg;
        if (augmentation_json && *augmentation_json)
            cfg = json::parse(augmentation_json);
        param_factory factory(cfg);
        auto          engines = make_slot_engines(seed, decode_size);
        size_t        at      = 0;
        for (int i = 0; i < n; ++i)
        {
            std::vector<bbox> bb(box_counts[i]);
            for (auto& b : bb)
            {
                b.xmin = boxes[at++];
                b.ymin = boxes[at++];
                b.xmax = boxes[at++];
                b.ymax = boxes[at++];
            }
            write_params(factory.make_ssd_params(engines[i % decode_size], in_w[i], in_h[i], out_w, out_h, bb), out + (size_t)i * 24);
        }
        return AEONB_OK;
    });
}

extern "C" int aeonb_draw_params(const char* augmentation_json, uint32_t seed, int decode_size, int n, const int32_t* in_w,
                                 const int32_t* in_h, int out_w, int out_h, double* out)
{
    return guarded([&]() {
        if (!in_w || !in_h || !out || decode_size <= 0 || n < 0)
            throw std::invalid_argument("aeonb_draw_params: bad argument");
        json cfg;
        if (augmentation_json && *augmentation_json)
            cfg = json::parse(augmentation_json);
        param_factory factory(cfg);
        auto          engines = make_slot_engines(seed, decode_size);
        for (int i = 0; i < n; ++i)
        {
            image_params p = factory.make_params(engines[i % decode_size], in_w[i], in_h[i], out_w, out_h);
            double*      o = out + (size_t)i * 24;
            o[0]           = p.cropbox.x;
            o[1]           = p.cropbox.y;
            o[2]           = p.cropbox.width;
            o[3]           = p.cropbox.height;
            o[4]           = p.output_size.width;
            o[5]           = p.output_size.height;
            o[6]           = p.flip;
            o[7]           = p.angle;
            o[8]           = p.hue;
            o[9]           = p.contrast;
            o[10]          = p.brightness;
            o[11]          = p.saturation;
            for (int k = 0; k < 3; ++k)
                o[12 + k] = k < (int)p.lighting.size() ? p.lighting[k] : 0.0;
            o[15] = p.color_noise_std;
            o[16] = p.padding_crop_offset.width;
            o[17] = p.padding_crop_offset.height;
            o[18] = p.expand_ratio;
            o[19] = p.expand_offset.width;
            o[20] = p.expand_offset.height;
            o[21] = p.expand_size.width;
            o[22] = p.expand_size.height;
            o[23] = 0;
        }
        return AEONB_OK;
    });
}

// ---- host box arithmetic of the localisation providers, exposed for callers that keep aeon's box classes and for
// the parity tests against the reference's known answers

extern "C" int aeonb_box_overlap(int normalized, const float a[4], const float b[4], float out[6])
{
    return guarded([&]() {
        if (!a || !b || !out)
            throw std::invalid_argument("aeonb_box_overlap: NULL argument");
        if (normalized)
        {
            const nbox x(a[0], a[1], a[2], a[3]), y(b[0], b[1], b[2], b[3]);
            const nbox i = x.intersect(y);
            out[0] = i.xmin, out[1] = i.ymin, out[2] = i.xmax, out[3] = i.ymax;
            out[4] = x.jaccard_overlap(y);
            out[5] = x.coverage(y);
        }
        else
        {
            bbox x, y;
            x.xmin = a[0], x.ymin = a[1], x.xmax = a[2], x.ymax = a[3];
            y.xmin = b[0], y.ymin = b[1], y.xmax = b[2], y.ymax = b[3];
            const bbox i = bbox_intersect(x, y);
            out[0] = i.xmin, out[1] = i.ymin, out[2] = i.xmax, out[3] = i.ymax;
            out[4] = bbox_jaccard(x, y);
            out[5] = bbox_coverage(x, y);
        }
        return AEONB_OK;
    });
}

extern "C" int aeonb_transform_boxes(const aeonb_box_params* p, const float* boxes, int n, float* out, int32_t* kept, int32_t* n_out)
{
    return guarded([&]() {
        if (!p || (n > 0 && !boxes) || !out || !n_out || n < 0)
            throw std::invalid_argument("aeonb_transform_boxes: bad argument");
        image_params ip;
        ip.cropbox       = recti{p->crop_x, p->crop_y, p->crop_w, p->crop_h};
        ip.output_size   = size2i{p->out_w, p->out_h};
        ip.flip          = p->flip != 0;
        ip.expand_ratio  = p->expand_ratio;
        ip.expand_offset = size2i{p->expand_off_x, p->expand_off_y};
        ip.expand_size   = size2i{p->expand_w, p->expand_h};
        ip.emit_constraint_type = p->emit_type == 1 ? emit_type::center : p->emit_type == 2 ? emit_type::min_overlap : emit_type::undefined;
        ip.emit_min_overlap     = p->emit_min_overlap;
        std::vector<bbox> in(n);
        for (int i = 0; i < n; ++i)
        {
            in[i].xmin = boxes[4 * i], in[i].ymin = boxes[4 * i + 1], in[i].xmax = boxes[4 * i + 2], in[i].ymax = boxes[4 * i + 3];
            in[i].label = i; // carries the input index through the transformation
        }
        const std::vector<bbox> tx = transform_boxes_for_ssd(in, ip);
        for (size_t i = 0; i < tx.size(); ++i)
        {
            out[4 * i] = tx[i].xmin, out[4 * i + 1] = tx[i].ymin, out[4 * i + 2] = tx[i].xmax, out[4 * i + 3] = tx[i].ymax;
            if (kept)
                kept[i] = tx[i].label;
        }
        *n_out = (int32_t)tx.size();
        return AEONB_OK;
    });
}

extern "C" int aeonb_ssd_load_boxes(const float* boxes, const int32_t* labels, const int32_t* difficult, int n, int width, int height,
                                    int max_gt_boxes, int32_t* image_shape, float* gt_boxes, int32_t* gt_box_count, int32_t* gt_class,
                                    int32_t* gt_difficult)
{
    return guarded([&]() {
        if ((n > 0 && (!boxes || !labels || !difficult)) || !image_shape || !gt_boxes || !gt_box_count || !gt_class || !gt_difficult ||
            n < 0 || max_gt_boxes < 0)
            throw std::invalid_argument("aeonb_ssd_load_boxes: bad argument");
        std::vector<bbox> gt(n);
        for (int i = 0; i < n; ++i)
        {
            gt[i].xmin = boxes[4 * i], gt[i].ymin = boxes[4 * i + 1], gt[i].xmax = boxes[4 * i + 2], gt[i].ymax = boxes[4 * i + 3];
            gt[i].label = labels[i], gt[i].difficult = difficult[i] != 0;
        }
        for (int i = 0; i < max_gt_boxes; ++i)
        {
            gt_boxes[4 * i] = gt_boxes[4 * i + 1] = gt_boxes[4 * i + 2] = gt_boxes[4 * i + 3] = 0.f;
            gt_class[i] = gt_difficult[i] = 0;
        }
        ssd_fill_buffers(gt, width, height, max_gt_boxes, image_shape, gt_boxes, gt_box_count, gt_class, gt_difficult);
        return AEONB_OK;
    });
}
