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
