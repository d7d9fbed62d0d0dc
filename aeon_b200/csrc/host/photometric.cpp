// Host-side preparation of the photometric parameters the image kernel consumes.
#include <cmath>
#include <cstdlib>

#include "../context.hpp"
#include "photometric.hpp"

namespace aeonb
{
    namespace
    {
        // aeon src/image.cpp:320-324
        const float k_cpca[3][3] = {{0.39731118f, 0.70119634f, -0.59200296f},
                                    {-0.81698062f, -0.02354167f, -0.57618440f},
                                    {0.41795513f, -0.71257945f, -0.56351045f}};
        const float k_cstd[3]    = {19.72083305f, 37.09388853f, 121.78006099f};
        const float k_gray[3]    = {0.0820f, 0.6094f, 0.3086f}; // src/image.cpp:367, BGR order

        int hsv_vector_block()
        {
            // OpenCV's HSV->BGR row kernel handles 32 pixels per vector iteration on AVX2 hosts (truncating),
            // and finishes each row in scalar code (rounding).  The environment variable lets a deployment
            // match an OpenCV build with a different vector width (0: every pixel rounds).
            if (const char* e = std::getenv("AEONB_HSV_VECTOR_BLOCK"))
                return std::max(0, std::atoi(e));
            return 32;
        }

        short sat_s16(long v) { return (short)std::min(32767L, std::max(-32768L, v)); }
    }

    void set_photometric(aeonb_image_desc& d, float contrast, float brightness, float saturation, int hue, const float* lighting,
                         float color_noise_std)
    {
        d.color_enable = (brightness != 1.0f || saturation != 1.0f) ? 1 : 0;
        if (d.color_enable)
        {
            // b*(s*I + (1-s)*1*g^T) evaluated the way the cv::MatExpr is: the rank-one term through a
            // double-accumulating product, the sum as a float weighted add.
            const float oms = 1.0f - saturation;
            const float sb  = (float)((double)saturation * (double)brightness);
            float       m[3][3];
            bool        diagonal = true;
            for (int i = 0; i < 3; ++i)
                for (int j = 0; j < 3; ++j)
                {
                    const float gray = (float)((double)oms * (double)k_gray[j]);
                    volatile float a = (i == j) ? sb : 0.0f;
                    volatile float b = gray * brightness;
                    m[i][j]          = a + b;
                    d.color_matrix[i * 3 + j] = sat_s16(std::lrintf(m[i][j] * 1024.0f)); // cv::transform's 10-bit form
                    if (i != j && std::fabs((double)m[i][j]) > 1.1920928955078125e-07)  // FLT_EPSILON
                        diagonal = false;
                }
            if (diagonal)
            {
                // cv::transform sends a diagonal matrix (saturation == 1) to a per-channel float scale
                d.color_enable = 2;
                for (int i = 0; i < 3; ++i)
                    d.color_scale[i] = m[i][i];
            }
        }
        else
            for (int i = 0; i < 9; ++i)
                d.color_matrix[i] = (i % 4 == 0) ? 1024 : 0;
        if (d.color_enable != 2)
            d.color_scale[0] = d.color_scale[1] = d.color_scale[2] = 1.0f;
        d.reserved0       = 0;
        d.hue             = hue;
        const int block   = hsv_vector_block();
        d.hsv_vector_cols = block > 0 ? (d.out_w / block) * block : 0;
        d.contrast        = contrast;
        if (lighting)
        {
            // pixel = CPCA * (CSTD o alpha); (img + pixel)/(1+std) becomes a scale and integer offsets
            const double alpha = 1.0 / (1.0 + (double)color_noise_std);
            float        t[3];
            for (int k = 0; k < 3; ++k)
                t[k] = k_cstd[k] * lighting[k];
            for (int i = 0; i < 3; ++i)
            {
                double acc = 0;
                for (int k = 0; k < 3; ++k)
                    acc += (double)k_cpca[i][k] * (double)t[k];
                const float pix      = (float)acc;
                d.lighting_offset[i] = (int)std::lrint((double)pix * alpha);
            }
            d.lighting_scale  = (float)alpha;
            d.lighting_enable = 1;
        }
        else
        {
            d.lighting_enable = 0;
            d.lighting_scale  = 1.0f;
            d.lighting_offset[0] = d.lighting_offset[1] = d.lighting_offset[2] = 0;
        }
    }
}

extern "C" int aeonb_image_desc_set_photometric(aeonb_image_desc* desc, float contrast, float brightness, float saturation,
                                                int hue, const float* lighting, float color_noise_std)
{
    return aeonb::guarded([&]() {
        if (!desc)
            throw std::invalid_argument("aeonb_image_desc_set_photometric: desc is NULL");
        aeonb::set_photometric(*desc, contrast, brightness, saturation, hue, lighting, color_noise_std);
        return AEONB_OK;
    });
}
