#pragma once
#include "../../../include/aeon_b200.h"

namespace aeonb
{
    // Turns aeon's photometric parameter values into the integer / float constants the image
    // kernel applies (aeon: src/image.cpp:336-346 and :362-371).
    void set_photometric(aeonb_image_desc& d, float contrast, float brightness, float saturation, int hue, const float* lighting,
                         float color_noise_std);
}
