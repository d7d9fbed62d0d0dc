// Small device helpers shared by the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    __device__ __forceinline__ unsigned int warp_sum(unsigned int v)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    }

    __device__ __forceinline__ float warp_sum(float v)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    }

    // aeon image::standardize (src/image.cpp:129-174): x*(1/255) - mean, then *(1/std), each step
    // rounded in the output precision.  Integer outputs are never standardised (the host rejects
    // mean/stddev for them, src/etl_image.cpp:216-222).
    template <typename T>
    __device__ __forceinline__ T standardize_value(T v, const aeonb_image_layout&, int)
    {
        return v;
    }
    template <>
    __device__ __forceinline__ float standardize_value<float>(float v, const aeonb_image_layout& lay, int c)
    {
        float t = __fmul_rn(v, (float)(1.0 / 255.0));
        t       = __fsub_rn(t, lay.mean[c]);
        return __fmul_rn(t, lay.rstd[c]);
    }
    template <>
    __device__ __forceinline__ double standardize_value<double>(double v, const aeonb_image_layout& lay, int c)
    {
        double t = __dmul_rn(v, 1.0 / 255.0);
        t        = __dsub_rn(t, lay.mean64[c]);
        return __dmul_rn(t, lay.rstd64[c]);
    }
}
