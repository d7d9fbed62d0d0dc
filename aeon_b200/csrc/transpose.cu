// Batch transpose kernel: (N records x D elements) -> (D x N), the layout aeon produces when
// "batch_major" is false (fixed_buffer_map::copy with transpose, src/buffer_batch.cpp:251-280,
// which uses the SSE block transposes of src/transpose.hpp on the CPU).
// 32x32 tiles go through padded shared memory so both the loads and the stores are coalesced.
#include <cuda_runtime.h>
#include <stdint.h>

namespace aeonb
{
    namespace
    {
        template <typename T>
        __global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int64_t rows, int64_t cols)
        {
            __shared__ T tile[32][33];
            const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
            const int     tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
            for (int j = ty; j < 32; j += 8)
                if (r0 + j < rows && c0 + tx < cols)
                    tile[j][tx] = src[(r0 + j) * cols + c0 + tx];
            __syncthreads();
            for (int j = ty; j < 32; j += 8)
                if (c0 + j < cols && r0 + tx < rows)
                    dst[(c0 + j) * rows + r0 + tx] = tile[tx][j];
        }

        template <typename T>
        cudaError_t launch_t(const void* src, void* dst, int64_t rows, int64_t cols, cudaStream_t stream)
        {
            // columns (large) on grid.x, rows (batch) on grid.y
            dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), 1);
            transpose_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(src), static_cast<T*>(dst), rows, cols);
            return cudaGetLastError();
        }
    }

    cudaError_t launch_transpose(const void* src, void* dst, int64_t rows, int64_t cols, int elem_size, cudaStream_t stream)
    {
        if (rows <= 0 || cols <= 0)
            return cudaSuccess;
        switch (elem_size)
        {
        case 1: return launch_t<uint8_t>(src, dst, rows, cols, stream);
        case 2: return launch_t<uint16_t>(src, dst, rows, cols, stream);
        case 4: return launch_t<uint32_t>(src, dst, rows, cols, stream);
        case 8: return launch_t<uint64_t>(src, dst, rows, cols, stream);
        }
        return cudaErrorInvalidValue;
    }
}
