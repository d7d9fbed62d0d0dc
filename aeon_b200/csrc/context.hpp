// Per-GPU context behind the C ABI: stream, descriptor staging ring, scratch arena.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    // Status + message carried across the C boundary (aeon throws; the ABI returns codes).
    struct error : std::runtime_error
    {
        int code;
        error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
    };

    void        set_last_error(const std::string& msg);
    int         fail(int code, const std::string& msg);
    std::string cuda_message(const char* what, cudaError_t e);

#define AEONB_CUDA(call)                                                                                               \
    do                                                                                                                 \
    {                                                                                                                  \
        cudaError_t e__ = (call);                                                                                      \
        if (e__ != cudaSuccess)                                                                                        \
            throw ::aeonb::error(AEONB_ERR_CUDA, ::aeonb::cuda_message(#call, e__));                                   \
    } while (0)

    // Runs `fn`, translating exceptions into a status code + thread-local message.
    template <typename F>
    int guarded(F&& fn)
    {
        try
        {
            return fn();
        }
        catch (const error& e)
        {
            return fail(e.code, e.what());
        }
        catch (const std::invalid_argument& e)
        {
            return fail(AEONB_ERR_INVALID, e.what());
        }
        catch (const std::exception& e)
        {
            return fail(AEONB_ERR_DECODE, e.what());
        }
    }

    // A pinned host buffer paired with a device buffer of the same size; used to ship small
    // descriptor arrays (and, in the provider, coefficient planes) with one async copy.
    struct staging_slot
    {
        void*       host     = nullptr;
        void*       dev      = nullptr;
        size_t      capacity = 0;
        cudaEvent_t copied   = nullptr; // recorded after the last H2D copy out of `host`
        bool        busy     = false;
        void        reserve(size_t bytes);
        void        release();
    };
}

namespace aeonb
{
    // one timed kernel launch of a context whose profile is switched on
    struct profile_span
    {
        int         kind;
        cudaEvent_t begin, end;
        int64_t     bytes;
    };
}

struct aeonb_ctx
{
    int                                device     = 0;
    cudaStream_t                       stream     = nullptr;
    bool                               own_stream = false;
    std::vector<aeonb::staging_slot>   ring;      // descriptor staging
    size_t                             ring_next  = 0;
    int64_t                            launches   = 0; // kernels launched through this context
    bool                               profiling  = false; // aeonb_ctx_profile: time every kernel with a pair of events
    std::vector<aeonb::profile_span>   spans;              // launches not yet added to the totals
    std::vector<cudaEvent_t>           event_pool;
    aeonb_kernel_profile               totals[AEONB_KERNEL_KINDS] = {};

    // Copies `bytes` of host data to the device on the stream; the returned device pointer is
    // valid for kernels enqueued after this call.
    void* upload(const void* host, size_t bytes);
};

namespace aeonb
{
    // Brackets the launch(es) of one batch call: counts them and, when the context's profile is on, records a timing
    // event on the context's stream before and after.
    struct launch_timer
    {
        launch_timer(aeonb_ctx* ctx, int kind, int64_t algorithmic_bytes);
        ~launch_timer();
        launch_timer(const launch_timer&) = delete;
        aeonb_ctx* ctx;
        int        span = -1;
    };

    // Validates a batch of image descriptors (throws std::invalid_argument / aeonb::error); reports the
    // common source pixel stride and whether every destination slot is 16-byte aligned.
    void check_image_batch(const aeonb_image_desc* d, int n, const aeonb_image_layout& L, int& pixel_stride, bool& aligned);

    // Kernel launchers (defined next to the kernels).
    cudaError_t launch_aug_pack(const aeonb_image_desc* descs_dev, const aeonb_image_desc* descs_host, int n,
                                const aeonb_image_layout& layout, int pixel_stride, bool slots_aligned, cudaStream_t stream,
                                const char** why);
    cudaError_t launch_jpeg_backend(const aeonb_jpeg_desc* descs_dev, const int2* work_dev, int n_work, size_t smem,
                                    cudaStream_t stream);
    size_t      jpeg_backend_smem(const aeonb_jpeg_desc& d);
    int         jpeg_backend_strip(); // MCU rows one CTA of the back-end kernel handles
    // Entropy kernels: the block-parallel one takes the records that have a work area and no restart markers,
    // the one-warp serial one the rest.  min_segment: smallest segment (bytes) a thread of the parallel kernel decodes;
    // threads: threads (= most segments) per stream of this launch, at most jpeg_entropy_threads().
    cudaError_t launch_jpeg_entropy(const aeonb_entropy_desc* descs_dev, int n, bool any_parallel, bool any_serial, int min_segment,
                                    int threads, cudaStream_t stream);
    int64_t     jpeg_entropy_scratch_bytes(const aeonb_entropy_desc& d);
    int         jpeg_entropy_min_segment(); // AEONB_ENTROPY_SEGMENT or the default
    int         jpeg_entropy_threads();     // AEONB_ENTROPY_THREADS or the default: most threads per stream
}
