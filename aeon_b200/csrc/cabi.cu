// C ABI: context management and the batch-kernel entry points.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <vector>

#include "context.hpp"

namespace aeonb
{
    namespace
    {
        thread_local std::string g_last_error;
    }

    void set_last_error(const std::string& msg) { g_last_error = msg; }

    int fail(int code, const std::string& msg)
    {
        g_last_error = msg;
        return code;
    }

    std::string cuda_message(const char* what, cudaError_t e)
    {
        std::ostringstream ss;
        ss << what << " failed: " << cudaGetErrorName(e) << " (" << cudaGetErrorString(e) << ")";
        return ss.str();
    }

    void staging_slot::reserve(size_t bytes)
    {
        if (bytes <= capacity)
            return;
        release();
        size_t cap = std::max<size_t>(bytes, 64 * 1024);
        AEONB_CUDA(cudaMallocHost(&host, cap));
        AEONB_CUDA(cudaMalloc(&dev, cap));
        if (!copied)
            AEONB_CUDA(cudaEventCreateWithFlags(&copied, cudaEventDisableTiming));
        capacity = cap;
    }

    void staging_slot::release()
    {
        if (host)
            cudaFreeHost(host);
        if (dev)
            cudaFree(dev);
        host = dev = nullptr;
        capacity   = 0;
    }
}

namespace aeonb
{
    launch_timer::launch_timer(aeonb_ctx* c, int kind, int64_t algorithmic_bytes) : ctx(c)
    {
        if (!ctx->profiling)
            return;
        profile_span sp{kind, nullptr, nullptr, algorithmic_bytes};
        for (cudaEvent_t* e : {&sp.begin, &sp.end})
        {
            if (!ctx->event_pool.empty())
            {
                *e = ctx->event_pool.back();
                ctx->event_pool.pop_back();
            }
            else
                AEONB_CUDA(cudaEventCreate(e));
        }
        AEONB_CUDA(cudaEventRecord(sp.begin, ctx->stream));
        ctx->spans.push_back(sp);
        span = (int)ctx->spans.size() - 1;
    }

    launch_timer::~launch_timer()
    {
        if (span >= 0)
            cudaEventRecord(ctx->spans[span].end, ctx->stream);
    }
}

using namespace aeonb;

namespace aeonb
{
    // Descriptor arrays reach the device through this kernel, which reads the pinned host copy directly (pinned memory
    // is mapped into the device's address space) -- not through the copy engine, where a few KB of descriptors would
    // queue behind the megabytes of the next batch's staging upload and hold up the kernel that waits for them.
    static __global__ void upload_kernel(int4* __restrict__ dst, const int4* __restrict__ src, size_t n16)
    {
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
            dst[i] = src[i];
    }
}

void* aeonb_ctx::upload(const void* host, size_t bytes)
{
    staging_slot& slot = ring[ring_next];
    ring_next          = (ring_next + 1) % ring.size();
    if (slot.busy)
    {
        AEONB_CUDA(cudaEventSynchronize(slot.copied));
        slot.busy = false;
    }
    if (bytes > slot.capacity)
    {
        // A kernel enqueued earlier may still read the old device buffer.
        AEONB_CUDA(cudaStreamSynchronize(stream));
        slot.reserve(bytes);
    }
    std::memcpy(slot.host, host, bytes);
    const size_t n16 = (bytes + 15) / 16; // both buffers are at least 64 KB and 256-byte aligned
    upload_kernel<<<(unsigned)std::min<size_t>((n16 + 255) / 256, 32), 256, 0, stream>>>(static_cast<int4*>(slot.dev),
                                                                                      static_cast<const int4*>(slot.host), n16);
    AEONB_CUDA(cudaGetLastError());
    AEONB_CUDA(cudaEventRecord(slot.copied, stream));
    slot.busy = true;
    return slot.dev;
}

extern "C" {

const char* aeonb_last_error(void)
{
    return g_last_error.c_str();
}

const char* aeonb_version(void)
{
    return "aeon_b200 0.1 (sm_100a)";
}

int aeonb_ctx_create(int device, void* stream, aeonb_ctx** out)
{
    return guarded([&]() {
        if (!out)
            throw std::invalid_argument("aeonb_ctx_create: out is NULL");
        int count = 0;
        AEONB_CUDA(cudaGetDeviceCount(&count));
        if (device < 0 || device >= count)
            throw std::invalid_argument("aeonb_ctx_create: no such CUDA device");
        AEONB_CUDA(cudaSetDevice(device));
        auto* ctx   = new aeonb_ctx();
        ctx->device = device;
        if (stream)
            ctx->stream = static_cast<cudaStream_t>(stream);
        else
        {
            AEONB_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
            ctx->own_stream = true;
        }
        ctx->ring.resize(8);
        *out = ctx;
        return AEONB_OK;
    });
}

void aeonb_ctx_destroy(aeonb_ctx* ctx)
{
    if (!ctx)
        return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& s : ctx->ring)
    {
        s.release();
        if (s.copied)
            cudaEventDestroy(s.copied);
    }
    for (const profile_span& sp : ctx->spans)
    {
        cudaEventDestroy(sp.begin);
        cudaEventDestroy(sp.end);
    }
    for (cudaEvent_t e : ctx->event_pool)
        cudaEventDestroy(e);
    if (ctx->own_stream)
        cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int aeonb_ctx_profile(aeonb_ctx* ctx, int enable)
{
    return guarded([&]() {
        if (!ctx)
            throw std::invalid_argument("context is NULL");
        AEONB_CUDA(cudaSetDevice(ctx->device));
        AEONB_CUDA(cudaStreamSynchronize(ctx->stream));
        for (const profile_span& sp : ctx->spans)
        {
            ctx->event_pool.push_back(sp.begin);
            ctx->event_pool.push_back(sp.end);
        }
        ctx->spans.clear();
        ctx->profiling = enable != 0;
        if (enable)
            for (aeonb_kernel_profile& t : ctx->totals)
                t = aeonb_kernel_profile{0, 0.0, 0};
        return AEONB_OK;
    });
}

int aeonb_ctx_profile_read(aeonb_ctx* ctx, aeonb_kernel_profile out[AEONB_KERNEL_KINDS])
{
    return guarded([&]() {
        if (!ctx || !out)
            throw std::invalid_argument("aeonb_ctx_profile_read: NULL argument");
        AEONB_CUDA(cudaSetDevice(ctx->device));
        AEONB_CUDA(cudaStreamSynchronize(ctx->stream));
        for (const profile_span& sp : ctx->spans)
        {
            float ms = 0;
            AEONB_CUDA(cudaEventElapsedTime(&ms, sp.begin, sp.end));
            aeonb_kernel_profile& t = ctx->totals[sp.kind];
            t.launches++;
            t.ms += ms;
            t.algorithmic_bytes += sp.bytes;
            ctx->event_pool.push_back(sp.begin);
            ctx->event_pool.push_back(sp.end);
        }
        ctx->spans.clear();
        for (int k = 0; k < AEONB_KERNEL_KINDS; ++k)
            out[k] = ctx->totals[k];
        return AEONB_OK;
    });
}

void* aeonb_ctx_stream(aeonb_ctx* ctx)
{
    return ctx ? ctx->stream : nullptr;
}

int aeonb_ctx_synchronize(aeonb_ctx* ctx)
{
    return guarded([&]() {
        if (!ctx)
            throw std::invalid_argument("context is NULL");
        AEONB_CUDA(cudaStreamSynchronize(ctx->stream));
        return AEONB_OK;
    });
}

static size_t dtype_size(int dtype)
{
    switch (dtype)
    {
    case AEONB_U8:
    case AEONB_I8: return 1;
    case AEONB_I16:
    case AEONB_U16: return 2;
    case AEONB_I32:
    case AEONB_F32: return 4;
    case AEONB_F64: return 8;
    }
    throw std::invalid_argument("unknown output dtype");
}

} // extern "C"

void aeonb::check_image_batch(const aeonb_image_desc* d, int n, const aeonb_image_layout& L, int& pixel_stride, bool& aligned)
{
    if (L.slot_w <= 0 || L.slot_h <= 0)
        throw std::invalid_argument("invalid width or height of the output slot");
    if (L.channels != 3 && L.channels != 1)
        throw std::invalid_argument("the output has 1 or 3 channels");
    if (L.channels == 1 && L.bgr_to_rgb)
        throw std::invalid_argument("invalid config: bgr_to_rgb can be 'true' only for channels set to '3'");
    if (L.standardize && !(L.dtype == AEONB_F32 || L.dtype == AEONB_F64))
        throw std::invalid_argument(
            "Standardization (mean, stddev) is supported only for float or double 'output_type'.");
    dtype_size(L.dtype);
    pixel_stride = 0;
    aligned      = true;
    for (int i = 0; i < n; ++i)
    {
        const aeonb_image_desc& r = d[i];
        std::ostringstream      ss;
        if (!r.dst)
            ss << "record " << i << ": destination is NULL";
        else if (r.src)
        {
            if (r.src_pixel_stride != 3 && r.src_pixel_stride != 4)
                ss << "record " << i << ": source pixel stride must be 3 or 4";
            else if (pixel_stride && r.src_pixel_stride != pixel_stride)
                ss << "record " << i << ": all sources of a batch must share one pixel stride";
            else if (r.src_w <= 0 || r.src_h <= 0 || r.src_pitch < r.src_w * r.src_pixel_stride)
                ss << "record " << i << ": invalid source size or pitch";
            else if (r.src_pixel_stride == 4 && (((uintptr_t)r.src | (uintptr_t)r.src_pitch) & 3))
                ss << "record " << i << ": 4-byte pixels need a 4-byte aligned source and pitch";
            else if (r.canvas_x < 0 || r.canvas_y < 0 || r.canvas_x + r.src_w > r.canvas_w || r.canvas_y + r.src_h > r.canvas_h)
                ss << "record " << i << ": Invalid parameters to expand image";
            else if (r.crop_w <= 0 || r.crop_h <= 0 || r.crop_x < 0 || r.crop_y < 0 || r.crop_x + r.crop_w > r.canvas_w ||
                     r.crop_y + r.crop_h > r.canvas_h)
                ss << "record " << i << ": crop box (" << r.crop_x << "," << r.crop_y << " " << r.crop_w << "x" << r.crop_h
                   << ") is outside the " << r.canvas_w << "x" << r.canvas_h << " image";
            else if (r.out_w <= 0 || r.out_h <= 0 || r.out_w > L.slot_w || r.out_h > L.slot_h)
                ss << "record " << i << ": output size " << r.out_w << "x" << r.out_h << " does not fit the slot";
            else if (r.interp != AEONB_INTERP_LINEAR && r.interp != AEONB_INTERP_NEAREST)
                ss << "record " << i << ": interpolation method outside the accelerated set (NEAREST, LINEAR)";
            if (r.src_pixel_stride == 3 || r.src_pixel_stride == 4)
                pixel_stride = r.src_pixel_stride;
        }
        const std::string msg = ss.str();
        if (!msg.empty())
            throw std::invalid_argument(msg);
        if ((uintptr_t)r.dst & 15)
            aligned = false;
    }
    if (!pixel_stride)
        pixel_stride = 3;
}

extern "C" {

int aeonb_image_batch(aeonb_ctx* ctx, const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout)
{
    return guarded([&]() {
        if (!ctx || !layout || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_image_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        int  pixel_stride;
        bool aligned;
        check_image_batch(descs, n, *layout, pixel_stride, aligned);
        AEONB_CUDA(cudaSetDevice(ctx->device));
        // Launch order: the kernel's blocks start in descriptor order and the launch ends with its last block, so the
        // records with the most source rows to filter go first and the cheap ones fill the tail.  Every descriptor
        // carries its own destination, so the order is free.
        std::vector<aeonb_image_desc> ordered(descs, descs + n);
        auto cost = [](const aeonb_image_desc& r) { return r.src ? std::min(r.crop_h, 2 * r.out_h) : 0; };
        std::stable_sort(ordered.begin(), ordered.end(), [&](const aeonb_image_desc& a, const aeonb_image_desc& b) { return cost(a) > cost(b); });
        auto* dev = static_cast<const aeonb_image_desc*>(ctx->upload(ordered.data(), sizeof(aeonb_image_desc) * n));
        const char*  why = nullptr;
        launch_timer timer(ctx, AEONB_KERNEL_IMAGE, ctx->profiling ? aeonb_image_batch_bytes(descs, n, layout) : 0);
        cudaError_t  e   = launch_aug_pack(dev, ordered.data(), n, *layout, pixel_stride, aligned, ctx->stream, &why);
        if (why)
            throw error(AEONB_ERR_UNSUPPORTED, why);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("image kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}

int64_t aeonb_image_batch_bytes(const aeonb_image_desc* descs, int n, const aeonb_image_layout* layout)
{
    if (!descs || !layout)
        return 0;
    int64_t total = 0;
    size_t  esz   = 1;
    try
    {
        esz = dtype_size(layout->dtype);
    }
    catch (...)
    {
        return 0;
    }
    for (int i = 0; i < n; ++i)
    {
        const aeonb_image_desc& r = descs[i];
        if (r.src)
        {
            // part of the crop box that lies on the source image; canvas zeros are never read
            int64_t x0 = std::max(r.crop_x, r.canvas_x), x1 = std::min(r.crop_x + r.crop_w, r.canvas_x + r.src_w);
            int64_t y0 = std::max(r.crop_y, r.canvas_y), y1 = std::min(r.crop_y + r.crop_h, r.canvas_y + r.src_h);
            if (x1 > x0 && y1 > y0)
                total += (x1 - x0) * (y1 - y0) * 3;
        }
        total += (int64_t)layout->slot_w * layout->slot_h * layout->channels * esz;
    }
    return total;
}

int aeonb_jpeg_backend_batch(aeonb_ctx* ctx, const aeonb_jpeg_desc* descs, int n)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_jpeg_backend_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        std::vector<int2> work;
        size_t            smem = 0;
        for (int i = 0; i < n; ++i)
        {
            const aeonb_jpeg_desc& r = descs[i];
            std::ostringstream     ss;
            const bool sampling_ok = r.ncomp == 1 || (r.ncomp == 3 && r.hs[1] == 1 && r.vs[1] == 1 && r.hs[2] == 1 && r.vs[2] == 1 &&
                                                      ((r.hs[0] == 1 && r.vs[0] == 1) || (r.hs[0] == 2 && r.vs[0] == 1) ||
                                                       (r.hs[0] == 2 && r.vs[0] == 2) || (r.hs[0] == 1 && r.vs[0] == 2) ||
                                                       (r.hs[0] == 4 && r.vs[0] == 1)));
            if (r.width <= 0 || r.height <= 0 || !r.dst)
                ss << "record " << i << ": empty image or NULL destination";
            else if (!sampling_ok || (r.ncomp == 1 && (r.hs[0] != 1 || r.vs[0] != 1)))
                ss << "record " << i << ": unsupported component layout (supported: grey, 4:4:4, 4:2:2, 4:2:0, 4:4:0, 4:1:1)";
            else if (r.dst_pixel_stride != 3 && r.dst_pixel_stride != 4)
                ss << "record " << i << ": destination pixel stride must be 3 or 4";
            else if (r.dst_pitch < r.width * r.dst_pixel_stride || (r.dst_pitch & (r.dst_pixel_stride == 4 ? 15 : 3)) ||
                     ((uintptr_t)r.dst & (r.dst_pixel_stride == 4 ? 15 : 3)))
                ss << "record " << i << ": destination must be " << (r.dst_pixel_stride == 4 ? 16 : 4)
                   << "-byte aligned with a pitch that is a multiple of that";
            else
            {
                for (int c = 0; c < r.ncomp; ++c)
                {
                    if (!r.coef[c] || !r.quant[c] || ((uintptr_t)r.coef[c] & 15) || ((uintptr_t)r.quant[c] & 1))
                        ss << "record " << i << ": coefficient planes must be 16-byte aligned device pointers";
                    else if (r.blocks_w[c] * 8 * r.hs[0] / r.hs[c] < r.width || r.blocks_h[c] * 8 * r.vs[0] / r.vs[c] < r.height ||
                             r.blocks_w[c] != r.blocks_w[0] / r.hs[0] * r.hs[c] || r.blocks_h[c] != r.blocks_h[0] / r.vs[0] * r.vs[c])
                        ss << "record " << i << ": coefficient plane size does not match the image";
                }
            }
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
            smem = std::max(smem, jpeg_backend_smem(r));
            const int mcu_rows = r.blocks_h[0] / r.vs[0];
            for (int m = 0; m < mcu_rows; m += jpeg_backend_strip())
                if (m * r.vs[0] * 8 < r.height)
                    work.push_back(make_int2(i, m));
        }
        if (smem > 200 * 1024)
            throw error(AEONB_ERR_UNSUPPORTED, "image too wide for the on-chip MCU-row strip");
        AEONB_CUDA(cudaSetDevice(ctx->device));
        auto* ddev = static_cast<const aeonb_jpeg_desc*>(ctx->upload(descs, sizeof(aeonb_jpeg_desc) * n));
        auto* wdev = static_cast<const int2*>(ctx->upload(work.data(), sizeof(int2) * work.size()));
        launch_timer timer(ctx, AEONB_KERNEL_JPEG_BACKEND, ctx->profiling ? aeonb_jpeg_backend_bytes(descs, n) : 0);
        cudaError_t  e = launch_jpeg_backend(ddev, wdev, (int)work.size(), smem, ctx->stream);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("jpeg back-end kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}

int aeonb_jpeg_entropy_batch(aeonb_ctx* ctx, const aeonb_entropy_desc* descs, int n)
{
    return guarded([&]() {
        if (!ctx || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_jpeg_entropy_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        bool any_parallel = false, any_serial = false;
        for (int i = 0; i < n; ++i)
        {
            const aeonb_entropy_desc& r = descs[i];
            std::ostringstream        ss;
            if (!r.scan || !r.tables || r.ncomp < 1 || r.ncomp > 3 || r.mcux <= 0 || r.mcuy <= 0)
                ss << "record " << i << ": NULL stream or tables, or an empty picture";
            else if (r.roi[0] < 0 || r.roi[1] < 0 || r.roi[2] > r.mcux || r.roi[3] > r.mcuy || r.roi[0] >= r.roi[2] || r.roi[1] >= r.roi[3])
                ss << "record " << i << ": region outside the picture";
            else if (r.restart_interval < 0)
                ss << "record " << i << ": negative restart interval";
            else
                for (int c = 0; c < r.ncomp; ++c)
                {
                    if (!r.coef[c] || ((uintptr_t)r.coef[c] & 15))
                        ss << "record " << i << ": coefficient planes must be 16-byte aligned device pointers";
                    else if (r.hs[c] < 1 || r.hs[c] > 4 || r.vs[c] < 1 || r.vs[c] > 4 || (r.dc_table[c] & ~1) || (r.ac_table[c] & ~1))
                        ss << "record " << i << ": sampling factors must be 1..4 and table slots 0 or 1";
                }
            if (ss.str().empty() && r.scratch && (((uintptr_t)r.scratch & 15) || (int64_t)r.scratch_bytes < jpeg_entropy_scratch_bytes(r)))
                ss << "record " << i << ": the work area must be 16-byte aligned and hold aeonb_jpeg_entropy_scratch_bytes() bytes";
            const std::string msg = ss.str();
            if (!msg.empty())
                throw std::invalid_argument(msg);
            if (r.scratch && r.restart_interval == 0)
                any_parallel = true;
            else
                any_serial = true;
        }
        AEONB_CUDA(cudaSetDevice(ctx->device));
        // Block order.  The kernel takes as long as its slowest block, and that is the block of the longest stream.  All
        // blocks of a batch are resident at once, two to an SM once there are more blocks than SMs; the first `sms` blocks
        // of a grid land on SMs of their own.  So the longest streams go to the blocks that keep their SM to themselves
        // (the last ones of the first wave when the second wave is not full), the next longest to the rest of the first
        // wave, the shortest to the second wave.  Measured on B200, 256 streams of 20-80 KB: 0.85 ms against 0.88 ms in
        // arrival order.  AEONB_ENTROPY_ORDER=0 keeps the arrival order.
        std::vector<aeonb_entropy_desc> ordered;
        static const bool reorder = [] {
            const char* e = std::getenv("AEONB_ENTROPY_ORDER");
            return !e || std::atoi(e) != 0;
        }();
        if (reorder && n > 1)
        {
            int sms = 148;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device);
            std::vector<int> by_size(n);
            for (int i = 0; i < n; ++i)
                by_size[i] = i;
            std::stable_sort(by_size.begin(), by_size.end(), [&](int a, int b) { return descs[a].scan_size > descs[b].scan_size; });
            const int first  = std::min(n, sms);                      // blocks of the first wave
            const int shared = n > sms ? std::min(n - sms, sms) : 0;  // first-wave blocks that get a second block on their SM
            ordered.resize(n);
            int next = 0;
            for (int b = shared; b < first; ++b)
                ordered[b] = descs[by_size[next++]];
            for (int b = 0; b < shared; ++b)
                ordered[b] = descs[by_size[next++]];
            for (int b = first; b < n; ++b)
                ordered[b] = descs[by_size[next++]];
            descs = ordered.data();
        }
        auto* ddev = static_cast<const aeonb_entropy_desc*>(ctx->upload(descs, sizeof(aeonb_entropy_desc) * n));
        int64_t bytes = 0; // compressed scan in + the coefficient blocks of the region out
        if (ctx->profiling)
            for (int i = 0; i < n; ++i)
            {
                const aeonb_entropy_desc& r = descs[i];
                bytes += r.scan_size;
                for (int c = 0; c < r.ncomp; ++c)
                    bytes += (int64_t)(r.roi[2] - r.roi[0]) * r.hs[c] * (r.roi[3] - r.roi[1]) * r.vs[c] * 128;
            }
        launch_timer timer(ctx, AEONB_KERNEL_ENTROPY, bytes);
        // A launch of short streams (video frames) takes smaller blocks: its streams have few segments, and more blocks fit an SM.
        uint32_t longest = 0;
        for (int i = 0; i < n; ++i)
            if (descs[i].scratch && descs[i].restart_interval == 0)
                longest = std::max(longest, descs[i].scan_size);
        const int segments = (int)((longest + (uint32_t)jpeg_entropy_min_segment() - 1) / (uint32_t)jpeg_entropy_min_segment());
        int       threads  = jpeg_entropy_threads();
        while (threads > 128 && segments <= threads / 2)
            threads /= 2;
        cudaError_t  e = launch_jpeg_entropy(ddev, n, any_parallel, any_serial, jpeg_entropy_min_segment(), threads, ctx->stream);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("jpeg entropy kernel launch", e));
        ctx->launches += (any_parallel ? 1 : 0) + (any_serial ? 1 : 0);
        return AEONB_OK;
    });
}

int64_t aeonb_jpeg_entropy_scratch_bytes(const aeonb_entropy_desc* desc)
{
    return desc ? jpeg_entropy_scratch_bytes(*desc) : 0;
}

int64_t aeonb_jpeg_backend_bytes(const aeonb_jpeg_desc* descs, int n)
{
    int64_t total = 0;
    for (int i = 0; descs && i < n; ++i)
    {
        const aeonb_jpeg_desc& r = descs[i];
        for (int c = 0; c < r.ncomp; ++c)
            total += (int64_t)r.blocks_w[c] * r.blocks_h[c] * 64 * 2;
        total += (int64_t)r.width * r.height * 3;
    }
    return total;
}

} // extern "C"
