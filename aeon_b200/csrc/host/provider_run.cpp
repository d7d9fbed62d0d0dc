// aeonb_provider::run -- one batch through the host stages and the GPU kernels.
#if defined(__SSE2__)
#include <emmintrin.h>
#endif
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <thread>

#include "avi.hpp"
#include "photometric.hpp"
#include "provider.hpp"

using namespace aeonb;
using std::string;
using std::vector;

namespace aeonb
{
    cudaError_t  launch_transpose(const void* src, void* dst, int64_t rows, int64_t cols, int elem_size, cudaStream_t stream);
    void parse_ssd_annotation(const void* data, size_t size, const std::unordered_map<string, int>& classes, int& width,
                              int& height, vector<bbox>& boxes);

    namespace
    {
        void check_status(int status)
        {
            if (status < 0)
                throw error(status, aeonb_last_error());
        }

        // Geometry + photometric fields of a descriptor from aeon's params
        // (image::transformer::transform_single_image, src/etl_image.cpp:146-202).
        aeonb_image_desc make_desc(const image_params& p, int src_w, int src_h, int slot_w, int slot_h, bool exact_fit)
        {
            string m = p.interpolation_method;
            std::transform(m.begin(), m.end(), m.begin(), ::toupper);
            aeonb_image_desc d{};
            if (m == "LINEAR")
                d.interp = AEONB_INTERP_LINEAR;
            else if (m == "NEAREST")
                d.interp = AEONB_INTERP_NEAREST;
            else if (m == "AREA")
                d.interp = AEONB_INTERP_AREA; // AREA and CUBIC run as a pass of their own (aeonb_resize_batch), never in the image kernel
            else if (m == "CUBIC")
                d.interp = AEONB_INTERP_CUBIC;
            else if (m == "LANCZOS4")
                d.interp = AEONB_INTERP_LANCZOS4;
            else
                throw std::invalid_argument("Provided interpolation method (" + p.interpolation_method + " is unrecognized.");
            d.src_w = src_w;
            d.src_h = src_h;
            if (p.expand_ratio > 1.0f)
            {
                d.canvas_w = p.expand_size.width;
                d.canvas_h = p.expand_size.height;
                d.canvas_x = p.expand_offset.width;
                d.canvas_y = p.expand_offset.height;
                if (src_w + d.canvas_x > d.canvas_w || src_h + d.canvas_y > d.canvas_h ||
                    (int64_t)d.canvas_x * d.canvas_y < 0)
                    throw std::invalid_argument("Invalid parameters to expand image");
            }
            else
            {
                d.canvas_w = src_w;
                d.canvas_h = src_h;
            }
            d.crop_x = p.cropbox.x;
            d.crop_y = p.cropbox.y;
            d.crop_w = p.cropbox.width;
            d.crop_h = p.cropbox.height;
            if (p.padding != 0 && !(p.padding_crop_offset.width == p.padding && p.padding_crop_offset.height == p.padding))
            {
                // add_padding (src/image.cpp:77-91): black border of `padding`, then a window of the cropped size
                if (p.expand_ratio > 1.0f || d.crop_x != 0 || d.crop_y != 0 || d.crop_w != src_w || d.crop_h != src_h)
                    throw error(AEONB_ERR_UNSUPPORTED, "'padding' together with a crop or expand is outside the accelerated path");
                d.canvas_w = src_w + 2 * p.padding;
                d.canvas_h = src_h + 2 * p.padding;
                d.canvas_x = d.canvas_y = p.padding;
                d.crop_x = p.padding_crop_offset.width;
                d.crop_y = p.padding_crop_offset.height;
            }
            d.out_w = p.output_size.width;
            d.out_h = p.output_size.height;
            if (exact_fit && (d.out_w != slot_w || d.out_h != slot_h))
                throw error(AEONB_ERR_UNSUPPORTED,
                            "output size differs from the configured size; set 'fixed_aspect_ratio' or enable cropping");
            d.flip = p.flip ? 1 : 0;
            set_photometric(d, p.contrast, p.brightness, p.saturation, p.hue, p.lighting.empty() ? nullptr : p.lighting.data(),
                            p.color_noise_std);
            return d;
        }

        // The geometry of an image descriptor as an INTER_AREA / INTER_CUBIC resize pass writing to dst.
        aeonb_resize_desc area_pass_of(const aeonb_image_desc& d, void* dst, int dst_pitch, int channels)
        {
            aeonb_resize_desc r{};
            r.channels         = channels;
            r.src              = d.src;
            r.src_pitch        = d.src_pitch;
            r.src_pixel_stride = d.src_pixel_stride;
            r.src_w            = d.src_w;
            r.src_h            = d.src_h;
            r.canvas_x         = d.canvas_x;
            r.canvas_y         = d.canvas_y;
            r.crop_x           = d.crop_x;
            r.crop_y           = d.crop_y;
            r.crop_w           = d.crop_w;
            r.crop_h           = d.crop_h;
            r.interp           = d.interp;
            r.out_w            = d.out_w;
            r.out_h            = d.out_h;
            r.dst              = static_cast<uint8_t*>(dst);
            r.dst_pitch        = dst_pitch;
            r.dst_pixel_stride = 3;
            return r;
        }

        const int16_t* wav_samples(const void* data, size_t size, size_t& count)
        {
            // Raw little-endian int16 samples, or a RIFF/WAVE file whose 'data' chunk holds them.
            const uint8_t* p = static_cast<const uint8_t*>(data);
            if (size >= 44 && !std::memcmp(p, "RIFF", 4) && !std::memcmp(p + 8, "WAVE", 4))
            {
                size_t pos = 12;
                while (pos + 8 <= size)
                {
                    uint32_t len;
                    std::memcpy(&len, p + pos + 4, 4);
                    if (!std::memcmp(p + pos, "fmt ", 4) && pos + 8 + 16 <= size)
                    {
                        uint16_t fmt, bits;
                        std::memcpy(&fmt, p + pos + 8, 2);
                        std::memcpy(&bits, p + pos + 8 + 14, 2);
                        if (fmt != 1 || bits != 16)
                            throw std::runtime_error("Unsupported number of bytes per sample: " + std::to_string(bits / 8));
                    }
                    if (!std::memcmp(p + pos, "data", 4))
                    {
                        count = std::min<size_t>(len, size - pos - 8) / 2;
                        return reinterpret_cast<const int16_t*>(p + pos + 8);
                    }
                    pos += 8 + len + (len & 1);
                }
                throw std::runtime_error("WAVE file without a data chunk");
            }
            count = size / 2;
            return reinterpret_cast<const int16_t*>(p);
        }
    }
}

aeonb_provider::~aeonb_provider()
{
    {
        std::lock_guard<std::mutex> lk(m_job_mutex);
        m_driver_stop = true; // the driver finishes what is queued, then leaves
    }
    m_job_cv.notify_all();
    if (m_driver.joinable())
        m_driver.join();
    for (cudaEvent_t e : m_done)
        if (e)
            cudaEventDestroy(e);
    for (cudaEvent_t e : m_kernels)
        if (e)
            cudaEventDestroy(e);
    for (auto& slot : m_trace)
        for (cudaEvent_t e : slot)
            if (e)
                cudaEventDestroy(e);
    for (int k = 0; k < k_sets; ++k)
        for (cudaEvent_t e : {m_uploaded[k], m_staged[k], m_consumed[k]})
            if (e)
                cudaEventDestroy(e);
    for (int k = 0; k < k_sets; ++k)
        for (cudaEvent_t e : {m_entropy_done[k], m_coef_free[k]})
            if (e)
                cudaEventDestroy(e);
    for (aeonb_ctx* e : m_entropy_ctx)
        if (e)
            aeonb_ctx_destroy(e);
    if (m_upload)
    {
        cudaStreamSynchronize(m_upload);
        cudaStreamDestroy(m_upload);
    }
    if (m_copy)
    {
        cudaStreamSynchronize(m_copy);
        cudaStreamDestroy(m_copy);
    }
}

namespace
{
    // Copy into the pinned staging buffer with stores that bypass the cache: the CPU never reads these bytes again (the
    // copy engine does), so they need not evict anything nor be read in before they are overwritten.
    inline void stream_copy(void* dst, const void* src, size_t n)
    {
#if defined(__SSE2__)
        static const bool plain = std::getenv("AEONB_PLAIN_STAGING_COPY") != nullptr;
        if (!plain && n >= 256)
        {
            // up to the first 16-byte boundary of dst the ordinary way
            const size_t head = (16 - (reinterpret_cast<uintptr_t>(dst) & 15)) & 15;
            std::memcpy(dst, src, head);
            n -= head;
            __m128i*       d = reinterpret_cast<__m128i*>(static_cast<char*>(dst) + head);
            const __m128i* s = reinterpret_cast<const __m128i*>(static_cast<const char*>(src) + head);
            const size_t   v = n / 64;
            for (size_t i = 0; i < v; ++i, d += 4, s += 4)
            {
                const __m128i a = _mm_loadu_si128(s), b = _mm_loadu_si128(s + 1), c = _mm_loadu_si128(s + 2), e = _mm_loadu_si128(s + 3);
                _mm_stream_si128(d, a);
                _mm_stream_si128(d + 1, b);
                _mm_stream_si128(d + 2, c);
                _mm_stream_si128(d + 3, e);
            }
            std::memcpy(d, s, n - v * 64);
            _mm_sfence();
            return;
        }
#endif
        std::memcpy(dst, src, n);
    }
}

void aeonb_provider::wait_ticket(int64_t t)
{
    {
        // may be called from another thread than the one that submits
        std::unique_lock<std::mutex> lk(m_job_mutex);
        if (t <= 0 || t > m_ticket)
            throw std::invalid_argument("aeonb_provider_wait: no such batch");
        if (m_ticket - t >= k_events)
            return; // its event slot was recycled, which only happens after the batch completed
        // the driver thread has enqueued (or given up on) the batch
        m_done_cv.wait(lk, [&] { return m_processed >= t; });
        if (m_failed[t % k_events])
        {
            std::exception_ptr e    = m_failed[t % k_events];
            m_failed[t % k_events] = nullptr;
            std::rethrow_exception(e);
        }
    }
    AEONB_CUDA(cudaSetDevice(ctx->device));
    AEONB_CUDA(cudaEventSynchronize(m_done[t % k_events]));
    if (m_trace[t % k_events][2] && std::getenv("AEONB_TRACE"))
    {
        float up_to_kernels = 0, kernels_to_done = 0, since_prev = 0;
        cudaEventElapsedTime(&up_to_kernels, m_trace[t % k_events][0], m_trace[t % k_events][1]);
        cudaEventElapsedTime(&kernels_to_done, m_trace[t % k_events][1], m_trace[t % k_events][2]);
        if (t >= 2 && m_trace[(t - 1) % k_events][2])
            cudaEventElapsedTime(&since_prev, m_trace[(t - 1) % k_events][2], m_trace[t % k_events][2]);
        float upload = 0, entropy = 0, rest = 0, ent_after_upload = 0;
        cudaEvent_t* e = m_trace[t % k_events];
        if (cudaEventQuery(e[4]) == cudaSuccess)
            cudaEventElapsedTime(&upload, e[3], e[4]);
        if (cudaEventQuery(e[6]) == cudaSuccess && cudaEventQuery(e[5]) == cudaSuccess)
        {
            cudaEventElapsedTime(&entropy, e[5], e[6]);
            cudaEventElapsedTime(&ent_after_upload, e[4], e[5]);
        }
        if (cudaEventQuery(e[7]) == cudaSuccess)
            cudaEventElapsedTime(&rest, e[7], e[1]);
        std::fprintf(stderr, "aeonb_provider_wait %lld: GPU upload+kernels %.3f ms, kernels->delivered %.3f ms, delivered after previous batch %.3f ms"
                             " | staging upload %.3f, upload end -> entropy begin %.3f, entropy %.3f, back end + image %.3f ms\n",
                     (long long)t, up_to_kernels, kernels_to_done, since_prev, upload, ent_after_upload, entropy, rest);
    }
    check_entropy_status((int)(t % k_events));
}

void aeonb_provider::check_entropy_status(int slot)
{
    const int32_t* status = static_cast<const int32_t*>(m_status[slot].p);
    const int      count  = m_status_count[slot];
    m_status_count[slot]  = 0;
    for (int i = 0; i < count; ++i)
        if (status[i] != 0)
            throw error(AEONB_ERR_DECODE, "Decoding image failed due to invalid data in the image file. (entropy-coded data of picture " +
                                              std::to_string(i) + " of the batch)");
}

void aeonb_provider::run(const void* const* elems, const size_t* sizes, int n, void* const* outs, bool on_device, bool wait)
{
    if (!elems || !sizes || !outs)
        throw std::invalid_argument("aeonb_provider_run: NULL argument");
    if (n <= 0 || n > batch_size)
        throw std::invalid_argument("aeonb_provider_run: record count must be in [1, batch_size]");
    const auto t0 = std::chrono::steady_clock::now();
    auto job = std::make_unique<batch_job>((int)stages.size());
    plan_records(job->plan, elems, sizes, n); // sequential planning pass (record order == RNG order), on the calling thread
    job->outs.assign(outs, outs + outputs.size());
    job->n         = n;
    job->on_device = on_device;
    job->plan_ms   = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    int64_t ticket;
    {
        std::unique_lock<std::mutex> lk(m_job_mutex);
        if (!m_driver.joinable())
            m_driver = std::thread([this] { driver_loop(); });
        m_done_cv.wait(lk, [&] { return m_ticket - m_processed < 2; }); // the driver is at most two batches behind
        ticket = job->ticket = ++m_ticket;
        m_jobs.push_back(std::move(job));
    }
    m_job_cv.notify_one();
    if (wait)
        wait_ticket(ticket);
}

void aeonb_provider::driver_loop()
{
    for (;;)
    {
        std::unique_ptr<batch_job> job;
        {
            std::unique_lock<std::mutex> lk(m_job_mutex);
            m_job_cv.wait(lk, [&] { return m_driver_stop || !m_jobs.empty(); });
            if (m_jobs.empty())
                return;
            job = std::move(m_jobs.front());
            m_jobs.pop_front();
        }
        const int          slot = (int)(job->ticket % k_events);
        std::exception_ptr failed;
        try
        {
            process(*job);
        }
        catch (...)
        {
            failed = std::current_exception();
        }
        {
            std::lock_guard<std::mutex> lk(m_job_mutex);
            m_failed[slot] = failed;
            m_processed    = job->ticket;
        }
        m_done_cv.notify_all();
    }
}

// Everything of a batch after planning, on the driver thread: memory, staging, launches, delivery.
void aeonb_provider::process(batch_job& job)
{
    batch_plan&   B         = job.plan;
    const int     n         = job.n;
    const bool    on_device = job.on_device;
    const int64_t T         = job.ticket;
    // AEONB_TRACE=1 prints the host time of each phase of the call to stderr
    static const bool trace = std::getenv("AEONB_TRACE") != nullptr;
    auto              t_prev = std::chrono::steady_clock::now();
    double            t_phase[6] = {0, job.plan_ms, 0, 0, 0, 0};
    auto mark = [&](int k) {
        const auto now = std::chrono::steady_clock::now();
        t_phase[k]     = std::chrono::duration<double, std::milli>(now - t_prev).count();
        t_prev         = now;
    };
    AEONB_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    if (!m_upload)
    {
        for (int k = 0; k < k_sets; ++k)
        {
            AEONB_CUDA(cudaEventCreateWithFlags(&m_uploaded[k], cudaEventDisableTiming));
            AEONB_CUDA(cudaEventCreateWithFlags(&m_staged[k], cudaEventDisableTiming));
            AEONB_CUDA(cudaEventCreateWithFlags(&m_consumed[k], cudaEventDisableTiming));
        }
        AEONB_CUDA(cudaStreamCreateWithFlags(&m_upload, cudaStreamNonBlocking));
        for (cudaEvent_t& e : m_done)
            AEONB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        for (cudaEvent_t& e : m_kernels)
            AEONB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        AEONB_CUDA(cudaStreamCreateWithFlags(&m_copy, cudaStreamNonBlocking));
        for (int k = 0; k < k_sets; ++k)
        {
            AEONB_CUDA(cudaEventCreateWithFlags(&m_entropy_done[k], cudaEventDisableTiming));
            AEONB_CUDA(cudaEventCreateWithFlags(&m_coef_free[k], cudaEventDisableTiming));
        }
        for (aeonb_ctx*& e : m_entropy_ctx)
            if (aeonb_ctx_create(ctx->device, nullptr, &e) != AEONB_OK)
                throw error(AEONB_ERR_CUDA, aeonb_last_error());
    }
    // Batch T writes its device-side outputs into buffer set `par`, last used by batch T - k_sets, whose copy to the
    // host may still be running on the copy stream: kernels wait for it.
    const int par = (int)(T % k_sets);
    if (!on_device && T > k_sets)
        AEONB_CUDA(cudaStreamWaitEvent(st, m_done[(T - k_sets) % k_events], 0));
    // The pinned staging set of this batch was last used k_sets batches ago: its copy to the device must have finished.
    if (m_staged_valid[par])
        AEONB_CUDA(cudaEventSynchronize(m_staged[par]));
    const int64_t launches_before = ctx->launches;
    h2d_bytes = d2h_bytes = 0;
    mark(0);
    const int trace_slot = (int)(T % k_events);
    if (trace)
    {
        for (cudaEvent_t& e : m_trace[trace_slot])
            if (!e)
                AEONB_CUDA(cudaEventCreate(&e));
        AEONB_CUDA(cudaEventRecord(m_trace[trace_slot][0], st));
        m_trace_slot = trace_slot;
    }
    reserve_arenas(B, job.outs.data(), on_device, par);
    mark(2);
    stage_inputs(B, par); // host work on the pool, uploads
    mark(3);
    launch_kernels(B, n, par);
    mark(4);
    deliver(B, job.outs.data(), n, on_device, par, T);
    launches = (int32_t)(ctx->launches - launches_before);
    if (trace)
    {
        mark(5);
        std::fprintf(stderr, "aeonb_provider_run: entry %.3f plan %.3f arenas %.3f stage %.3f kernels %.3f deliver %.3f ms\n", t_phase[0],
                     t_phase[1], t_phase[2], t_phase[3], t_phase[4], t_phase[5]);
    }
}

// Phase 1: parses headers, draws the augmentation parameters record by record (the order of the draws is the
// reference's) and plans every pass; host-produced outputs (labels, boxes) are written here.
void aeonb_provider::plan_records(batch_plan& B, const void* const* elems, const size_t* sizes, int n)
{
    const int nin = (int)stages.size();
    B.out_host.resize(outputs.size());
    for (size_t o = 0; o < outputs.size(); ++o)
        if (outputs[o].host_produced)
            B.out_host[o].assign((size_t)batch_size * outputs[o].shape.byte_size(), 0);

    // Parses the headers of one JPEG stream and registers it as a decode job (sizes only; no layout yet).
    auto plan_jpeg = [&](const void* data, size_t size) -> int {
        jpeg_job job;
        job.data = static_cast<const uint8_t*>(data);
        job.size = size;
        if (is_png(data, size))
        {
            png_parse(data, size, job.pinfo);
            job.png                    = true;
            job.pw                     = job.pinfo.width;
            job.ph                     = job.pinfo.height;
            job.frame.info.orientation = 1;
            B.jobs.push_back(job);
            return (int)B.jobs.size() - 1;
        }
        jpeg_parse(data, size, job.frame);
        const bool swapped = job.frame.info.orientation >= 5;
        job.pw             = swapped ? job.frame.info.height : job.frame.info.width;
        job.ph             = swapped ? job.frame.info.width : job.frame.info.height;
        B.jobs.push_back(job);
        return (int)B.jobs.size() - 1;
    };
    // Fixes the region of the picture a job has to produce -- the MCUs that the crop box of `d` (given in
    // canvas coordinates, the picture sitting at canvas_x/canvas_y) can touch, plus one chroma sample of
    // context -- and reserves its space in the staging buffer and in the pixel arena.  `d` == nullptr keeps
    // the whole picture.  A job shared by several descriptors (repeated video frame) keeps its first layout.
    auto layout_jpeg = [&](int j, const aeonb_image_desc* d) {
        jpeg_job& job = B.jobs[j];
        if (job.laid_out)
            return;
        if (job.png)
        {
            job.pitch       = (int)align_up((size_t)job.pw * 3, 16);
            job.stage_off   = align_up(B.stage_bytes, 256);
            job.stage_bytes = (size_t)job.pitch * job.ph;
            B.stage_bytes   = job.stage_off + job.stage_bytes;
            job.rw          = job.pw;
            job.rh          = job.ph;
            job.laid_out    = true;
            return;
        }
        const aeonb_jpeg_info& in = job.frame.info;
        const int mw = 8 * in.hs[0], mh = 8 * in.vs[0];
        const int mcux = in.blocks_w[0] / in.hs[0], mcuy = in.blocks_h[0] / in.vs[0];
        jpeg_roi roi{0, 0, mcux, mcuy};
        job.oriented = in.orientation != 1;
        if (job.oriented)
        {
            job.opitch     = (int)align_up((size_t)job.pw * 3, 16);
            job.opixel_off = align_up(B.oriented_bytes, 256);
            B.oriented_bytes = job.opixel_off + (size_t)job.opitch * job.ph;
        }
        else if (d && roi_decode) // a crop box that lies on the zero canvas only reads nothing of the picture: one MCU is kept
            roi = jpeg_roi_for_box(in, d->crop_x - d->canvas_x, d->crop_y - d->canvas_y, d->crop_x + d->crop_w - d->canvas_x,
                                   d->crop_y + d->crop_h - d->canvas_y);
        job.roi = roi;
        job.rx  = roi.mx0 * mw;
        job.ry  = roi.my0 * mh;
        job.rw  = std::min(in.width, roi.mx1 * mw) - job.rx;
        job.rh  = std::min(in.height, roi.my1 * mh) - job.ry;
        size_t off    = align_up(B.stage_bytes, 256);
        job.stage_off = off;
        off += 3 * 64 * sizeof(uint16_t);
        job.on_device = device_entropy && jpeg_entropy_prepare(job.frame, job.tables, job.edesc);
        if (job.on_device)
        {
            job.tables_off = off;
            off += sizeof job.tables;
            job.scan_off = align_up(off, 16);
            off          = job.scan_off + job.frame.scan_size;
        }
        for (int c = 0; c < in.ncomp; ++c)
        {
            job.roi_blocks_w[c] = (roi.mx1 - roi.mx0) * in.hs[c];
            job.roi_blocks_h[c] = (roi.my1 - roi.my0) * in.vs[c];
            const size_t bytes  = (size_t)job.roi_blocks_w[c] * job.roi_blocks_h[c] * 64 * sizeof(int16_t);
            if (job.on_device)
            {
                job.plane_dev_off[c] = align_up(B.coef_bytes, 256);
                B.coef_bytes           = job.plane_dev_off[c] + bytes;
            }
            else
            {
                off              = align_up(off, 256);
                job.plane_off[c] = off;
                off += bytes;
            }
        }
        if (job.on_device)
        {
            job.edesc.roi[0]  = std::max(roi.mx0, 0);
            job.edesc.roi[1]  = std::max(roi.my0, 0);
            job.edesc.roi[2]  = std::min(roi.mx1, mcux);
            job.edesc.roi[3]  = std::min(roi.my1, mcuy);
            job.scratch_bytes = (size_t)jpeg_entropy_scratch_bytes(job.edesc);
            job.scratch_off   = align_up(B.coef_bytes, 256);
            B.coef_bytes        = job.scratch_off + job.scratch_bytes;
        }
        job.stage_bytes = off - job.stage_off;
        B.stage_bytes     = off;
        job.pitch       = (int)align_up((size_t)job.rw * pixel_stride, 16);
        job.pixel_off   = align_up(B.pixel_bytes, 256);
        B.pixel_bytes     = job.pixel_off + (size_t)job.pitch * job.rh;
        job.laid_out    = true;
    };

    // Plans the passes one picture (an image record, or a video frame) goes through before the main image kernel
    // -- rotation (image::rotate, the first step of transform_single_image) and resize_short (applied to the whole,
    // possibly expanded, picture before the crop; src/etl_image.cpp:160-168) -- and returns the main descriptor.
    auto plan_picture = [&](int s, int j, const image_params& params, int slot_w, int slot_h, bool exact_fit) {
        struct
        {
            int width, height;
        } const in{B.jobs[j].pw, B.jobs[j].ph}; // the picture as delivered (after the EXIF turn)
        int rot = -1;
        if (params.angle != 0)
        {
            auto it = B.rotation_of_job.find(j);
            if (it != B.rotation_of_job.end())
                rot = it->second;
            else
            {
                batch_plan::rotation ro;
                ro.job        = j;
                ro.nearest    = B.jobs[j].mask;
                ro.angle      = params.angle;
                ro.pitch      = (int)align_up((size_t)in.width * 3, 16);
                ro.off        = align_up(B.rotated_bytes, 256);
                B.rotated_bytes = ro.off + (size_t)ro.pitch * in.height;
                rot           = (int)B.rotations.size();
                B.rotations.push_back(ro);
                B.rotation_of_job[j] = rot;
            }
            layout_jpeg(j, nullptr); // the rotation reads the whole picture
        }
        aeonb_image_desc d;
        int              pre = -1;
        if (params.resize_short_size != 0)
        {
            image_params whole = params;
            whole.resize_short_size = 0;
            whole.padding           = 0;
            whole.flip              = false;
            whole.contrast = whole.brightness = whole.saturation = 1.0f;
            whole.hue               = 0;
            whole.lighting.clear();
            const int cw = params.expand_ratio > 1.0f ? params.expand_size.width : in.width;
            const int ch = params.expand_ratio > 1.0f ? params.expand_size.height : in.height;
            whole.cropbox           = recti{0, 0, cw, ch};
            whole.output_size       = get_resized_short_size(cw, ch, params.resize_short_size);
            pre                     = (int)B.pre_descs[s].size();
            B.pre_descs[s].push_back(make_desc(whole, in.width, in.height, 0, 0, false));
            B.pre_job[s].push_back(j);
            B.pre_rot[s].push_back(rot);
            rot = -1;                // the crop pass reads the resized picture
            layout_jpeg(j, nullptr); // the resize pass reads the whole picture
            image_params rest = params;
            rest.resize_short_size = 0;
            rest.expand_ratio      = 1.0f;
            d = make_desc(rest, whole.output_size.width, whole.output_size.height, slot_w, slot_h, exact_fit);
        }
        else
        {
            d = make_desc(params, in.width, in.height, slot_w, slot_h, exact_fit);
            layout_jpeg(j, &d); // keeps an earlier whole-picture layout
        }
        B.desc_rot[s].push_back(rot);
        B.desc_pre[s].push_back(pre);
        int64_t area = -1;
        if (d.interp >= AEONB_INTERP_CUBIC &&
            (d.crop_w != d.out_w || d.crop_h != d.out_h)) // same size: aeon skips the resize
        {
            area         = (int64_t)align_up(B.area_bytes, 256);
            B.area_bytes = (size_t)area + align_up((size_t)d.out_w * 3, 16) * d.out_h;
        }
        B.desc_area[s].push_back(area);
        return d;
    };

    // ---- 0. SSD records: the annotation and the seeded patch sampling (up to a few hundred trial boxes, each checked
    // against every ground-truth box: about 20 us per record) are worked out ahead by a few threads.  Every record of a
    // chunk of decode_size records draws from an engine of its own and this is the only draw of such a record, so the draws
    // are what the sequential pass would have made.
    struct ssd_ahead
    {
        vector<bbox>       boxes;
        int                w = 0, h = 0;
        image_params       params;
        std::exception_ptr failure;
    };
    vector<ssd_ahead> ahead;
    // (not with lighting: std::normal_distribution keeps half of every pair it draws for the next call, which couples a
    // record's draws to the record before it)
    if (nin > 0 && stages[0].kind == stage_kind::ssd && n >= 8 && factory.lighting.stddev() == 0)
    {
        if (!plan_pool)
            plan_pool.reset(new worker_pool(3));
        ahead.resize(n);
        const stage& sg = stages[0];
        for (int first = 0; first < n; first += decode_size)
        {
            const int count = std::min(decode_size, n - first);
            plan_pool->start(count, [&, first](int i) {
                const int  r = first + i;
                ssd_ahead& a = ahead[r];
                try
                {
                    if (sizes[(size_t)r * nin] == 0)
                        return; // reported by the sequential pass, in record order
                    parse_ssd_annotation(elems[(size_t)r * nin], sizes[(size_t)r * nin], sg.class_map, a.w, a.h, a.boxes);
                    a.params = factory.make_ssd_params(engines[(slot_cursor + r) % decode_size], a.w, a.h, sg.ssd.width, sg.ssd.height,
                                                       a.boxes);
                }
                catch (...)
                {
                    a.failure = std::current_exception();
                }
            });
            plan_pool->help();
            plan_pool->wait();
        }
    }

    // ---- 1. sequential planning pass (record order == RNG order)
    for (int r = 0; r < n; ++r)
    {
        random_engine_t& engine = engines[(slot_cursor + r) % decode_size];
        bool             have_params = false;
        image_params     params;
        for (int s = 0; s < nin; ++s)
        {
            const stage& sg   = stages[s];
            const void*  data = elems[(size_t)r * nin + s];
            const size_t size = sizes[(size_t)r * nin + s];
            auto empty = [&](const char* what) {
                std::stringstream ss;
                ss << "received " << what << " with size 0, at idx " << r;
                throw std::runtime_error(ss.str());
            };
            switch (sg.kind)
            {
            case stage_kind::image:
            {
                if (size == 0)
                    empty("encoded image");
                const int  j  = plan_jpeg(data, size);
                if (sg.image.channels == 1)
                {
                    // IMREAD_GRAYSCALE: a JPEG gives its luma plane, a colour PNG goes through libpng's colour -> grey conversion
                    B.jobs[j].grey = true;
                }
                if (!have_params)
                {
                    params      = factory.make_params(engine, B.jobs[j].pw, B.jobs[j].ph, sg.image.width, sg.image.height);
                    have_params = true;
                }
                if (sg.image.channels == 1 && (params.brightness != 1.0f || params.saturation != 1.0f || params.hue != 0))
                    throw std::invalid_argument("brightness, saturation and hue need a 3-channel picture (cv::transform / cv::cvtColor "
                                                "reject one channel)");
                aeonb_image_desc d = plan_picture(s, j, params, sg.image.width, sg.image.height, !factory.fixed_aspect_ratio);
                if (d.out_w > sg.image.width || d.out_h > sg.image.height)
                    throw std::invalid_argument("transformed image does not fit the configured output size");
                B.descs[s].push_back(d);
                B.desc_job[s].push_back(j);
                B.desc_dst[s].push_back((int64_t)r * outputs[sg.first_output].shape.byte_size());
                break;
            }
            case stage_kind::mask:
            {
                // provider::pixelmask::provide (src/provider.cpp:365-394): the mask is read as one channel
                // (IMREAD_ANYDEPTH, src/etl_pixel_mask.cpp:39), shares the record's parameters and takes only their
                // geometry: rotation without interpolation, crop box, NEAREST resize, flip (src/etl_pixel_mask.cpp:62-92).
                if (size == 0)
                    empty("pixelmask");
                const int j = plan_jpeg(data, size);
                jpeg_job& job = B.jobs[j];
                if (job.png && job.pinfo.bit_depth == 16)
                    throw error(AEONB_ERR_UNSUPPORTED, "a 16-bit mask (kept at 16 bits by IMREAD_ANYDEPTH) is outside the accelerated path");
                job.grey = true;
                job.mask = true;
                if (!have_params)
                {
                    params      = factory.make_params(engine, job.pw, job.ph, sg.image.width, sg.image.height);
                    have_params = true;
                }
                image_params geometry;
                geometry.angle                = params.angle;
                geometry.cropbox              = params.cropbox;
                geometry.output_size          = params.output_size;
                geometry.flip                 = params.flip;
                geometry.interpolation_method = "NEAREST";
                // the crop box is taken from the rotated mask itself; cv::Mat refuses a window that leaves the picture
                const recti& cb = params.cropbox;
                if (cb.x < 0 || cb.y < 0 || cb.width <= 0 || cb.height <= 0 || cb.x + cb.width > job.pw || cb.y + cb.height > job.ph)
                    throw std::runtime_error("pixelmask: the crop box lies outside the mask picture");
                aeonb_image_desc d = plan_picture(s, j, geometry, sg.image.width, sg.image.height, !factory.fixed_aspect_ratio);
                if (d.out_w > sg.image.width || d.out_h > sg.image.height)
                    throw std::invalid_argument("transformed image does not fit the configured output size");
                B.descs[s].push_back(d);
                B.desc_job[s].push_back(j);
                B.desc_dst[s].push_back((int64_t)r * outputs[sg.first_output].shape.byte_size());
                break;
            }
            case stage_kind::video:
            {
                if (size == 0)
                    empty("encoded video");
                vector<avi_frame> frames = avi_mjpeg_frames(data, size);
                if (frames.empty())
                    throw std::runtime_error("Decoding video failed due to invalid data in the video file.");
                const image_config& fc = sg.video.frame;
                const int           T  = sg.video.max_frame_count;
                const int64_t       rec = outputs[sg.first_output].shape.byte_size();
                int                 prev = -1;
                vector<int>         frame_jobs;
                for (int t = 0; t < (int)frames.size() && t < T; ++t)
                {
                    if (frames[t].size == 0)
                    {
                        // a dropped-frame marker repeats the previous picture (src/cap_mjpeg_decoder.cpp:132-147)
                        if (prev < 0)
                            throw std::runtime_error("Decoding video failed due to invalid data in the video file.");
                    }
                    else
                        prev = plan_jpeg(frames[t].data, frames[t].size);
                    frame_jobs.push_back(prev);
                }
                const jpeg_job& first = B.jobs[frame_jobs[0]];
                if (!have_params)
                {
                    params      = video_factory.make_params(engine, first.pw, first.ph, fc.width, fc.height);
                    have_params = true;
                }
                for (int t = 0; t < T; ++t)
                {
                    aeonb_image_desc d{};
                    int              j = -1;
                    if (t < (int)frame_jobs.size())
                    {
                        j = frame_jobs[t];
                        d = plan_picture(s, j, params, fc.width, fc.height, true);
                    }
                    else
                    {
                        B.desc_rot[s].push_back(-1); // zero padding frame
                        B.desc_pre[s].push_back(-1);
                        B.desc_area[s].push_back(-1);
                    }
                    B.descs[s].push_back(d);
                    B.desc_job[s].push_back(j);
                    B.desc_dst[s].push_back((int64_t)r * rec + (int64_t)t * fc.height * fc.width);
                }
                break;
            }
            case stage_kind::ssd:
            {
                if (size == 0)
                    empty("localization_ssd data");
                vector<bbox> boxes;
                int          w = 0, h = 0;
                if (s == 0 && !ahead.empty())
                {
                    if (ahead[r].failure)
                        std::rethrow_exception(ahead[r].failure);
                    boxes.swap(ahead[r].boxes);
                    params      = ahead[r].params; // the first stage of the record: nothing has drawn parameters yet
                    have_params = true;
                }
                else
                {
                    parse_ssd_annotation(data, size, sg.class_map, w, h, boxes);
                    if (!have_params)
                    {
                        params      = factory.make_ssd_params(engine, w, h, sg.ssd.width, sg.ssd.height, boxes);
                        have_params = true;
                    }
                }
                vector<bbox> gt = transform_boxes_for_ssd(boxes, params);
                const int    o  = sg.first_output;
                const int    M  = sg.ssd.max_gt_boxes;
                int32_t* im_shape = reinterpret_cast<int32_t*>(B.out_host[o].data()) + (size_t)r * 2;
                float*   gtb      = reinterpret_cast<float*>(B.out_host[o + 1].data()) + (size_t)r * M * 4;
                int32_t* count    = reinterpret_cast<int32_t*>(B.out_host[o + 2].data()) + r;
                int32_t* cls      = reinterpret_cast<int32_t*>(B.out_host[o + 3].data()) + (size_t)r * M;
                int32_t* diff     = reinterpret_cast<int32_t*>(B.out_host[o + 4].data()) + (size_t)r * M;
                ssd_fill_buffers(gt, sg.ssd.width, sg.ssd.height, M, im_shape, gtb, count, cls, diff);
                break;
            }
            case stage_kind::bbox:
            {
                // provider::boundingbox::provide (src/provider.cpp:411-441) + boundingbox::loader::load
                // (src/etl_boundingbox.cpp:296-318): the first max_bbox_count transformed boxes, zero rows after them
                if (size == 0)
                    empty("boundingbox");
                vector<bbox> boxes;
                int          w = 0, h = 0;
                parse_ssd_annotation(data, size, sg.class_map, w, h, boxes);
                if (!have_params)
                {
                    params      = factory.make_params(engine, w, h, sg.bbox.width, sg.bbox.height);
                    have_params = true;
                }
                if (params.angle != 0) // the reference's transformer returns no boxes at all for a rotated record
                    throw std::invalid_argument("boundingbox does not support 'angle'");
                const vector<bbox> out   = transform_boxes_for_ssd(boxes, params);
                const int          o     = sg.first_output;
                float*             dst   = reinterpret_cast<float*>(B.out_host[o].data() + (size_t)r * outputs[o].shape.byte_size());
                const int          count = std::min<int>(sg.bbox.max_bbox_count, (int)out.size());
                for (int i = 0; i < count; ++i)
                {
                    dst[4 * i + 0] = out[i].xmin;
                    dst[4 * i + 1] = out[i].ymin;
                    dst[4 * i + 2] = out[i].xmax;
                    dst[4 * i + 3] = out[i].ymax;
                }
                break;
            }
            case stage_kind::rcnn:
            {
                // provider::localization::rcnn::provide (src/provider.cpp:254-287) and the host part of
                // transformer::transform (src/etl_localization_rcnn.cpp:97-125): scale, scaled picture size, boxes
                if (size == 0)
                    empty("localization_rcnn data");
                vector<bbox> boxes;
                int          w = 0, h = 0;
                parse_ssd_annotation(data, size, sg.class_map, w, h, boxes);
                if (!have_params)
                {
                    params      = factory.make_params(engine, w, h, sg.rcnn.width, sg.rcnn.height);
                    have_params = true;
                }
                rcnn_record rec;
                const int   cw = params.cropbox.width, ch = params.cropbox.height;
                rec.image_scale = factory.fixed_scaling_factor > 0 ? factory.fixed_scaling_factor
                                                                   : calculate_scale(cw, ch, sg.rcnn.width, sg.rcnn.height);
                rec.im_width  = unbiased_round((float)cw * rec.image_scale);
                rec.im_height = unbiased_round((float)ch * rec.image_scale);
                rec.gt_boxes  = transform_boxes_for_ssd(boxes, params);
                if (rec.gt_boxes.size() > 1024)
                    throw error(AEONB_ERR_UNSUPPORTED, "more than 1024 ground-truth boxes in a record is outside the accelerated path");
                B.rcnn[s].push_back(std::move(rec));
                break;
            }
            case stage_kind::label:
            {
                if (size == 0)
                    empty("encoded image"); // aeon reuses the image wording here (src/provider.cpp:207-212)
                int lbl;
                if (sg.label.binary)
                {
                    if (size != 4)
                    {
                        std::stringstream ss;
                        ss << "Only 4 byte buffers can be loaded as int32.  label_extractor::extract received " << size << " bytes";
                        throw std::runtime_error(ss.str());
                    }
                    std::memcpy(&lbl, data, 4);
                }
                else
                    lbl = std::stoi(string((const char*)data, size));
                const size_t esz = outputs[sg.first_output].shape.otype.size;
                std::memcpy(B.out_host[sg.first_output].data() + (size_t)r * esz, &lbl, std::min<size_t>(esz, 4));
                break;
            }
            case stage_kind::blob:
            {
                if (size == 0)
                    empty("blob");
                const size_t room = outputs[sg.first_output].shape.byte_size();
                if (size > room) // aeon copies without looking (src/etl_blob.hpp:98-102); a longer blob would overrun the buffer
                {
                    std::stringstream ss;
                    ss << "blob of " << size << " bytes does not fit the " << room << " bytes of its output buffer, at idx " << r;
                    throw std::runtime_error(ss.str());
                }
                std::memcpy(B.out_host[sg.first_output].data() + (size_t)r * room, data, size);
                break;
            }
            case stage_kind::audio:
            {
                if (size == 0)
                    empty("encoded audio");
                size_t         count   = 0;
                const int16_t* samples = wav_samples(data, size, count);
                const size_t   limit   = (size_t)(sg.audio.max_time_steps - 1) * sg.audio.frame_stride + sg.audio.frame_length;
                count                  = std::min(count, limit);
                const size_t off       = align_up(B.stage_bytes, 256);
                B.stage_bytes            = off + count * 2;
                B.copies.push_back(batch_plan::copy_job{samples, count * 2, off});
                aeonb_specgram_desc d{};
                d.n_samples = (int32_t)count;
                B.sdescs[s].push_back(d);
                B.sdesc_off[s].push_back(off);
                break;
            }
            }
        }
    }
    slot_cursor = (slot_cursor + n) % decode_size;

}

// Phase 2: grow-only arenas for everything the plan placed.
void aeonb_provider::reserve_arenas(batch_plan& B, void* const* outs, bool on_device, int par)
{
    // ---- 2. arenas
    staging[par].reserve(B.stage_bytes + 256);
    staging_dev[par].reserve(B.stage_bytes + 256);
    pixels_dev.reserve(B.pixel_bytes + 256);
    if (B.oriented_bytes > 0)
        oriented_dev.reserve(B.oriented_bytes + 256);
    if (B.rotated_bytes > 0)
        rotated_dev.reserve(B.rotated_bytes + 256);
    if (B.area_bytes > 0)
        area_dev.reserve(B.area_bytes + 256);
    B.status_room = align_up(sizeof(int32_t) * (B.jobs.size() + 1), 256);
    if (B.coef_bytes > 0)
        coef_dev[par].reserve(B.status_room + B.coef_bytes + 256);
    B.produced.assign(outputs.size(), nullptr); // where each device-produced output is written
    for (size_t o = 0; o < outputs.size(); ++o)
    {
        if (outputs[o].host_produced)
            continue;
        const size_t bytes = (size_t)batch_size * outputs[o].shape.byte_size();
        if (on_device && batch_major)
            B.produced[o] = static_cast<char*>(outs[o]);
        else
        {
            out_dev[par][o].reserve(bytes);
            B.produced[o] = static_cast<char*>(out_dev[par][o].p);
        }
        if (!batch_major)
            out_dev_t[par][o].reserve(bytes);
    }

}

// Phase 3: the worker pool fills the pinned staging buffer (compressed scans and tables, or coefficient planes when
// Huffman decoding runs on the host; audio samples), shipped to the device in slices while the pool is still working.
void aeonb_provider::stage_inputs(batch_plan& B, int par)
{
    cudaStream_t st = ctx->stream;
    // ---- 3. entropy decode on the pool, shipping finished slices while the rest decode
    char* const hstage = static_cast<char*>(staging[par].p);
    char* const dstage = static_cast<char*>(staging_dev[par].p);
    // the device copy of this set was read by the kernels of k_sets batches ago
    if (m_consumed_valid[par])
        AEONB_CUDA(cudaStreamWaitEvent(m_upload, m_consumed[par], 0));
    const int   njobs  = (int)B.jobs.size();
    const int   nwork  = njobs + (int)B.copies.size();
    if (nwork > 0)
    {
        const int                     groups = std::max(1, std::min(8, nwork));
        vector<std::atomic<int>>      remaining(groups);
        vector<int>                   first(groups + 1);
        for (int g = 0; g <= groups; ++g)
            first[g] = (int)((int64_t)nwork * g / groups);
        for (int g = 0; g < groups; ++g)
            remaining[g] = first[g + 1] - first[g];
        auto group_of = [&](int i) { return (int)(std::upper_bound(first.begin(), first.end(), i) - first.begin()) - 1; };
        auto offset_of = [&](int i) { return i < njobs ? B.jobs[i].stage_off : B.copies[i - njobs].stage_off; };
        std::exception_ptr failure;
        std::mutex         failure_mutex;
        // Jobs that only copy (scans and tables for the GPU's Huffman decoder, audio samples) are light: a few threads
        // finish them sooner than the whole pool, whose wake-up takes the cores from the thread that plans and launches
        // (measured with 256 records per batch and the batch left on the GPU: 195 k records/s with 3 threads, 105 k with 14).
        bool heavy = false;
        for (const jpeg_job& job : B.jobs)
            heavy |= job.png || !job.on_device;
        pool->start(nwork, [&](int i) {
            try
            {
                if (i < njobs)
                {
                    jpeg_job& job = B.jobs[i];
                    if (job.png)
                    {
                        png_decode_bgr(job.data, job.size, job.pinfo, reinterpret_cast<uint8_t*>(hstage + job.stage_off), job.pitch,
                                       job.grey);
                        remaining[group_of(i)].fetch_sub(1, std::memory_order_release);
                        return;
                    }
                    std::memcpy(hstage + job.stage_off, job.frame.quant, sizeof job.frame.quant);
                    if (job.on_device)
                    {
                        std::memcpy(hstage + job.tables_off, job.tables, sizeof job.tables);
                        stream_copy(hstage + job.scan_off, job.frame.scan, job.frame.scan_size);
                        remaining[group_of(i)].fetch_sub(1, std::memory_order_release);
                        return;
                    }
                    int16_t* planes[3] = {reinterpret_cast<int16_t*>(hstage + job.plane_off[0]),
                                          reinterpret_cast<int16_t*>(hstage + job.plane_off[1]),
                                          reinterpret_cast<int16_t*>(hstage + job.plane_off[2])};
                    jpeg_entropy_decode(job.frame, planes, &job.roi);
                }
                else
                {
                    const batch_plan::copy_job& c = B.copies[i - njobs];
                    stream_copy(hstage + c.stage_off, c.src, c.bytes);
                }
            }
            catch (...)
            {
                std::lock_guard<std::mutex> lk(failure_mutex);
                if (!failure)
                    failure = std::current_exception();
            }
            remaining[group_of(i)].fetch_sub(1, std::memory_order_release);
        }, !heavy);
        // the calling thread copies too (it is awake already), then ships the slices as their last job finishes
        pool->help();
        static const bool trace = std::getenv("AEONB_TRACE") != nullptr;
        if (trace && m_trace[m_trace_slot][3])
            AEONB_CUDA(cudaEventRecord(m_trace[m_trace_slot][3], m_upload));
        cudaError_t copy_error = cudaSuccess;
        for (int g = 0; g < groups; ++g)
        {
            for (int spin = 0; remaining[g].load(std::memory_order_acquire) > 0; ++spin)
                if (spin > 2000)
                    std::this_thread::sleep_for(std::chrono::microseconds(20));
            const size_t begin = offset_of(first[g]);
            const size_t end   = first[g + 1] < nwork ? offset_of(first[g + 1]) : B.stage_bytes;
            if (end > begin && copy_error == cudaSuccess && !failure)
            {
                copy_error = cudaMemcpyAsync(dstage + begin, hstage + begin, end - begin, cudaMemcpyHostToDevice, m_upload);
                h2d_bytes += (int64_t)(end - begin);
            }
        }
        pool->wait();
        if (failure)
            std::rethrow_exception(failure);
        AEONB_CUDA(copy_error);
    }
    {
        static const bool trace = std::getenv("AEONB_TRACE") != nullptr;
        if (trace && m_trace[m_trace_slot][4])
            AEONB_CUDA(cudaEventRecord(m_trace[m_trace_slot][4], m_upload));
    }
    AEONB_CUDA(cudaEventRecord(m_staged[par], m_upload));
    m_staged_valid[par] = true;
    AEONB_CUDA(cudaStreamWaitEvent(st, m_staged[par], 0)); // the kernels of this batch start once its inputs have arrived

}

// Phase 4: one launch per kernel for the whole batch.
void aeonb_provider::launch_kernels(batch_plan& B, int n, int par)
{
    cudaStream_t st     = ctx->stream;
    const int    nin    = (int)stages.size();
    const int    njobs  = (int)B.jobs.size();
    char* const  dstage = static_cast<char*>(staging_dev[par].p);
    // ---- 4. kernels
    B.n_device_jobs = 0;
    if (njobs > 0)
    {
        char* const cdev = static_cast<char*>(coef_dev[par].p);
        vector<aeonb_entropy_desc> ed;
        for (int i = 0; i < njobs; ++i)
        {
            const jpeg_job& job = B.jobs[i];
            if (!job.on_device)
                continue;
            aeonb_entropy_desc d = job.edesc;
            d.scan               = reinterpret_cast<const uint8_t*>(dstage + job.scan_off);
            d.tables             = reinterpret_cast<const uint8_t*>(dstage + job.tables_off);
            for (int c = 0; c < job.frame.info.ncomp; ++c)
                d.coef[c] = reinterpret_cast<int16_t*>(cdev + B.status_room + job.plane_dev_off[c]);
            d.scratch       = cdev + B.status_room + job.scratch_off;
            d.scratch_bytes = job.scratch_bytes;
            d.status        = reinterpret_cast<int32_t*>(cdev) + ed.size();
            ed.push_back(d);
        }
        B.n_device_jobs = (int)ed.size();
        if (B.n_device_jobs > 0)
        {
            // The entropy kernel runs on a stream of its own: it needs this batch's staged inputs and the coefficient set
            // that the back end of k_sets batches ago has read, nothing else -- so it runs beside the previous batch's back
            // end and image kernel, and (k_sets such streams, taken in turn) beside the last long streams of the previous
            // batch's entropy kernel: a launch lasts as long as its longest stream, the SMs of the others fall idle.  (With the per-kernel
            // profile on, everything stays on one stream: a timed kernel then runs alone.)
            static const bool own_stream = [] {
                const char* e = std::getenv("AEONB_ENTROPY_STREAM"); // 0: everything on the context's stream
                return !e || std::atoi(e) != 0;
            }();
            aeonb_ctx* ectx = ctx->profiling || !own_stream ? ctx : m_entropy_ctx[par];
            if (ectx != ctx)
            {
                AEONB_CUDA(cudaStreamWaitEvent(ectx->stream, m_staged[par], 0));
                if (m_coef_free_valid[par])
                    AEONB_CUDA(cudaStreamWaitEvent(ectx->stream, m_coef_free[par], 0));
            }
            static const bool trace = std::getenv("AEONB_TRACE") != nullptr;
            if (trace && m_trace[m_trace_slot][5])
                AEONB_CUDA(cudaEventRecord(m_trace[m_trace_slot][5], ectx->stream));
            check_status(aeonb_jpeg_entropy_batch(ectx, ed.data(), B.n_device_jobs));
            h2d_bytes += (int64_t)(sizeof(aeonb_entropy_desc) * B.n_device_jobs);
            if (trace && m_trace[m_trace_slot][6])
                AEONB_CUDA(cudaEventRecord(m_trace[m_trace_slot][6], ectx->stream));
            if (ectx != ctx)
            {
                ctx->launches += 1;
                AEONB_CUDA(cudaEventRecord(m_entropy_done[par], ectx->stream));
                AEONB_CUDA(cudaStreamWaitEvent(st, m_entropy_done[par], 0));
            }
        }
        {
            static const bool trace = std::getenv("AEONB_TRACE") != nullptr;
            if (trace && m_trace[m_trace_slot][7])
                AEONB_CUDA(cudaEventRecord(m_trace[m_trace_slot][7], st));
        }
        vector<aeonb_jpeg_desc> jd;
        jd.reserve(njobs);
        for (int i = 0; i < njobs; ++i)
        {
            const jpeg_job& job = B.jobs[i];
            if (job.png)
                continue; // already pixels
            const aeonb_jpeg_info& in = job.frame.info;
            jd.emplace_back();
            aeonb_jpeg_desc& d = jd.back();
            d.width  = job.rw;
            d.height = job.rh;
            d.ncomp  = job.grey ? 1 : in.ncomp;
            for (int c = 0; c < d.ncomp; ++c)
            {
                d.coef[c]     = job.on_device ? reinterpret_cast<const int16_t*>(cdev + B.status_room + job.plane_dev_off[c])
                                              : reinterpret_cast<const int16_t*>(dstage + job.plane_off[c]);
                d.quant[c]    = reinterpret_cast<const uint16_t*>(dstage + job.stage_off) + 64 * c;
                d.hs[c]       = job.grey ? 1 : in.hs[c];
                d.vs[c]       = job.grey ? 1 : in.vs[c];
                d.blocks_w[c] = job.roi_blocks_w[c];
                d.blocks_h[c] = job.roi_blocks_h[c];
            }
            d.dst              = static_cast<uint8_t*>(pixels_dev.p) + job.pixel_off;
            d.dst_pitch        = job.pitch;
            d.dst_pixel_stride = pixel_stride;
        }
        check_status(aeonb_jpeg_backend_batch(ctx, jd.data(), (int)jd.size()));
        h2d_bytes += (int64_t)(sizeof(aeonb_jpeg_desc) * jd.size());

    }
    // Where a decoded picture stands for the passes that read it: the decoded region, or the turned copy.
    struct picture
    {
        const uint8_t* p;
        int            pitch, stride, w, h, x, y; // (x, y): where the region's origin lies in the whole picture
    };
    auto picture_of = [&](int j) {
        const jpeg_job& job = B.jobs[j];
        if (job.png)
            return picture{reinterpret_cast<const uint8_t*>(dstage + job.stage_off), job.pitch, 3, job.pw, job.ph, 0, 0};
        if (job.oriented)
            return picture{static_cast<const uint8_t*>(oriented_dev.p) + job.opixel_off, job.opitch, 3, job.pw, job.ph, 0, 0};
        return picture{static_cast<const uint8_t*>(pixels_dev.p) + job.pixel_off, job.pitch, pixel_stride, job.rw, job.rh, job.rx, job.ry};
    };
    {
        vector<aeonb_orient_desc> od;
        for (const jpeg_job& job : B.jobs)
            if (job.oriented)
            {
                aeonb_orient_desc o{};
                o.src              = static_cast<const uint8_t*>(pixels_dev.p) + job.pixel_off;
                o.src_pitch        = job.pitch;
                o.src_pixel_stride = pixel_stride;
                o.width            = job.rw;
                o.height           = job.rh;
                o.orientation      = job.frame.info.orientation;
                o.dst              = static_cast<uint8_t*>(oriented_dev.p) + job.opixel_off;
                o.dst_pitch        = job.opitch;
                o.dst_pixel_stride = 3;
                od.push_back(o);
            }
        if (!od.empty())
        {
            check_status(aeonb_orient_batch(ctx, od.data(), (int)od.size()));
            h2d_bytes += (int64_t)(sizeof(aeonb_orient_desc) * od.size());
        }
    }
    if (!B.rotations.empty())
    {
        vector<aeonb_rotate_desc> rd(B.rotations.size());
        for (size_t i = 0; i < B.rotations.size(); ++i)
        {
            const batch_plan::rotation& ro  = B.rotations[i];
            const picture   pic = picture_of(ro.job);
            rd[i].src              = pic.p;
            rd[i].src_pitch        = pic.pitch;
            rd[i].src_pixel_stride = pic.stride;
            rd[i].width            = pic.w;
            rd[i].height           = pic.h;
            rd[i].angle            = ro.angle;
            rd[i].nearest          = ro.nearest ? 1 : 0;
            rd[i].dst              = static_cast<uint8_t*>(rotated_dev.p) + ro.off;
            rd[i].dst_pitch        = ro.pitch;
            rd[i].dst_pixel_stride = 3;
        }
        check_status(aeonb_rotate_batch(ctx, rd.data(), (int)rd.size()));
        h2d_bytes += (int64_t)(sizeof(aeonb_rotate_desc) * rd.size());
    }
    for (int s = 0; s < nin; ++s)
    {
        const stage& sg = stages[s];
        if (sg.kind == stage_kind::image || sg.kind == stage_kind::video || sg.kind == stage_kind::mask)
        {
            const bool          video = sg.kind == stage_kind::video;
            const image_config& ic    = video ? sg.video.frame : sg.image;
            const int           o     = sg.first_output;
            aeonb_image_layout  L{};
            L.slot_w   = ic.width;
            L.slot_h   = ic.height;
            L.channels = 3;
            if (video)
            {
                // video::loader::load always writes uint8 planes without a channel swap (src/etl_video.cpp:76-107)
                L.dtype    = AEONB_U8;
                L.stride_c = (int64_t)sg.video.max_frame_count * ic.height * ic.width;
                L.stride_y = ic.width;
                L.stride_x = 1;
                if (outputs[o].shape.otype.size != 1)
                    AEONB_CUDA(cudaMemsetAsync(B.produced[o], 0, (size_t)n * outputs[o].shape.byte_size(), st));
            }
            else
            {
                L.dtype      = ic.shape.otype.dtype;
                L.bgr_to_rgb = ic.bgr_to_rgb;
                if (ic.channel_major)
                {
                    L.stride_c = (int64_t)ic.height * ic.width;
                    L.stride_y = ic.width;
                    L.stride_x = 1;
                }
                else
                {
                    L.stride_c = 1;
                    L.stride_y = (int64_t)ic.width * ic.channels;
                    L.stride_x = ic.channels;
                }
                L.channels = ic.channels;
                if (!factory.mean.empty() && sg.kind == stage_kind::image) // the mask's loader gets no mean / stddev
                {
                    L.standardize = 1;
                    for (int c = 0; c < ic.channels; ++c)
                    {
                        const double sd = factory.stddev[c];
                        L.mean64[c]     = factory.mean[c];
                        L.rstd64[c]     = sd ? 1. / sd : 1.;
                        L.mean[c]       = (float)L.mean64[c];
                        L.rstd[c]       = (float)L.rstd64[c];
                    }
                }
            }
            const bool pre = !B.pre_descs[s].empty();
            size_t     pre_slot = 0;
            int        pre_pitch = 0;
            if (pre)
            {
                aeonb_image_layout P{};
                for (const aeonb_image_desc& d : B.pre_descs[s])
                {
                    P.slot_w = std::max(P.slot_w, d.out_w);
                    P.slot_h = std::max(P.slot_h, d.out_h);
                }
                P.channels = 3;
                P.dtype    = AEONB_U8;
                P.stride_c = 1;
                P.stride_x = 3;
                pre_pitch  = (int)align_up((size_t)P.slot_w * 3, 16);
                P.stride_y = pre_pitch;
                pre_slot   = align_up((size_t)pre_pitch * P.slot_h, 256);
                resized_dev.reserve(pre_slot * B.pre_descs[s].size());
                for (size_t i = 0; i < B.pre_descs[s].size(); ++i)
                {
                    aeonb_image_desc& d = B.pre_descs[s][i];
                    const int         j = B.pre_job[s][i];
                    const picture     pic = picture_of(j);
                    d.src               = pic.p;
                    d.src_pitch         = pic.pitch;
                    d.src_pixel_stride  = pic.stride;
                    if (B.pre_rot[s][i] >= 0)
                    {
                        d.src              = static_cast<const uint8_t*>(rotated_dev.p) + B.rotations[B.pre_rot[s][i]].off;
                        d.src_pitch        = B.rotations[B.pre_rot[s][i]].pitch;
                        d.src_pixel_stride = 3;
                    }
                    d.dst               = static_cast<char*>(resized_dev.p) + i * pre_slot;
                }
                if (B.pre_descs[s][0].interp >= AEONB_INTERP_CUBIC) // CUBIC, AREA, LANCZOS4; one method per configuration
                {
                    vector<aeonb_resize_desc> rd;
                    for (const aeonb_image_desc& d : B.pre_descs[s])
                        rd.push_back(area_pass_of(d, d.dst, pre_pitch, ic.channels));
                    check_status(aeonb_resize_batch(ctx, rd.data(), (int)rd.size()));
                    h2d_bytes += (int64_t)(sizeof(aeonb_resize_desc) * rd.size());
                }
                else
                {
                    check_status(aeonb_image_batch(ctx, B.pre_descs[s].data(), (int)B.pre_descs[s].size(), &P));
                    h2d_bytes += (int64_t)(sizeof(aeonb_image_desc) * B.pre_descs[s].size());
                }
            }
            for (size_t i = 0; i < B.descs[s].size(); ++i)
            {
                aeonb_image_desc& d = B.descs[s][i];
                const int         j = B.desc_job[s][i];
                d.dst               = B.produced[o] + B.desc_dst[s][i];
                if (B.desc_pre[s][i] >= 0)
                {
                    d.src              = static_cast<const uint8_t*>(resized_dev.p) + (size_t)B.desc_pre[s][i] * pre_slot;
                    d.src_pitch        = pre_pitch;
                    d.src_pixel_stride = 3;
                }
                else if (B.desc_rot[s][i] >= 0)
                {
                    d.src              = static_cast<const uint8_t*>(rotated_dev.p) + B.rotations[B.desc_rot[s][i]].off;
                    d.src_pitch        = B.rotations[B.desc_rot[s][i]].pitch;
                    d.src_pixel_stride = 3;
                }
                else if (j >= 0)
                {
                    // the decoded region stands where that part of the picture stands on the canvas
                    const picture pic  = picture_of(j);
                    d.src              = pic.p;
                    d.src_pitch        = pic.pitch;
                    d.src_pixel_stride = pic.stride;
                    d.src_w            = pic.w;
                    d.src_h            = pic.h;
                    d.canvas_x += pic.x;
                    d.canvas_y += pic.y;
                }
            }
            // INTER_AREA: the crop -> output resize is a pass of its own; the image kernel then reads its result 1:1
            vector<aeonb_resize_desc> area;
            for (size_t i = 0; i < B.descs[s].size(); ++i)
            {
                aeonb_image_desc& d = B.descs[s][i];
                if (d.interp < AEONB_INTERP_CUBIC)
                    continue;
                if (B.desc_area[s][i] < 0)
                {
                    d.interp = AEONB_INTERP_LINEAR; // same size: a copy
                    continue;
                }
                const int pitch = (int)align_up((size_t)d.out_w * 3, 16);
                uint8_t*  pic   = static_cast<uint8_t*>(area_dev.p) + B.desc_area[s][i];
                area.push_back(area_pass_of(d, pic, pitch, ic.channels));
                d.interp = AEONB_INTERP_LINEAR; // identity from here on
                d.src              = pic;
                d.src_pitch        = pitch;
                d.src_pixel_stride = 3;
                d.src_w = d.canvas_w = d.crop_w = d.out_w;
                d.src_h = d.canvas_h = d.crop_h = d.out_h;
                d.canvas_x = d.canvas_y = d.crop_x = d.crop_y = 0;
            }
            if (!area.empty())
            {
                check_status(aeonb_resize_batch(ctx, area.data(), (int)area.size()));
                h2d_bytes += (int64_t)(sizeof(aeonb_resize_desc) * area.size());
            }
            check_status(aeonb_image_batch(ctx, B.descs[s].data(), (int)B.descs[s].size(), &L));
            h2d_bytes += (int64_t)(sizeof(aeonb_image_desc) * B.descs[s].size());
        }
        else if (sg.kind == stage_kind::rcnn)
        {
            // one launch labels every anchor of every record; labels and best boxes come back for the host's sampling
            const size_t A = sg.anchors.size();
            const int    m = (int)B.rcnn[s].size();
            if (!rcnn_anchor_dev[s].p)
            {
                rcnn_anchor_dev[s].reserve(A * sizeof(box4));
                AEONB_CUDA(cudaMemcpyAsync(rcnn_anchor_dev[s].p, sg.anchors.data(), A * sizeof(box4), cudaMemcpyHostToDevice, st));
                AEONB_CUDA(cudaStreamSynchronize(st)); // the source is pageable memory owned by the stage
                h2d_bytes += (int64_t)(A * sizeof(box4));
            }
            const size_t per = align_up(A, 16) + align_up(A * sizeof(int16_t), 16); // labels, then best boxes
            rcnn_result_dev[s].reserve(per * m + 16);
            rcnn_result_host[s].reserve(per * m + 16);
            vector<box4>   gt;
            vector<size_t> first(m);
            for (int r = 0; r < m; ++r)
            {
                first[r] = gt.size();
                for (const bbox& b : B.rcnn[s][r].gt_boxes)
                    gt.push_back(box4{b.xmin, b.ymin, b.xmax, b.ymax});
            }
            gt.push_back(box4{0, 0, 0, 0}); // never empty
            const box4* gt_dev = static_cast<const box4*>(ctx->upload(gt.data(), gt.size() * sizeof(box4)));
            h2d_bytes += (int64_t)(gt.size() * sizeof(box4));
            vector<aeonb_rcnn_desc> rd(m);
            for (int r = 0; r < m; ++r)
            {
                const rcnn_record& rec = B.rcnn[s][r];
                char*              out = static_cast<char*>(rcnn_result_dev[s].p) + per * r;
                rd[r].gt_boxes  = reinterpret_cast<const float*>(gt_dev + first[r]);
                rd[r].n_gt      = (int32_t)rec.gt_boxes.size();
                rd[r].im_width  = rec.im_width;
                rd[r].im_height = rec.im_height;
                rd[r].labels    = reinterpret_cast<int8_t*>(out);
                rd[r].best_box  = reinterpret_cast<int16_t*>(out + align_up(A, 16));
            }
            check_status(aeonb_rcnn_label_batch(ctx, static_cast<const float*>(rcnn_anchor_dev[s].p), (int32_t)A, rd.data(), m,
                                                sg.rcnn.negative_overlap, sg.rcnn.positive_overlap));
            h2d_bytes += (int64_t)(sizeof(aeonb_rcnn_desc) * m);
            AEONB_CUDA(cudaMemcpyAsync(rcnn_result_host[s].p, rcnn_result_dev[s].p, per * m, cudaMemcpyDeviceToHost, st));
            d2h_bytes += (int64_t)(per * m);
        }
        else if (sg.kind == stage_kind::audio)
        {
            const int             o = sg.first_output;
            const bool            mel = sg.audio.feature_type != "specgram";
            aeonb_specgram_config cfg{sg.audio.frame_length, sg.audio.frame_stride, sg.audio.max_time_steps,
                                      mel ? sg.audio.num_filters : 0, sg.audio.sample_rate, sg.audio.window_code(),
                                      sg.audio.feature_type == "mfcc" ? sg.audio.num_cepstra : 0, 0};
            for (size_t i = 0; i < B.sdescs[s].size(); ++i)
            {
                B.sdescs[s][i].samples = reinterpret_cast<const int16_t*>(dstage + B.sdesc_off[s][i]);
                B.sdescs[s][i].dst     = reinterpret_cast<float*>(B.produced[o] + (int64_t)i * outputs[o].shape.byte_size());
            }
            check_status(aeonb_specgram_batch(ctx, B.sdescs[s].data(), (int)B.sdescs[s].size(), &cfg));
            h2d_bytes += (int64_t)(sizeof(aeonb_specgram_desc) * B.sdescs[s].size());
        }
    }
    // every kernel that reads the device copy of this staging set is now enqueued
    AEONB_CUDA(cudaEventRecord(m_consumed[par], st));
    m_consumed_valid[par] = true;
}

// Phase 5: host-produced outputs, transposes, copies to the host on the copy stream, completion event.
void aeonb_provider::deliver(batch_plan& B, void* const* outs, int n, bool on_device, int par, int64_t ticket)
{
    cudaStream_t st = ctx->stream;
    // ---- 5. deliver
    // localization_rcnn: the labels of the GPU pass are needed on the host now -- sampling draws from them and the ten
    // buffers are filled from the sample -- so a batch with such a stage waits for its kernels here.
    for (size_t s = 0; s < stages.size(); ++s)
    {
        const stage& sg = stages[s];
        if (sg.kind != stage_kind::rcnn)
            continue;
        AEONB_CUDA(cudaStreamSynchronize(st));
        const size_t A   = sg.anchors.size();
        const size_t per = align_up(A, 16) + align_up(A * sizeof(int16_t), 16);
        for (size_t r = 0; r < B.rcnn[s].size(); ++r)
        {
            const char*    res    = static_cast<const char*>(rcnn_result_host[s].p) + per * r;
            const int8_t*  labels = reinterpret_cast<const int8_t*>(res);
            const int16_t* best   = reinterpret_cast<const int16_t*>(res + align_up(A, 16));
            const vector<int> sampled = rcnn_sample_anchors(labels, (int)A, sg.rcnn.rois_per_image, sg.rcnn.foreground_fraction,
                                                            sg.rcnn.deterministic_sampling ? nullptr : &rcnn_engine);
            void* bufs[10];
            for (int k = 0; k < 10; ++k)
                bufs[k] = B.out_host[sg.first_output + k].data() + r * (size_t)outputs[sg.first_output + k].shape.byte_size();
            rcnn_load(sg.rcnn, sg.anchors, B.rcnn[s][r], labels, best, sampled, bufs);
        }
    }
    size_t small_total = 0;
    for (size_t o = 0; o < outputs.size(); ++o)
        if (outputs[o].host_produced && on_device)
            small_total += align_up(B.out_host[o].size(), 256);
    if (small_total > 0 && m_uploaded_valid[par])
        AEONB_CUDA(cudaEventSynchronize(m_uploaded[par])); // the small pinned set is reused too (last used k_sets batches ago)
    small_pinned[par].reserve(small_total + 256);
    size_t small_off = 0;
    for (size_t o = 0; o < outputs.size(); ++o)
    {
        const size_t  rec   = (size_t)outputs[o].shape.byte_size();
        const int     esz   = (int)outputs[o].shape.otype.size;
        const int64_t elems_per_rec = outputs[o].shape.element_count();
        if (outputs[o].host_produced)
        {
            vector<char>  tmp;
            const char*   src = B.out_host[o].data();
            if (!batch_major)
            {
                tmp.resize(B.out_host[o].size());
                for (int r = 0; r < batch_size; ++r)
                    for (int64_t e = 0; e < elems_per_rec; ++e)
                        std::memcpy(&tmp[((size_t)e * batch_size + r) * esz], src + ((size_t)r * elems_per_rec + e) * esz, esz);
                src = tmp.data();
            }
            const size_t bytes = batch_major ? rec * n : rec * batch_size;
            if (on_device)
            {
                char* pin = static_cast<char*>(small_pinned[par].p) + small_off;
                small_off += align_up(B.out_host[o].size(), 256);
                std::memcpy(pin, src, bytes);
                AEONB_CUDA(cudaMemcpyAsync(outs[o], pin, bytes, cudaMemcpyHostToDevice, st));
                h2d_bytes += (int64_t)bytes;
            }
            else
                std::memcpy(outs[o], src, bytes);
        }
    }
    if (small_total > 0)
    {
        AEONB_CUDA(cudaEventRecord(m_uploaded[par], st));
        m_uploaded_valid[par] = true;
    }
    // Recycling an event slot: the batch that used it (k_events submissions ago) is long complete once the
    // newer batches between were waited for; synchronise to make that certain.
    const int slot = (int)(ticket % k_events);
    AEONB_CUDA(cudaEventSynchronize(m_done[slot]));
    vector<void*> sources(outputs.size(), nullptr); // what is copied to the host, per device-produced output
    for (size_t o = 0; o < outputs.size(); ++o)
    {
        if (outputs[o].host_produced)
            continue;
        sources[o] = B.produced[o];
        if (!batch_major)
        {
            void* target = on_device ? outs[o] : out_dev_t[par][o].p;
            AEONB_CUDA(launch_transpose(B.produced[o], target, batch_size, outputs[o].shape.element_count(),
                                        (int)outputs[o].shape.otype.size, st));
            ctx->launches++;
            sources[o] = target;
        }
    }
    m_status_count[slot] = 0;
    if (B.n_device_jobs > 0)
    {
        // on the kernels' stream: the next batch's entropy kernel rewrites these words
        m_status[slot].reserve(sizeof(int32_t) * B.n_device_jobs);
        AEONB_CUDA(cudaMemcpyAsync(m_status[slot].p, coef_dev[par].p, sizeof(int32_t) * B.n_device_jobs, cudaMemcpyDeviceToHost, st));
        d2h_bytes += (int64_t)(sizeof(int32_t) * B.n_device_jobs);
        m_status_count[slot] = B.n_device_jobs;
        // from here on the entropy kernel of the batch after next may rewrite this coefficient set
        AEONB_CUDA(cudaEventRecord(m_coef_free[par], st));
        m_coef_free_valid[par] = true;
    }
    // Batches delivered to host memory are copied on a second stream, so that the next batch's uploads and
    // kernels do not queue behind this batch's (much longer) device -> host copy.
    cudaStream_t cs = st;
    if (!on_device)
    {
        cs = m_copy;
        AEONB_CUDA(cudaEventRecord(m_kernels[slot], st));
        AEONB_CUDA(cudaStreamWaitEvent(cs, m_kernels[slot], 0));
        for (size_t o = 0; o < outputs.size(); ++o)
        {
            if (outputs[o].host_produced)
                continue;
            const size_t bytes = (size_t)outputs[o].shape.byte_size() * (batch_major ? n : batch_size);
            AEONB_CUDA(cudaMemcpyAsync(outs[o], sources[o], bytes, cudaMemcpyDeviceToHost, cs));
            d2h_bytes += (int64_t)bytes;
        }
    }
    static const bool trace_gpu = std::getenv("AEONB_TRACE") != nullptr;
    if (trace_gpu && m_trace[slot][1])
    {
        AEONB_CUDA(cudaEventRecord(m_trace[slot][1], st));
        AEONB_CUDA(cudaEventRecord(m_trace[slot][2], cs));
    }
    AEONB_CUDA(cudaEventRecord(m_done[slot], cs));
}
