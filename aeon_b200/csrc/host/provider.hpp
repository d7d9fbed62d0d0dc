// The provider: encoded records in host memory -> one augmented batch on the GPU.
//
// It plays the part of aeon's provider_base (src/provider.cpp:24-119) together with the
// per-slot random engines of batch_decoder (src/batch_decoder.cpp:47-71).  Per batch it
//   1. walks the records in order on one thread: parses headers, draws the augmentation
//      parameters from the record's slot engine (same draw order as the reference), parses
//      annotations / labels, and lays out one pinned staging buffer;
//   2. entropy-decodes all JPEG streams on a worker pool straight into that staging buffer,
//      shipping it to the GPU in slices while the pool is still decoding;
//   3. launches one JPEG back-end kernel and one image kernel per image-like stage
//      (plus the spectrogram kernel for audio stages);
//   4. delivers the outputs to device or host memory, transposed when batch_major is false.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <condition_variable>
#include <deque>
#include <exception>
#include <mutex>
#include <thread>
#include <vector>

#include "../specgram_host.hpp"
#include "config.hpp"
#include "jpeg_host.hpp"
#include "png_host.hpp"
#include "rcnn_host.hpp"
#include "params.hpp"
#include "runtime.hpp"

namespace aeonb
{
    enum class stage_kind
    {
        image,
        mask, // pixelmask: a one-channel target picture that follows the image's geometry
        label,
        blob, // bytes copied as they are (host only)
        video,
        ssd,
        audio,
        bbox, // boundingbox: the transformed boxes as rows of four floats (host only)
        rcnn // localization_rcnn: anchor labels on the GPU, sampling and the ten buffers on the host
    };

    struct stage
    {
        stage_kind   kind;
        int          first_output = 0; // index of the stage's first output buffer
        image_config image;
        label_config label;
        blob_config  blob;
        video_config video;
        ssd_config   ssd;
        audio_config audio;
        rcnn_config  rcnn;
        bbox_config  bbox;
        std::vector<box4> anchors; // localization_rcnn: the anchor table (anchor::generate), fixed per configuration
        std::unordered_map<std::string, int> class_map;
    };

    struct output_info
    {
        std::string name;
        shape_type  shape;
        std::string axes;          // comma separated axis names
        bool        host_produced; // small outputs computed on the CPU (labels, boxes)
    };

    // One JPEG stream to decode: where its bytes are and where its pieces live in the arenas.
    struct jpeg_job
    {
        const uint8_t* data = nullptr;
        size_t         size = 0;
        jpeg_frame     frame;
        size_t         stage_off = 0;    // quantiser tables, then the coefficient planes
        size_t         plane_off[3]{};   // offsets of the planes inside the staging buffer
        size_t         stage_bytes = 0;
        size_t         pixel_off = 0;    // decoded picture inside the pixel arena
        int            pitch = 0;
        // Region of MCUs that is actually decoded (the part of the picture the crop box can touch) and the
        // picture it yields: origin (rx, ry) in source pixels, size rw x rh, plane sizes in blocks.
        jpeg_roi       roi;
        bool           laid_out = false;
        int            rx = 0, ry = 0, rw = 0, rh = 0;
        int            roi_blocks_w[3]{}, roi_blocks_h[3]{};
        // Device entropy decoding: the staging buffer then carries the quantiser tables, the Huffman tables and the
        // scan bytes instead of coefficients; planes and the decoder's work area live in a device-only arena.
        // The picture as cv::imdecode delivers it: pw x ph after the EXIF orientation turn (sizes swapped for tags 5..8).
        // A turned picture is decoded whole and turned by a pass of its own into the orientation arena.
        int                pw = 0, ph = 0;
        // A PNG record: decoded on the pool straight into the staging buffer as a B,G,R picture (stage_off, pitch),
        // which the image kernel reads from the device copy; none of the JPEG fields apply.
        bool               png = false;
        png_info           pinfo;
        // A stage with "channels": 1 reads the picture as cv::imdecode(..., GRAYSCALE) delivers it: for a JPEG the luma
        // plane alone goes through the back end (B = G = R = Y), the chroma planes are decoded but not used.
        bool               grey = false;
        bool               mask = false; // a pixelmask record: rotated without interpolation
        bool               oriented = false;
        size_t             opixel_off = 0;
        int                opitch = 0;
        bool               on_device = false;
        aeonb_entropy_desc edesc{};
        uint8_t            tables[4 * 272]{};
        size_t             tables_off = 0, scan_off = 0;
        size_t             plane_dev_off[3]{};
        size_t             scratch_off = 0, scratch_bytes = 0;
    };
    // What one call of aeonb_provider::run plans before any GPU work: the JPEG streams to decode, the passes every
    // picture goes through, and where everything lives in the staging buffer and in the device arenas.
    struct batch_plan
    {
        struct copy_job // bytes copied as they are into the staging buffer (audio samples)
        {
            const void* src;
            size_t      bytes, stage_off;
        };
        // rotation pass (image::rotate, the first step of transform_single_image): whole decoded picture -> rotated copy
        struct rotation
        {
            int    job, angle, pitch;
            size_t off;
            bool   nearest = false; // a mask is rotated without interpolation
        };
        explicit batch_plan(int stages)
            : descs(stages), desc_job(stages), desc_dst(stages), pre_descs(stages), pre_job(stages), desc_rot(stages),
              pre_rot(stages), desc_pre(stages), desc_area(stages), rcnn(stages), sdescs(stages), sdesc_off(stages)
        {
        }
        std::vector<jpeg_job>                      jobs;
        std::vector<std::vector<char>>             out_host; // host-produced outputs of this batch (labels, boxes), per output
        std::vector<copy_job>                      copies;
        // per stage: main image-kernel descriptors, the JPEG job each reads (-1: zero frame) and its offset in the output
        std::vector<std::vector<aeonb_image_desc>> descs;
        std::vector<std::vector<int>>              desc_job;
        std::vector<std::vector<int64_t>>          desc_dst;
        std::vector<std::vector<aeonb_image_desc>> pre_descs; // resize_short pass: whole (expanded) picture -> short-side size
        std::vector<std::vector<int>>              pre_job;
        std::vector<rotation>                      rotations;
        std::unordered_map<int, int>               rotation_of_job; // a repeated video frame is rotated once
        std::vector<std::vector<int>>              desc_rot, pre_rot; // per descriptor: index into `rotations`, or -1
        std::vector<std::vector<int>>              desc_pre;          // per descriptor: index into pre_descs[s], or -1
        // INTER_AREA: the crop -> output resize runs as a pass of its own; the main kernel then reads a picture of the
        // output size 1:1.  Per descriptor: offset of that picture in the area arena, or -1.
        std::vector<std::vector<int64_t>>          desc_area;
        size_t                                     area_bytes = 0;
        std::vector<std::vector<rcnn_record>>      rcnn; // per stage: what transformer::transform leaves for the loader
        std::vector<std::vector<aeonb_specgram_desc>> sdescs;
        std::vector<std::vector<size_t>>           sdesc_off;
        size_t stage_bytes = 0, pixel_bytes = 0, coef_bytes = 0, oriented_bytes = 0, rotated_bytes = 0;
        size_t status_room   = 0; // bytes reserved for the entropy decoder's status words at the start of the coefficient arena
        int    n_device_jobs = 0; // streams Huffman-decoded on the GPU
        std::vector<char*> produced; // where each device-produced output is written
    };
}

struct aeonb_provider
{
    aeonb_ctx*                           ctx = nullptr;
    int                                  batch_size  = 0;
    int                                  decode_size = 0;
    uint32_t                             seed        = 0;
    bool                                 batch_major = true;
    bool                                 roi_decode  = true; // decode only the MCUs the crop box can touch
    bool                                 device_entropy = true; // Huffman-decode on the GPU ("entropy_decode": "device" | "host")
    int                                  pixel_stride = 3;
    std::vector<aeonb::stage>            stages;
    std::vector<aeonb::output_info>      outputs;
    aeonb::param_factory                 factory;       // augmentation[0]
    aeonb::param_factory                 video_factory; // augmentation[0]["frame"]
    std::vector<aeonb::random_engine_t>  engines;
    int                                  slot_cursor = 0;
    std::unique_ptr<aeonb::worker_pool>  pool;
    std::unique_ptr<aeonb::worker_pool>  plan_pool; // a few threads for the planning pass of the calling thread (SSD patch sampling)

    // Every per-batch buffer exists k_sets times, taken in turn (batch t uses set t % k_sets): a batch takes about two
    // kernel periods from its staging upload to its last kernel (upload -> entropy kernel -> back end -> image kernel), so
    // with three sets the upload and entropy kernel of batches t+1 and t+2 run beside the back end and image kernel of batch t.
    static constexpr int k_sets = 3;
    // Staging: compressed scans + tables (or coefficients) / decoded PNG pictures / samples: the host fills set p for
    // batch t while the upload stream still copies the set of batch t-1 and the kernels of batch t-1 read its device copy.
    aeonb::pinned_buffer                 staging[k_sets];
    aeonb::device_buffer                 staging_dev[k_sets];
    // device entropy decoding: status words, coefficient planes, work areas: the entropy kernel of batch t+1 (on a stream
    // of its own) runs beside the back end and image kernel of batch t, and beside the last long streams of batch t's own
    // entropy kernel
    aeonb::device_buffer                 coef_dev[k_sets];
    aeonb_ctx*                           m_entropy_ctx[k_sets] = {}; // contexts whose streams carry the entropy kernels, in turn
    cudaEvent_t                          m_entropy_done[k_sets] = {}; // planes of set p are complete
    cudaEvent_t                          m_coef_free[k_sets]    = {}; // the back end has read set p (batch t - k_sets)
    bool                                 m_coef_free_valid[k_sets] = {};
    aeonb::device_buffer                 pixels_dev;   // decoded pictures
    aeonb::device_buffer                 oriented_dev; // pictures after the EXIF orientation pass
    aeonb::device_buffer                 rotated_dev;  // pictures after the rotation pass
    aeonb::device_buffer                 resized_dev;  // pictures after the resize_short pass
    aeonb::device_buffer                 area_dev;     // pictures after an INTER_AREA crop -> output resize pass
    // localization_rcnn, per stage: the anchor table on the device, the labels / best-box arrays of the batch on the
    // device and their pinned host copies; one engine for the anchor sampling of all records
    std::vector<aeonb::device_buffer>    rcnn_anchor_dev, rcnn_result_dev;
    std::vector<aeonb::pinned_buffer>    rcnn_result_host;
    aeonb::random_engine_t               rcnn_engine;
    // Device-side outputs of batches delivered to host memory: the copy of batch t to the host (on the copy stream)
    // overlaps the kernels of the next batches, which write the other sets.
    std::vector<aeonb::device_buffer>    out_dev[k_sets];   // per output, batch_size records
    std::vector<aeonb::device_buffer>    out_dev_t[k_sets]; // transposed copies (batch_major == false)
    aeonb::pinned_buffer                 small_pinned[k_sets]; // host-produced outputs on their way to device memory

    static constexpr int k_events = 8;
    cudaEvent_t m_done[k_events]    = {}; // batch t complete: m_done[t % k_events]
    cudaEvent_t m_kernels[k_events] = {}; // the kernels of batch t have finished
    cudaStream_t m_copy             = nullptr; // device -> host copies of finished batches
    // AEONB_TRACE timing events per batch: 0 call start on the kernels' stream, 1 end of kernels, 2 end of delivery,
    // 3 / 4 first and last byte of the staging upload, 5 / 6 entropy kernel begin / end, 7 back end begin
    cudaEvent_t m_trace[k_events][8] = {};
    int         m_trace_slot = 0; // slot of the batch being enqueued
    cudaStream_t m_upload           = nullptr; // host -> device copies of the staging sets: they run under the previous batch's kernels
    cudaEvent_t m_staged[k_sets]         = {}; // staging set p has been copied to the device (upload stream)
    bool        m_staged_valid[k_sets]   = {};
    cudaEvent_t m_consumed[k_sets]       = {}; // the kernels that read the device copy of set p have finished
    bool        m_consumed_valid[k_sets] = {};
    cudaEvent_t m_uploaded[k_sets]       = {}; // small pinned set p has been copied
    bool        m_uploaded_valid[k_sets] = {};
    int64_t     m_ticket            = 0;       // number of batches submitted so far (calling thread)
    // A submitted batch is planned on the calling thread (headers, draws: the only phase that needs the records in
    // record order) and handed to the driver thread, which reserves memory, stages, launches and delivers one batch
    // at a time in submission order; the caller plans batch t+1 meanwhile.
    struct batch_job
    {
        explicit batch_job(int stages) : plan(stages) {}
        aeonb::batch_plan  plan;
        std::vector<void*> outs;
        int                n = 0;
        bool               on_device = false;
        int64_t            ticket = 0;
        double             plan_ms = 0;
    };
    std::thread                             m_driver;
    std::mutex                              m_job_mutex;
    std::condition_variable                 m_job_cv, m_done_cv;
    std::deque<std::unique_ptr<batch_job>>  m_jobs;
    int64_t                                 m_processed = 0; // last batch the driver has finished enqueuing (or failed on)
    bool                                    m_driver_stop = false;
    std::exception_ptr                      m_failed[k_events]; // what the driver threw for the batch of that slot
    void driver_loop();
    void process(batch_job& job);
    aeonb::pinned_buffer m_status[k_events];   // per in-flight batch: the device entropy decoder's status words
    int                  m_status_count[k_events] = {};
    void                 check_entropy_status(int slot); // throws aeon's decode error if a stream was malformed

    int64_t h2d_bytes = 0, d2h_bytes = 0;
    int32_t launches  = 0;

    aeonb_provider(aeonb_ctx* c, const aeonb::json& cfg);
    // Processes one batch.  With wait == false the call returns once the batch is planned and queued for the driver
    // thread; wait_ticket(ticket()) then blocks until that batch is complete.  Records and output buffers must stay
    // valid until then.  At most two batches wait for the driver: a third submission blocks until it has caught up.
    void    run(const void* const* elems, const size_t* sizes, int n, void* const* outs, bool on_device, bool wait = true);
    int64_t ticket() const { return m_ticket; }
    void    wait_ticket(int64_t t);
    ~aeonb_provider();
    int  input_count() const { return (int)stages.size(); }

private:
    // the phases of run()
    void plan_records(aeonb::batch_plan& plan, const void* const* elems, const size_t* sizes, int n);
    void reserve_arenas(aeonb::batch_plan& plan, void* const* outs, bool on_device, int par);
    void stage_inputs(aeonb::batch_plan& plan, int par);
    void launch_kernels(aeonb::batch_plan& plan, int n, int par);
    void deliver(aeonb::batch_plan& plan, void* const* outs, int n, bool on_device, int par, int64_t ticket);
};
