#include "provider.hpp"

#include <algorithm>
#include <cstring>
#include <sstream>

#include "avi.hpp"
#include "photometric.hpp"

using namespace aeonb;
using std::string;
using std::vector;

namespace aeonb
{
    std::vector<random_engine_t> make_slot_engines(uint32_t seed, int decode_size);
    cudaError_t launch_transpose(const void* src, void* dst, int64_t rows, int64_t cols, int elem_size, cudaStream_t stream);

    namespace
    {
        string join_axes(const shape_type& s)
        {
            string out;
            for (size_t i = 0; i < s.axis_names.size(); ++i)
                out += (i ? "," : "") + s.axis_names[i];
            return out;
        }

        string prefixed(const string& name, const string& base) { return name.empty() ? base : name + "." + base; }

    }

    // aeon boundingbox::extractor::extract (src/etl_boundingbox.cpp:64-132)
    void parse_ssd_annotation(const void* data, size_t size, const std::unordered_map<string, int>& classes, int& width,
                              int& height, vector<bbox>& boxes)
        {
            json j = json::parse(string((const char*)data, size));
            const json* objects = j.find("object");
            const json* sz      = j.find("size");
            if (!objects || objects->is_null())
                throw std::invalid_argument("'object' missing from metadata");
            if (!sz || sz->is_null())
                throw std::invalid_argument("'size' missing from metadata");
            for (const char* k : {"width", "height", "depth"})
                if (!sz->find(k) || sz->find(k)->is_null())
                    throw std::invalid_argument(string("'") + k + "' missing from metadata");
            height = (int)sz->find("height")->as_int();
            width  = (int)sz->find("width")->as_int();
            for (const json& o : objects->elements())
            {
                const json* bb = o.find("bndbox");
                for (const char* k : {"xmax", "xmin", "ymax", "ymin"})
                    if (!bb || !bb->find(k) || bb->find(k)->is_null())
                        throw std::invalid_argument(string("'") + k + "' missing from metadata");
                const json* nm = o.find("name");
                if (!nm || nm->is_null())
                    throw std::invalid_argument("'name' missing from metadata");
                auto it = classes.find(nm->as_string());
                if (it == classes.end())
                    throw std::invalid_argument("label '" + nm->as_string() + "' not found in class_names");
                bbox b;
                b.xmin      = (float)bb->find("xmin")->as_double();
                b.ymin      = (float)bb->find("ymin")->as_double();
                b.xmax      = (float)bb->find("xmax")->as_double();
                b.ymax      = (float)bb->find("ymax")->as_double();
                b.label     = it->second;
                const json* d = o.find("difficult");
                const json* t = o.find("truncated");
                b.difficult = d && !d->is_null() ? d->as_bool() : false;
                b.truncated = t && !t->is_null() ? t->as_bool() : false;
                boxes.push_back(b);
            }
        }

    // aeon boundingbox::transformer::transform_box (src/etl_boundingbox.cpp:146-261)
    vector<bbox> transform_boxes_for_ssd(const vector<bbox>& boxes, const image_params& p)
    {
        {
            const recti crop    = p.cropbox;
            const float x_scale = (float)p.output_size.width / (float)crop.width;
            const float y_scale = (float)p.output_size.height / (float)crop.height;
            vector<bbox> rc;
            for (bbox b : boxes)
            {
                if (p.expand_ratio > 1.)
                    b = bbox_expand(b, p.expand_offset, p.expand_size, p.expand_ratio);
                if (p.emit_constraint_type != emit_type::undefined)
                {
                    bbox cb;
                    cb.xmin = crop.x;
                    cb.ymin = crop.y;
                    cb.xmax = crop.x + crop.width - 1;
                    cb.ymax = crop.y + crop.height - 1;
                    bool keep;
                    if (p.emit_constraint_type == emit_type::center)
                    {
                        const float xc = b.xcenter(), yc = b.ycenter();
                        keep = xc >= cb.xmin && xc <= cb.xmax && yc >= cb.ymin && yc <= cb.ymax;
                    }
                    else
                        keep = bbox_coverage(b, cb) >= p.emit_min_overlap;
                    if (!keep)
                        continue;
                }
                if (b.xmax < crop.x || b.xmin >= crop.x + crop.width || b.ymax < crop.y || b.ymin >= crop.y + crop.height)
                    continue;
                b.xmin = b.xmin < crop.x ? 0 : b.xmin - crop.x;
                b.ymin = b.ymin < crop.y ? 0 : b.ymin - crop.y;
                b.xmax = b.xmax >= crop.x + crop.width ? crop.width - 1 : b.xmax - crop.x;
                b.ymax = b.ymax >= crop.y + crop.height ? crop.height - 1 : b.ymax - crop.y;
                if (p.flip)
                {
                    const float xmax = b.xmax;
                    b.xmax           = crop.width - b.xmin - 1;
                    b.xmin           = crop.width - xmax - 1;
                }
                b.xmin = b.xmin * x_scale;
                b.ymin = b.ymin * y_scale;
                b.xmax = (b.xmax + 1) * x_scale - 1;
                b.ymax = (b.ymax + 1) * y_scale - 1;
                rc.push_back(b);
            }
            return rc;
        }
    }
}

aeonb_provider::aeonb_provider(aeonb_ctx* c, const json& cfg) : ctx(c)
{
    if (!ctx)
        throw std::invalid_argument("provider needs a context");
    const json* etl = cfg.find("etl");
    if (!etl || !etl->is_array())
        throw std::invalid_argument("Required Argument: 'etl' not set");
    if (!cfg.contains("batch_size"))
        throw std::invalid_argument("Required Argument: 'batch_size' not set");
    batch_size = (int)cfg.find("batch_size")->as_int();
    if (batch_size <= 0)
        throw std::invalid_argument("batch_size must be positive");
    decode_size = cfg.contains("decode_size") ? (int)cfg.find("decode_size")->as_int() : batch_size;
    if (decode_size <= 0 || decode_size % batch_size != 0)
        throw std::invalid_argument("batch_decoder: decode_size have to be multiple of batch_size");
    seed        = cfg.contains("random_seed") ? (uint32_t)cfg.find("random_seed")->as_int() : 0;
    batch_major = cfg.contains("batch_major") ? cfg.find("batch_major")->as_bool() : true;
    if (cfg.contains("scratch_pixel_stride"))
        pixel_stride = (int)cfg.find("scratch_pixel_stride")->as_int();
    if (cfg.contains("roi_decode"))
        roi_decode = cfg.find("roi_decode")->as_bool();
    if (cfg.contains("entropy_decode"))
    {
        const std::string where = cfg.find("entropy_decode")->as_string();
        if (where != "device" && where != "host")
            throw std::invalid_argument("entropy_decode must be \"device\" or \"host\"");
        device_entropy = where == "device";
    }
    if (pixel_stride != 3 && pixel_stride != 4)
        throw std::invalid_argument("scratch_pixel_stride must be 3 or 4");
    int threads = cfg.contains("decode_threads") ? (int)cfg.find("decode_threads")->as_int() : default_worker_count();
    pool.reset(new worker_pool(threads));

    // only augmentation[0] is honoured (src/provider_factory.cpp:39-48)
    json aug;
    if (const json* a = cfg.find("augmentation"))
        if (a->is_array() && a->size() > 0)
            aug = a->elements()[0];
    factory = param_factory(aug);
    if (const json* f = aug.find("frame"))
        video_factory = param_factory(*f);

    // A seed of 0 means "non-deterministic" in aeon; the engines are then seeded from the clock source.
    uint32_t s = seed;
    if (s == 0)
        s = std::random_device{}();
    engines = make_slot_engines(s, decode_size);

    for (const json& e : etl->elements())
    {
        const json* type = e.find("type");
        if (!type)
            throw std::invalid_argument("missing required 'type' element in etl object");
        const string t = type->as_string();
        stage        st;
        st.first_output = (int)outputs.size();
        auto add = [&](const string& nm, const shape_type& sh, bool host) {
            outputs.push_back(output_info{nm, sh, join_axes(sh), host});
        };
        if (t == "image")
        {
            st.kind  = stage_kind::image;
            st.image = image_config(e);
            if (!factory.mean.empty() || !factory.stddev.empty())
            {
                const string& ot = st.image.output_type_name;
                if (!(ot == "float" || ot == "double"))
                    throw std::invalid_argument(
                        "Standardization (mean, stddev) is supported only for float or double 'output_type'.");
                if ((int)factory.mean.size() != st.image.channels || (int)factory.stddev.size() != st.image.channels)
                    throw std::invalid_argument("Size of 'mean' and 'stddev' must be equal to number of channels or empty.");
            }
            add(prefixed(st.image.name, "image"), st.image.shape, false);
        }
        else if (t == "pixelmask")
        {
            // provider::pixelmask (src/provider.cpp:353-394): an image config, the image loader without mean / stddev.
            // The extractor always yields one channel (src/etl_pixel_mask.cpp:39-55), and the loader's channel copy
            // only works when the configuration says so too.
            st.kind  = stage_kind::mask;
            st.image = image_config(e);
            if (st.image.channels != 1)
                throw std::invalid_argument("pixelmask: the decoded mask has one channel; set 'channels' to 1");
            add(prefixed(st.image.name, "pixelmask"), st.image.shape, false);
        }
        else if (t == "label")
        {
            st.kind  = stage_kind::label;
            st.label = label_config(e);
            add(prefixed(st.label.name, "label"), st.label.shape, true);
        }
        else if (t == "blob")
        {
            // provider::blob (src/provider.cpp:445-470)
            st.kind = stage_kind::blob;
            st.blob = blob_config(e);
            add(prefixed(st.blob.name, "blob"), st.blob.shape, true);
        }
        else if (t == "video")
        {
            st.kind  = stage_kind::video;
            st.video = video_config(e);
            if (st.video.frame.channels != 3)
                throw error(AEONB_ERR_UNSUPPORTED, "single-channel video output is outside the accelerated path");
            add(prefixed(st.video.name, "video"), st.video.shape, false);
        }
        else if (t == "localization_ssd")
        {
            st.kind = stage_kind::ssd;
            st.ssd  = ssd_config(e);
            for (size_t i = 0; i < st.ssd.class_names.size(); ++i)
                st.class_map.insert({st.ssd.class_names[i], (int)i});
            const char* names[5] = {"image_shape", "gt_boxes", "gt_box_count", "gt_class_count", "difficult_flag"};
            for (int i = 0; i < 5; ++i)
                add(prefixed(st.ssd.name, names[i]), st.ssd.shapes[i], true);
        }
        else if (t == "boundingbox")
        {
            // provider::boundingbox (src/provider.cpp:399-441)
            st.kind = stage_kind::bbox;
            st.bbox = bbox_config(e);
            for (size_t i = 0; i < st.bbox.class_names.size(); ++i)
                st.class_map.insert({st.bbox.class_names[i], (int)i});
            add(prefixed(st.bbox.name, "boundingbox"), st.bbox.shape, true);
        }
        else if (t == "localization_rcnn")
        {
            // provider::localization::rcnn (src/provider.cpp:220-287): ten buffers per record
            st.kind = stage_kind::rcnn;
            st.rcnn = rcnn_config(e);
            for (size_t i = 0; i < st.rcnn.class_names.size(); ++i)
                st.class_map.insert({st.rcnn.class_names[i], (int)i});
            st.anchors = rcnn_generate_anchors(st.rcnn.abi());
            const char* names[10] = {"bbtargets", "bbtargets_mask", "labels_flat", "labels_mask", "image_shape", "gt_boxes",
                                     "gt_box_count", "gt_class_count", "image_scale", "difficult_flag"};
            for (int i = 0; i < 10; ++i)
                add(prefixed(st.rcnn.name, names[i]), st.rcnn.shapes[i], true);
        }
        else if (t == "audio")
        {
            st.kind  = stage_kind::audio;
            st.audio = audio_config(e);
            add(prefixed(st.audio.name, "audio"), st.audio.shape, false);
        }
        else
        {
            std::stringstream ss;
            ss << "unsupported etl type '" << t << "'";
            throw std::invalid_argument(ss.str());
        }
        stages.push_back(std::move(st));
    }
    for (int k = 0; k < k_sets; ++k)
    {
        out_dev[k].resize(outputs.size());
        out_dev_t[k].resize(outputs.size());
    }
    rcnn_anchor_dev.resize(stages.size());
    rcnn_result_dev.resize(stages.size());
    rcnn_result_host.resize(stages.size());
    rcnn_engine.seed(s);
}
