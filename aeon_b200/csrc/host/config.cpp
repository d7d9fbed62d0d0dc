#include "config.hpp"
#include "rcnn_host.hpp"

#include <algorithm>
#include <sstream>
#include <stdexcept>

using namespace std;

namespace aeonb
{
    namespace
    {
        struct type_row
        {
            const char* name;
            int         dtype;
            size_t      size;
        };
        const type_row k_types[] = {{"int8_t", AEONB_I8, 1},   {"uint8_t", AEONB_U8, 1},   {"int16_t", AEONB_I16, 2},
                                    {"uint16_t", AEONB_U16, 2}, {"int32_t", AEONB_I32, 4}, {"uint32_t", AEONB_I32, 4},
                                    {"float", AEONB_F32, 4},   {"double", AEONB_F64, 8},   {"char", AEONB_I8, 1}};

        // classic two-row edit distance, used only for the "did you mean" hint
        int edit_distance(const string& s, const string& t)
        {
            if (s == t)
                return 0;
            if (s.empty())
                return (int)t.size();
            if (t.empty())
                return (int)s.size();
            vector<int> prev(t.size() + 1), cur(t.size() + 1);
            for (size_t i = 0; i <= t.size(); ++i)
                prev[i] = (int)i;
            for (size_t i = 0; i < s.size(); ++i)
            {
                cur[0] = (int)i + 1;
                for (size_t j = 0; j < t.size(); ++j)
                    cur[j + 1] = min({cur[j] + 1, prev[j + 1] + 1, prev[j] + (s[i] == t[j] ? 0 : 1)});
                prev.swap(cur);
            }
            return prev[t.size()];
        }

        void required(const json& js, const char* key)
        {
            if (!js.contains(key))
                throw invalid_argument(string("Required Argument: '") + key + "' not set");
        }
        int get_int(const json& js, const char* key, int dflt)
        {
            const json* v = js.find(key);
            return v ? (int)v->as_int() : dflt;
        }
        bool get_bool(const json& js, const char* key, bool dflt)
        {
            const json* v = js.find(key);
            return v ? v->as_bool() : dflt;
        }
        string get_string(const json& js, const char* key, const string& dflt)
        {
            const json* v = js.find(key);
            return v ? v->as_string() : dflt;
        }
        void check_output_type(const string& key, const string& v)
        {
            if (!output_type::is_valid(v))
                throw invalid_argument("value for '" + key + "' out of range");
        }
    }

    bool output_type::is_valid(const string& s)
    {
        for (const auto& r : k_types)
            if (s == r.name)
                return true;
        return false;
    }

    output_type output_type::from_name(const string& s)
    {
        for (const auto& r : k_types)
            if (s == r.name)
            {
                output_type o;
                o.name  = s;
                o.dtype = r.dtype;
                o.size  = r.size;
                return o;
            }
        throw runtime_error("Unable to map output type " + s);
    }

    void verify_config(const string&, const vector<string>& known, const json& js)
    {
        if (!js.is_object())
            return;
        for (const auto& kv : js.items())
        {
            if (find(known.begin(), known.end(), kv.first) != known.end())
                continue;
            int    distance = 1 << 30;
            string suggestion;
            for (const string& k : known)
            {
                int d = edit_distance(k, kv.first);
                if (d < distance)
                {
                    distance   = d;
                    suggestion = k;
                }
            }
            stringstream ss;
            ss << "config element {" << kv.first << ": " << kv.second.dump() << "} is not understood";
            if (distance < (int)(kv.first.size() / 2))
                ss << ", did you mean '" << suggestion << "'";
            throw invalid_argument(ss.str());
        }
    }

    image_config::image_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing image config in json config");
        js.erase("type");
        required(js, "height");
        required(js, "width");
        height           = get_int(js, "height", 0);
        width            = get_int(js, "width", 0);
        channels         = get_int(js, "channels", 3);
        channel_major    = get_bool(js, "channel_major", true);
        bgr_to_rgb       = get_bool(js, "bgr_to_rgb", false);
        output_type_name = get_string(js, "output_type", "uint8_t");
        name             = get_string(js, "name", "");
        if (channels != 1 && channels != 3)
            throw invalid_argument("value for 'channels' out of range");
        check_output_type("output_type", output_type_name);
        verify_config("image", {"height", "width", "channels", "channel_major", "bgr_to_rgb", "output_type", "name"}, js);
        shape.otype = output_type::from_name(output_type_name);
        if (channel_major)
        {
            shape.shape      = {channels, height, width};
            shape.axis_names = {"channels", "height", "width"};
        }
        else
        {
            shape.shape      = {height, width, channels};
            shape.axis_names = {"height", "width", "channels"};
        }
        if (width <= 0)
            throw invalid_argument("invalid width");
        if (height <= 0)
            throw invalid_argument("invalid height");
        if (bgr_to_rgb && channels != 3)
            throw invalid_argument("invalid config: bgr_to_rgb can be 'true' only for channels set to '3'");
    }

    label_config::label_config(json js)
    {
        js.erase("type");
        binary           = get_bool(js, "binary", false);
        output_type_name = get_string(js, "output_type", "uint32_t");
        name             = get_string(js, "name", "");
        check_output_type("output_type", output_type_name);
        verify_config("label", {"binary", "output_type", "name", "type"}, js);
        shape.otype = output_type::from_name(output_type_name);
        shape.shape = {1};
    }

    blob_config::blob_config(json js)
    {
        js.erase("type");
        required(js, "output_count");
        output_count     = get_int(js, "output_count", 0);
        output_type_name = get_string(js, "output_type", "float");
        name             = get_string(js, "name", "");
        check_output_type("output_type", output_type_name);
        verify_config("blob", {"output_count", "output_type", "name", "type"}, js);
        if (output_count <= 0)
            throw invalid_argument("blob: output_count must be positive");
        shape.otype = output_type::from_name(output_type_name);
        shape.shape = {(int64_t)output_count};
    }

    video_config::video_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing video config in json config");
        js.erase("type");
        required(js, "frame");
        frame = image_config(*js.find("frame"));
        required(js, "max_frame_count");
        max_frame_count = get_int(js, "max_frame_count", 0);
        name            = get_string(js, "name", "");
        verify_config("video", {"max_frame_count", "frame", "name"}, js);
        if (max_frame_count <= 0)
            throw invalid_argument("invalid max_frame_count");
        shape.otype      = frame.shape.otype;
        shape.shape      = {frame.channels, max_frame_count, frame.height, frame.width};
        shape.axis_names = {"channels", "frames", "height", "width"};
    }

    ssd_config::ssd_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing ssd config in json config");
        js.erase("type");
        required(js, "height");
        required(js, "width");
        required(js, "class_names");
        height       = get_int(js, "height", 0);
        width        = get_int(js, "width", 0);
        max_gt_boxes = get_int(js, "max_gt_boxes", 64);
        name         = get_string(js, "name", "");
        for (const json& c : js.find("class_names")->elements())
            class_names.push_back(c.as_string());
        verify_config("localization_ssd", {"height", "width", "class_names", "max_gt_boxes", "name"}, js);
        auto add = [&](vector<int64_t> s, const char* t) {
            shape_type st;
            st.shape = s;
            st.otype = output_type::from_name(t);
            shapes.push_back(st);
        };
        add({2, 1}, "int32_t");
        add({max_gt_boxes, 4}, "float");
        add({1, 1}, "int32_t");
        add({max_gt_boxes, 1}, "int32_t");
        add({max_gt_boxes, 1}, "int32_t");
        if (width <= 0)
            throw invalid_argument("invalid width");
        if (height <= 0)
            throw invalid_argument("invalid height");
        if (max_gt_boxes <= 0)
            throw invalid_argument("invalid max_gt_boxes");
        if (class_names.empty())
            throw invalid_argument("class_names cannot be empty");
    }

    bbox_config::bbox_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing bbox config in json config");
        js.erase("type");
        for (const char* key : {"height", "width", "max_bbox_count", "class_names"})
            required(js, key);
        height           = get_int(js, "height", 0);
        width            = get_int(js, "width", 0);
        max_bbox_count   = get_int(js, "max_bbox_count", 0);
        output_type_name = get_string(js, "output_type", "float");
        name             = get_string(js, "name", "");
        for (const json& c : js.find("class_names")->elements())
            class_names.push_back(c.as_string());
        check_output_type("output_type", output_type_name);
        verify_config("bbox", {"height", "width", "max_bbox_count", "class_names", "output_type", "name"}, js);
        if (max_bbox_count <= 0)
            throw invalid_argument("invalid max_bbox_count");
        shape.shape = {max_bbox_count, (int64_t)(4 * sizeof(float))};
        shape.otype = output_type::from_name(output_type_name);
    }

    rcnn_config::rcnn_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing localization_rcnn config in json config");
        js.erase("type");
        required(js, "height");
        required(js, "width");
        required(js, "class_names");
        height         = get_int(js, "height", 0);
        width          = get_int(js, "width", 0);
        name           = get_string(js, "name", "");
        rois_per_image = get_int(js, "rois_per_image", 256);
        base_size      = get_int(js, "base_size", 16);
        max_gt_boxes   = get_int(js, "max_gt_boxes", 64);
        deterministic_sampling = get_bool(js, "debug_deterministic", false);
        auto real = [&](const char* key, float dflt) {
            const json* v = js.find(key);
            return v ? (float)v->as_double() : dflt;
        };
        auto reals = [&](const char* key, vector<float>& out) {
            if (const json* v = js.find(key))
            {
                out.clear();
                for (const json& e : v->elements())
                    out.push_back((float)e.as_double());
            }
        };
        scaling_factor      = real("scaling_factor", scaling_factor);
        negative_overlap    = real("negative_overlap", negative_overlap);
        positive_overlap    = real("positive_overlap", positive_overlap);
        foreground_fraction = real("foreground_fraction", foreground_fraction);
        reals("ratios", ratios);
        reals("scales", scales);
        for (const json& c : js.find("class_names")->elements())
            class_names.push_back(c.as_string());
        verify_config("localization_rcnn",
                      {"height", "width", "class_names", "name", "rois_per_image", "base_size", "scaling_factor", "ratios", "scales",
                       "negative_overlap", "positive_overlap", "foreground_fraction", "max_gt_boxes", "debug_deterministic"},
                      js);
        for (const char* key : {"negative_overlap", "positive_overlap", "foreground_fraction"})
        {
            const float v = real(key, 0.5f);
            if (!(v >= 0.0f && v <= 1.0f))
                throw invalid_argument(string("value for '") + key + "' out of range");
        }
        if (width <= 0 || height <= 0 || base_size <= 0 || rois_per_image <= 0 || max_gt_boxes <= 0 || !(scaling_factor > 0))
            throw invalid_argument("localization_rcnn: sizes, base_size, rois_per_image, max_gt_boxes and scaling_factor must be positive");
        if (ratios.empty() || scales.empty() || ratios.size() > 8 || scales.size() > 8)
            throw invalid_argument("localization_rcnn: between 1 and 8 ratios and scales");
        const int64_t A = total_anchors();
        auto set = [&](int i, vector<int64_t> dims, const char* t) {
            shapes[i].shape = dims;
            shapes[i].otype = output_type::from_name(t);
        };
        // the ten buffers of localization::rcnn::config::config (src/etl_localization_rcnn.cpp:44-70)
        set(0, {A * 4}, "float");
        set(1, {A * 4}, "float");
        set(2, {1, A * 2}, "int32_t");
        set(3, {A * 2, 1}, "int32_t");
        set(4, {2, 1}, "int32_t");
        set(5, {max_gt_boxes, 4}, "float");
        set(6, {1, 1}, "int32_t");
        set(7, {max_gt_boxes, 1}, "int32_t");
        set(8, {1, 1}, "float");
        set(9, {max_gt_boxes, 1}, "int32_t");
    }

    int rcnn_config::total_anchors() const
    {
        return (int)(ratios.size() * scales.size()) * (int)std::floor((float)height * scaling_factor) *
               (int)std::floor((float)width * scaling_factor);
    }

    aeonb_rcnn_config rcnn_config::abi() const
    {
        aeonb_rcnn_config c{};
        c.width          = width;
        c.height         = height;
        c.base_size      = base_size;
        c.n_ratios       = (int)ratios.size();
        c.n_scales       = (int)scales.size();
        c.scaling_factor = scaling_factor;
        for (size_t i = 0; i < ratios.size(); ++i)
            c.ratios[i] = ratios[i];
        for (size_t i = 0; i < scales.size(); ++i)
            c.scales[i] = scales[i];
        return c;
    }

    audio_config::audio_config(json js)
    {
        if (js.is_null())
            throw runtime_error("missing audio config in json config");
        js.erase("type");
        frame_length   = get_int(js, "frame_length", 320);
        frame_stride   = get_int(js, "frame_stride", 160);
        max_time_steps = get_int(js, "max_time_steps", 0);
        max_samples    = get_int(js, "max_samples", 0);
        num_filters    = get_int(js, "num_filters", 64);
        sample_rate    = get_int(js, "sample_rate", 16000);
        window_type    = get_string(js, "window_type", "hann");
        feature_type   = get_string(js, "feature_type", "mfsc");
        num_cepstra    = get_int(js, "num_cepstra", 40);
        name           = get_string(js, "name", "");
        verify_config("audio",
                      {"frame_length", "frame_stride", "max_time_steps", "max_samples", "num_filters", "sample_rate",
                       "window_type", "feature_type", "num_cepstra", "name"},
                      js);
        if (frame_length <= 1 || frame_stride <= 0)
            throw invalid_argument("invalid frame_length or frame_stride");
        if (max_time_steps <= 0 && max_samples >= frame_length)
            max_time_steps = (max_samples - frame_length) / frame_stride + 1;
        if (max_time_steps <= 0)
            throw invalid_argument("audio config needs 'max_time_steps' or 'max_samples'");
        if (feature_type != "mfsc" && feature_type != "specgram" && feature_type != "mfcc")
            throw invalid_argument("feature_type must be 'specgram', 'mfsc' or 'mfcc'");
        if (feature_type == "mfcc" && (num_cepstra <= 0 || num_cepstra > num_filters))
            throw invalid_argument("num_cepstra <= cepsgram.cols"); // the reference's affirm (src/specgram.cpp:141)
        window_code();
        const int bins   = feature_type == "mfcc" ? num_cepstra : feature_type == "mfsc" ? num_filters : frame_length / 2 + 1;
        shape.otype      = output_type::from_name("float");
        shape.shape      = {max_time_steps, bins};
        shape.axis_names = {"time", "frequency"};
    }

    int audio_config::window_code() const
    {
        if (window_type == "none")
            return 0;
        if (window_type == "hann")
            return 1;
        if (window_type == "hamming")
            return 2;
        if (window_type == "blackman")
            return 3;
        if (window_type == "bartlett")
            return 4;
        throw runtime_error("Unsupported window function");
    }
}
