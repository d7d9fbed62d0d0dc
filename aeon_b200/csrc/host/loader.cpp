#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include "loader.hpp"
#include "block_stream.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <numeric>
#include <sstream>

using namespace aeonb;
using std::string;
using std::vector;

namespace
{
    const vector<string> k_loader_keys = {"manifest_filename", "manifest_root", "batch_size", "cache_directory", "block_size",
                                          "batch_major", "subset_fraction", "shuffle_enable", "shuffle_manifest", "cpu_list",
                                          "pinned", "random_seed", "iteration_mode", "iteration_mode_count", "etl",
                                          "augmentation", "node_id", "node_count", "ssd_config",
                                          // keys of this implementation
                                          "device_output", "decode_threads", "decode_size", "scratch_pixel_stride"};

    template <typename T>
    T get(const json& js, const char* key, T dflt)
    {
        const json* v = js.find(key);
        if (!v)
            return dflt;
        if constexpr (std::is_same<T, bool>::value)
            return v->as_bool();
        else if constexpr (std::is_same<T, string>::value)
            return v->as_string();
        else if constexpr (std::is_floating_point<T>::value)
            return (T)v->as_double();
        else
            return (T)v->as_int();
    }

    vector<char> read_file(const string& path)
    {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0)
            throw std::runtime_error("error opening file '" + path + "'");
        struct stat st;
        vector<char> data;
        if (::fstat(fd, &st) == 0 && st.st_size > 0)
        {
            data.resize((size_t)st.st_size);
            size_t at = 0;
            while (at < data.size())
            {
                const ssize_t got = ::read(fd, data.data() + at, data.size() - at);
                if (got <= 0)
                    break;
                at += (size_t)got;
            }
            data.resize(at);
        }
        ::close(fd);
        return data;
    }
}

namespace
{
    // The source side of the loader configuration (src/loader.hpp:77-106, src/loader.cpp:94-139): manifest, node split,
    // blocks, shuffle switches, cache directory.
    struct source_config
    {
        int      batch_size = 0, block_size = 5000;
        bool     shuffle_enable = false;
        uint32_t seed = 0, node_id = 0, node_count = 0;
        string   cache_directory;
    };

    source_config open_source(const json& cfg, manifest& m)
    {
        source_config sc;
        for (const char* k : {"manifest_filename", "batch_size"})
            if (!cfg.contains(k))
                throw std::invalid_argument(string("Required Argument: '") + k + "' not set");
        const string manifest_filename = get<string>(cfg, "manifest_filename", "");
        const string manifest_root     = get<string>(cfg, "manifest_root", "");
        sc.batch_size                  = get<int>(cfg, "batch_size", 0);
        if (sc.batch_size <= 0)
            throw std::invalid_argument("batch_size must be positive");
        sc.block_size = get<int>(cfg, "block_size", 5000);
        if (sc.block_size == 0)
            sc.block_size = 2 * sc.batch_size;
        const float subset = get<float>(cfg, "subset_fraction", 1.0f);
        if (!(subset <= 1.0f && subset >= 0.0f))
            throw std::invalid_argument("value for 'subset_fraction' out of range");
        sc.shuffle_enable           = get<bool>(cfg, "shuffle_enable", false);
        const bool shuffle_manifest = get<bool>(cfg, "shuffle_manifest", false);
        sc.seed                     = get<uint32_t>(cfg, "random_seed", 0);
        sc.node_id                  = get<uint32_t>(cfg, "node_id", 0);
        sc.node_count               = get<uint32_t>(cfg, "node_count", 0);
        sc.cache_directory          = get<string>(cfg, "cache_directory", "");
        if (sc.node_count > 1)
        {
            if (sc.node_id >= sc.node_count)
                throw std::runtime_error("node_id can't be greater than node_count");
            if (sc.seed == 0)
                sc.seed = 1; // aeon forces a seed for multi-node runs (src/loader.cpp:110-114)
        }
        std::ifstream in(manifest_filename);
        if (!in.is_open())
            throw std::runtime_error("Manifest file " + manifest_filename + " doesn't exist.");
        m.parse(in, manifest_root, subset, shuffle_manifest, sc.seed, sc.node_id, sc.node_count, sc.batch_size, sc.block_size);
        if (m.record_count == 0)
            throw std::runtime_error("manifest file is empty");
        return sc;
    }

    // aeon block_loader_file::filler (src/block_loader_file.cpp:56-104): the elements of one record
    void load_fields(const manifest& m, const vector<string>& fields, vector<vector<char>>& elems)
    {
        elems.clear();
        for (size_t j = 0; j < fields.size(); ++j)
        {
            const string& e = fields[j];
            switch (m.types[j])
            {
            case element_t::FILE: elems.push_back(read_file(e)); break;
            case element_t::BINARY: elems.push_back(base64_decode(e)); break;
            case element_t::STRING: elems.emplace_back(e.begin(), e.end()); break;
            case element_t::ASCII_INT:
            {
                int32_t v = (int32_t)std::stod(e);
                elems.emplace_back((char*)&v, (char*)&v + sizeof v);
                break;
            }
            case element_t::ASCII_FLOAT:
            {
                float v = std::stof(e);
                elems.emplace_back((char*)&v, (char*)&v + sizeof v);
                break;
            }
            }
        }
    }
}

aeonb_loader::aeonb_loader(const json& cfg, int device) : m_device(device)
{
    if (!cfg.contains("etl"))
        throw std::invalid_argument("Required Argument: 'etl' not set");
    for (const char* k : {"manifest_filename", "batch_size"})
        if (!cfg.contains(k))
            throw std::invalid_argument(string("Required Argument: '") + k + "' not set");
    verify_config("loader", k_loader_keys, cfg);
    const string mode       = get<string>(cfg, "iteration_mode", "ONCE");
    const int    mode_count = get<int>(cfg, "iteration_mode_count", 0);
    m_device_output         = get<bool>(cfg, "device_output", false);
    if (mode == "COUNT")
    {
        if (mode_count <= 0)
            throw std::invalid_argument("iteration_mode_count must be a positive integer");
    }
    else if (mode != "ONCE" && mode != "INFINITE")
        throw std::invalid_argument("iteration_mode must be one of ONCE, COUNT, or INFINITE");
    const source_config sc = open_source(cfg, m_manifest);
    m_batch_size           = sc.batch_size;
    m_block_size           = sc.block_size;
    m_shuffle              = sc.shuffle_enable;
    const uint32_t seed = sc.seed, node_id = sc.node_id;
    // block_manager and cache_system draw from generators of their own, seeded alike (src/block_manager.cpp:37,
    // src/cache_system.cpp:41)
    m_stream.reset(new block_stream(m_manifest, sc.cache_directory, m_shuffle, seed,
                                    [this](const vector<string>& fields, encoded_record& elems) { load_fields(m_manifest, fields, elems); }));

    m_batch_count = (int)((m_manifest.record_count + m_batch_size - 1) / m_batch_size);
    m_infinite    = mode == "INFINITE";
    if (mode == "COUNT")
        m_batch_count = mode_count;

    // Random-engine slots: aeon sizes its decode chunk from the worker-thread count (src/loader.cpp:159-164)
    json pcfg = cfg;
    if (!cfg.contains("decode_size"))
    {
        string cpu_list = get<string>(cfg, "cpu_list", "");
        if (const char* env = std::getenv("AEON_CPU_LIST"))
            if (*env)
                cpu_list = env;
        int threads = (int)parse_cpu_list(cpu_list).size();
        if (threads == 0)
            threads = default_worker_count();
        pcfg["decode_size"] = json((int64_t)m_batch_size * ((threads * 8 - 1) / m_batch_size + 1));
    }
    pcfg["random_seed"] = json((int64_t)(seed + node_id)); // src/loader.cpp:174
    if (seed == 0)
        pcfg["random_seed"] = json((int64_t)0);
    config_text = cfg.dump();

    if (aeonb_ctx_create(device, nullptr, &m_ctx) != AEONB_OK)
        throw error(AEONB_ERR_CUDA, aeonb_last_error());
    try
    {
        m_provider = new aeonb_provider(m_ctx, pcfg);
        if ((int)m_manifest.types.size() != m_provider->input_count())
            throw std::invalid_argument("the manifest has " + std::to_string(m_manifest.types.size()) +
                                        " elements per record but the etl list needs " + std::to_string(m_provider->input_count()));
        for (const auto& o : m_provider->outputs)
            axis_text.push_back(o.axes);
        for (slot& s : m_slots)
            for (const auto& o : m_provider->outputs)
            {
                void*        p     = nullptr;
                const size_t bytes = (size_t)m_batch_size * o.shape.byte_size();
                if (m_device_output)
                {
                    AEONB_CUDA(cudaMalloc(&p, bytes));
                    AEONB_CUDA(cudaMemset(p, 0, bytes));
                }
                else
                {
                    AEONB_CUDA(cudaMallocHost(&p, bytes));
                    std::memset(p, 0, bytes);
                }
                s.buffers.push_back(p);
            }
    }
    catch (...)
    {
        delete m_provider;
        aeonb_ctx_destroy(m_ctx);
        throw;
    }
    start_producer();
}

aeonb_loader::~aeonb_loader()
{
    stop_producer();
    cudaSetDevice(m_device);
    for (slot& s : m_slots)
        for (void* p : s.buffers)
            m_device_output ? cudaFree(p) : cudaFreeHost(p);
    delete m_provider;
    aeonb_ctx_destroy(m_ctx);
}

void aeonb_loader::start_producer()
{
    m_stop = false;
    for (slot& s : m_slots)
    {
        s.state = slot_state::FREE;
        s.error = nullptr;
    }
    m_consume = 0;
    m_held    = -1;
    m_thread  = std::thread([this] { producer(); });
}

void aeonb_loader::stop_producer()
{
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        m_stop = true;
    }
    m_cv.notify_all();
    if (m_thread.joinable())
        m_thread.join();
    // batches still in the provider's pipeline read this loader's records and write its buffers: let them finish
    for (slot& s : m_slots)
        if (s.state == slot_state::SUBMITTED && !s.error && s.ticket > 0)
        {
            try
            {
                m_provider->wait_ticket(s.ticket);
            }
            catch (...)
            {
            }
        }
}

void aeonb_loader::producer()
{
    cudaSetDevice(m_device);
    const int nin  = m_provider->input_count();
    int       fill = 0;
    for (;;)
    {
        {
            std::unique_lock<std::mutex> lk(m_mutex);
            m_cv.wait(lk, [&] { return m_stop || m_slots[fill].state == slot_state::FREE; });
            if (m_stop)
                return;
        }
        slot& s = m_slots[fill];
        s.ticket = 0;
        try
        {
            vector<const void*> elems((size_t)m_batch_size * nin);
            vector<size_t>      sizes((size_t)m_batch_size * nin);
            s.held.resize(m_batch_size);
            for (int r = 0; r < m_batch_size; ++r)
            {
                s.held[r] = m_stream->next();
                for (int e = 0; e < nin; ++e)
                {
                    elems[(size_t)r * nin + e] = s.held[r][e].data();
                    sizes[(size_t)r * nin + e] = s.held[r][e].size();
                }
            }
            // planned here, then staged and launched by the provider's driver thread while this thread reads the next batch
            m_provider->run(elems.data(), sizes.data(), m_batch_size, s.buffers.data(), m_device_output, false);
            s.ticket = m_provider->ticket();
        }
        catch (...)
        {
            s.error = std::current_exception();
        }
        {
            std::lock_guard<std::mutex> lk(m_mutex);
            s.state = slot_state::SUBMITTED;
        }
        m_cv.notify_all();
        fill = (fill + 1) % k_slots;
    }
}

int aeonb_loader::next(void** buffers)
{
    if (!m_infinite && m_position >= m_batch_count)
        return AEONB_END;
    std::unique_lock<std::mutex> lk(m_mutex);
    if (m_held >= 0)
    {
        m_slots[m_held].state = slot_state::FREE; // the batch handed out by the previous call is released now
        m_held                = -1;
        m_cv.notify_all();
    }
    slot& s = m_slots[m_consume];
    m_cv.wait(lk, [&] { return s.state == slot_state::SUBMITTED; });
    m_held    = m_consume;
    m_consume = (m_consume + 1) % k_slots;
    s.state   = slot_state::HELD;
    lk.unlock();
    if (s.error)
    {
        std::exception_ptr e = s.error;
        s.error              = nullptr;
        std::rethrow_exception(e);
    }
    m_provider->wait_ticket(s.ticket); // the batch is complete (throws what went wrong with it)
    for (size_t i = 0; i < s.buffers.size(); ++i)
        buffers[i] = s.buffers[i];
    m_position++;
    if (m_infinite && m_position == m_batch_count)
        m_position = 0;
    return AEONB_OK;
}

void aeonb_loader::reset()
{
    // restart the epoch from the first record of the data set (src/loader.hpp:205-210)
    stop_producer();
    m_stream->reset();
    m_position = 0;
    m_provider->slot_cursor = 0;
    start_producer();
}

extern "C" {

int aeonb_loader_create(const char* config_json, int device, aeonb_loader** out)
{
    return guarded([&]() {
        if (!config_json || !out)
            throw std::invalid_argument("aeonb_loader_create: NULL argument");
        *out = new aeonb_loader(json::parse(config_json), device);
        return AEONB_OK;
    });
}

void aeonb_loader_destroy(aeonb_loader* l)
{
    delete l;
}

int aeonb_loader_record_count(const aeonb_loader* l) { return l ? l->record_count() : 0; }
int aeonb_loader_batch_size(const aeonb_loader* l) { return l ? l->batch_size() : 0; }
int aeonb_loader_batch_count(const aeonb_loader* l) { return l ? l->batch_count() : 0; }
int aeonb_loader_output_count(const aeonb_loader* l) { return l ? aeonb_provider_output_count(l->provider()) : 0; }
const char* aeonb_loader_output_name(const aeonb_loader* l, int i) { return l ? aeonb_provider_output_name(l->provider(), i) : nullptr; }
int aeonb_loader_output_shape(const aeonb_loader* l, int i, int64_t* dims, int32_t* dtype)
{
    return l ? aeonb_provider_output_shape(l->provider(), i, dims, dtype) : fail(AEONB_ERR_INVALID, "loader is NULL");
}
const char* aeonb_loader_axis_names(const aeonb_loader* l, int i)
{
    if (!l || i < 0 || i >= (int)l->axis_text.size())
        return nullptr;
    return l->axis_text[i].c_str();
}
const char* aeonb_loader_config(const aeonb_loader* l) { return l ? l->config_text.c_str() : nullptr; }

int aeonb_loader_next(aeonb_loader* l, void** buffers)
{
    return guarded([&]() {
        if (!l || !buffers)
            throw std::invalid_argument("aeonb_loader_next: NULL argument");
        return l->next(buffers);
    });
}

int aeonb_loader_reset(aeonb_loader* l)
{
    return guarded([&]() {
        if (!l)
            throw std::invalid_argument("aeonb_loader_reset: loader is NULL");
        l->reset();
        return AEONB_OK;
    });
}

int aeonb_loader_position(const aeonb_loader* l) { return l ? l->position() : 0; }

int aeonb_stream_create(const char* config_json, aeonb_stream** out)
{
    return guarded([&]() {
        if (!config_json || !out)
            throw std::invalid_argument("aeonb_stream_create: NULL argument");
        std::unique_ptr<aeonb_stream> st(new aeonb_stream());
        const json          cfg = json::parse(config_json);
        const source_config sc  = open_source(cfg, st->m);
        aeonb_stream*       raw = st.get();
        st->stream.reset(new block_stream(st->m, sc.cache_directory, sc.shuffle_enable, sc.seed,
                                          [raw](const vector<string>& fields, encoded_record& elems) { load_fields(raw->m, fields, elems); }));
        *out = st.release();
        return AEONB_OK;
    });
}

void aeonb_stream_destroy(aeonb_stream* s) { delete s; }

int aeonb_stream_info(const aeonb_stream* s, int64_t* record_count, int32_t* elements_per_record, int32_t* block_count,
                      int32_t* cache_state, char* cache_dir, size_t cache_dir_size)
{
    return guarded([&]() {
        if (!s)
            throw std::invalid_argument("aeonb_stream_info: stream is NULL");
        if (record_count)
            *record_count = (int64_t)s->m.record_count;
        if (elements_per_record)
            *elements_per_record = (int32_t)s->m.types.size();
        if (block_count)
            *block_count = (int32_t)s->m.blocks.size();
        const block_cache* c = s->stream->cache();
        if (cache_state)
            *cache_state = !c ? 0 : c->is_complete() ? 3 : c->is_ownership() ? 2 : 1;
        if (cache_dir && cache_dir_size)
        {
            const string d = c ? c->directory() : string();
            std::strncpy(cache_dir, d.c_str(), cache_dir_size - 1);
            cache_dir[cache_dir_size - 1] = 0;
        }
        return AEONB_OK;
    });
}

int aeonb_stream_next(aeonb_stream* s, const void** elems, size_t* sizes)
{
    return guarded([&]() {
        if (!s || !elems || !sizes)
            throw std::invalid_argument("aeonb_stream_next: NULL argument");
        s->held = s->stream->next();
        for (size_t e = 0; e < s->held.size(); ++e)
        {
            elems[e] = s->held[e].data();
            sizes[e] = s->held[e].size();
        }
        return AEONB_OK;
    });
}

int aeonb_stream_reset(aeonb_stream* s)
{
    return guarded([&]() {
        if (!s)
            throw std::invalid_argument("aeonb_stream_reset: stream is NULL");
        s->stream->reset();
        return AEONB_OK;
    });
}

int64_t aeonb_node_record_indices(int64_t total, int node_id, int node_count, int batch_size, int64_t* out)
{
    if (total < 0 || batch_size <= 0 || node_id < 0 || (node_count > 1 && node_id >= node_count))
        return fail(AEONB_ERR_INVALID, "aeonb_node_record_indices: bad argument");
    const vector<size_t> idx = node_record_indices((size_t)total, (uint32_t)node_id, (uint32_t)std::max(node_count, 0), batch_size);
    if (out)
        for (size_t i = 0; i < idx.size(); ++i)
            out[i] = (int64_t)idx[i];
    return (int64_t)idx.size();
}

} // extern "C"
