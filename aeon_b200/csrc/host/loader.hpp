// Thin host shell that keeps aeon's loader surface on top of the provider:
// configuration keys and defaults of loader_config (src/loader.hpp:50-109), the TSV manifest
// (src/manifest_file.cpp:115-320), record loading (src/block_loader_file.cpp:45-117), the
// endless block stream with epoch wrap-around (src/block_manager.cpp:61-106) and the
// ONCE / INFINITE / COUNT position logic (src/loader.cpp:141-155,234-257).
// A producer thread reads records and submits batches to the provider's pipeline, a few output buffer sets ahead
// of the one the consumer holds, as aeon's async_manager stages do (src/async_manager.hpp:91-117).
#pragma once

#include <condition_variable>
#include <deque>
#include <exception>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "provider.hpp"

namespace aeonb
{
    enum class element_t
    {
        FILE,
        BINARY,
        STRING,
        ASCII_INT,
        ASCII_FLOAT
    };

    // aeon manifest_file (src/manifest_file.cpp): the record list of this node, cut into blocks, with the order in
    // which the blocks of the current epoch are read.
    struct manifest
    {
        std::vector<element_t>                   types;
        std::vector<std::vector<std::string>>    records; // this node's records (after subset, shuffle, node split)
        size_t                                   record_count = 0;
        uint32_t                                 crc          = 0; // CRC32C over all fields: the identity of a block cache
        std::vector<std::pair<size_t, size_t>>   blocks;          // [first, last) into records
        std::vector<size_t>                      block_sequence;  // block order of the current epoch
        void parse(std::istream& in, const std::string& root, float subset_fraction, bool shuffle, uint32_t seed, uint32_t node_id,
                   uint32_t node_count, int batch_size, int block_size);
        void reset(); // next epoch

    private:
        void generate();
        std::vector<std::vector<std::string>> m_all; // every record of the manifest (after subset)
        std::minstd_rand0                     m_random;
        bool                                  m_shuffle    = false;
        uint32_t                              m_node_id = 0, m_node_count = 0;
        int                                   m_batch_size = 1, m_block_size = 5000;
    };

    std::vector<size_t> node_record_indices(size_t total, uint32_t node_id, uint32_t node_count, int batch_size);
    std::vector<std::pair<size_t, size_t>> block_ranges(size_t record_count, size_t block_size);
    uint32_t crc32c_update(uint32_t crc, const void* data, size_t size);

    std::vector<char> base64_decode(const std::string& in);
    std::vector<int>  parse_cpu_list(const std::string& s);
}

namespace aeonb
{
    class block_stream;
}

struct aeonb_loader
{
    explicit aeonb_loader(const aeonb::json& cfg, int device);
    ~aeonb_loader();

    int  record_count() const { return (int)m_manifest.record_count; }
    int  batch_size() const { return m_batch_size; }
    int  batch_count() const { return m_batch_count; }
    int  position() const { return m_position; }
    int  next(void** buffers); // AEONB_OK or AEONB_END
    void reset();

    aeonb_provider*  provider() const { return m_provider; }
    std::string      config_text;
    std::vector<std::string> axis_text;

private:
    enum class slot_state
    {
        FREE,      // the producer may fill it
        SUBMITTED, // its batch is in the provider's pipeline (or failed before it got there: `error`)
        HELD       // handed out to the consumer until the next call
    };
    struct slot
    {
        std::vector<void*> buffers; // per output: pinned host or device memory for one batch
        std::exception_ptr error;
        slot_state         state  = slot_state::FREE;
        int64_t            ticket = 0;
        std::vector<std::vector<std::vector<char>>> held; // the batch's records: they stay put until the batch is complete
    };
    static constexpr int k_slots = 4;
    void producer();
    void start_producer();
    void stop_producer();

    aeonb::manifest m_manifest;
    aeonb_ctx*      m_ctx      = nullptr;
    aeonb_provider* m_provider = nullptr;
    int             m_device   = 0;
    int             m_batch_size = 0, m_batch_count = 0, m_position = 0;
    bool            m_infinite = false, m_device_output = false, m_shuffle = false;
    int             m_block_size = 5000;
    std::unique_ptr<aeonb::block_stream> m_stream; // the endless record stream (blocks, shuffle, CPIO cache)

    slot                    m_slots[k_slots];
    int                     m_consume = 0;  // slot the consumer reads next
    int                     m_held    = -1; // slot the consumer holds (released on the next call), or -1
    std::thread             m_thread;
    std::mutex              m_mutex;
    std::condition_variable m_cv;
    bool                    m_stop = false;
};

// The source side alone (manifest -> blocks -> cache -> shuffled record stream), host only.
struct aeonb_stream
{
    aeonb::manifest                       m;
    std::unique_ptr<aeonb::block_stream>  stream;
    std::vector<std::vector<char>>        held; // the record handed out by the last aeonb_stream_next
    ~aeonb_stream();
};
