// The endless stream of encoded records behind the loader: aeon's manifest blocks -> block_loader_file ->
// block_manager chain (src/block_loader_file.cpp:45-117, src/block_manager.cpp:61-106) with the CPIO block cache
// (src/cache_system.cpp:69-146, src/cpio.cpp), as one pull-style object: the loader's producer thread asks for the
// next record and the stream loads, caches and shuffles whole blocks behind it, one block ahead of the consumer on a
// thread of its own (aeon runs these stages as async_manager threads, src/async_manager.hpp:91-117).
#pragma once

#include <condition_variable>
#include <cstdint>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "loader.hpp"

namespace aeonb
{
    typedef std::vector<std::vector<char>> encoded_record; // the elements of one record

    // One block of records as a CPIO archive in aeon's layout (src/cpio.cpp): old binary cpio members "cpiohdr" (64-byte
    // file header: "MACR", format 1, writer 1, data type, record count, elements per record), one member
    // "rec_NNNNNNN.EE" per element, "cpiotlr" (16 bytes) and "TRAILER!!!".
    void cpio_write_block(const std::string& path, const std::vector<encoded_record>& records);
    std::vector<encoded_record> cpio_read_block(const std::string& path, size_t elements_per_record);

    // aeon cache_system: a directory aeon_cache_<crc> under the cache root holding block_<n>.cpio files.  The process
    // that takes the lock file "caching_in_progress" writes the blocks during its first pass and marks the directory with
    // "cache_complete"; from then on every process reads blocks from the cache instead of the manifest's files.
    class block_cache
    {
    public:
        block_cache(uint32_t uid, size_t block_count, size_t elements_per_record, const std::string& root, bool shuffle, uint32_t seed);
        ~block_cache();
        bool is_complete() const { return m_stage == stage::complete; }
        bool is_ownership() const { return m_stage == stage::ownership; }
        void restart() { m_current = 0; }
        void try_get_access();
        std::vector<encoded_record> load_block();
        void store_block(const std::vector<encoded_record>& block);
        const std::string& directory() const { return m_dir; }

    private:
        enum class stage
        {
            complete,
            ownership,
            blocked
        };
        std::string block_path(size_t n) const;
        size_t              m_block_count, m_elements, m_current = 0;
        std::string         m_dir;
        bool                m_shuffle;
        std::minstd_rand0   m_random;
        std::vector<size_t> m_sequence;
        stage               m_stage = stage::blocked;
        int                 m_lock  = -1;
    };

    class block_stream
    {
    public:
        // `load` turns the manifest fields of one record into its elements (file reads, base64, ...)
        block_stream(manifest& m, const std::string& cache_root, bool shuffle, uint32_t seed,
                     std::function<void(const std::vector<std::string>&, encoded_record&)> load);
        encoded_record        next(); // the next record of the stream (moved out); loads the next block when one is used up
        void                  reset(); // aeon loader::reset: back to the first block; generators keep their state
        const block_cache*    cache() const { return m_cache.get(); }

        ~block_stream();

    private:
        enum class ahead
        {
            none,   // nothing asked for
            wanted, // the worker is loading the next block
            ready   // it is in m_next (or m_next_error says why not)
        };
        void                         next_block();
        std::vector<encoded_record>  load_block(); // worker thread only
        void                         worker();
        void                         request_block();
        void                         settle();
        manifest&                    m_manifest;
        std::function<void(const std::vector<std::string>&, encoded_record&)> m_load;
        bool                         m_shuffle;
        std::minstd_rand0            m_random;
        std::unique_ptr<block_cache> m_cache;
        size_t                       m_block_number = 0; // blocks read from the manifest in this pass
        size_t                       m_manifest_at  = 0; // position in the manifest's block sequence
        std::vector<encoded_record>  m_block;            // the block being handed out
        size_t                       m_at = 0;
        // one block ahead, loaded by a thread of its own
        std::thread                  m_worker;
        std::mutex                   m_mutex;
        std::condition_variable      m_cv;
        ahead                        m_state = ahead::none;
        bool                         m_quit  = false;
        std::vector<encoded_record>  m_next;
        std::exception_ptr           m_next_error;
    };
}
