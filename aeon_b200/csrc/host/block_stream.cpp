#include "block_stream.hpp"

#include <fcntl.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <thread>

using namespace std;

namespace aeonb
{
    namespace
    {
        // ---- old binary cpio member header: thirteen 16-bit fields, name (with its NUL) and data each padded to even length
        void put16(ostream& o, uint16_t v) { o.write(reinterpret_cast<const char*>(&v), 2); }
        void write_member_header(ostream& o, uint32_t size, const char* name)
        {
            const uint16_t namesize = (uint16_t)(strlen(name) + 1);
            const uint32_t mtime    = (uint32_t)time(nullptr);
            put16(o, 070707);
            put16(o, 0);       // dev
            put16(o, 0);       // ino
            put16(o, 0100644); // mode
            put16(o, 0);       // uid
            put16(o, 0);       // gid
            put16(o, 0);       // nlink
            put16(o, 0);       // rdev
            put16(o, (uint16_t)(mtime >> 16));
            put16(o, (uint16_t)mtime);
            put16(o, namesize);
            put16(o, (uint16_t)(size >> 16));
            put16(o, (uint16_t)size);
            o.write(name, namesize);
            if (namesize % 2)
                o.put(0);
        }

        void write_file_header(ostream& o, uint32_t record_count, uint32_t elements_field)
        {
            const uint32_t one = 1;
            o.write("MACR", 4);
            o.write(reinterpret_cast<const char*>(&one), 4); // format version
            o.write(reinterpret_cast<const char*>(&one), 4); // writer version
            o.write("        ", 8);                          // data type
            o.write(reinterpret_cast<const char*>(&record_count), 4);
            o.write(reinterpret_cast<const char*>(&elements_field), 4);
            const char unused[36] = {};
            o.write(unused, sizeof unused);
        }

        // fn(i) for i in [0, n) on a few threads of this call's own (a block is thousands of records: file reads and copies of
        // tens of kilobytes each); small jobs run on the calling thread.  The first exception is rethrown.
        template <typename F>
        void parallel_for(size_t n, size_t grain, F fn)
        {
            const size_t hw      = std::max(1u, thread::hardware_concurrency());
            const size_t threads = std::min<size_t>(std::min<size_t>(8, std::max<size_t>(1, hw / 2)), n / std::max<size_t>(grain, 1));
            if (threads <= 1)
            {
                for (size_t i = 0; i < n; ++i)
                    fn(i);
                return;
            }
            atomic<size_t>  next{0};
            exception_ptr   failure;
            mutex           failure_mutex;
            auto body = [&] {
                for (;;)
                {
                    const size_t first = next.fetch_add(grain);
                    if (first >= n)
                        return;
                    try
                    {
                        for (size_t i = first; i < std::min(n, first + grain); ++i)
                            fn(i);
                    }
                    catch (...)
                    {
                        lock_guard<mutex> lk(failure_mutex);
                        if (!failure)
                            failure = current_exception();
                        next.store(n);
                    }
                }
            };
            vector<thread> team;
            for (size_t t = 1; t < threads; ++t)
                team.emplace_back(body);
            body();
            for (thread& t : team)
                t.join();
            if (failure)
                rethrow_exception(failure);
        }

        bool exists(const string& path)
        {
            struct stat st;
            return stat(path.c_str(), &st) == 0;
        }
    }

    void cpio_write_block(const string& path, const vector<encoded_record>& records)
    {
        ofstream o(path, ios::binary);
        if (!o)
            throw runtime_error("cache system: unable to write cache file");
        write_member_header(o, 64, "cpiohdr");
        const streampos header_at = o.tellp();
        write_file_header(o, 0, 0);
        uint32_t element_index = 0; // aeon numbers the elements through the whole block (src/cpio.cpp:276-290)
        for (size_t r = 0; r < records.size(); ++r)
            for (const vector<char>& e : records[r])
            {
                char name[16];
                snprintf(name, sizeof name, "rec_%07d.%02d", (int)r, (int)element_index++);
                write_member_header(o, (uint32_t)e.size(), name);
                o.write(e.data(), (streamsize)e.size());
                if (e.size() % 2)
                    o.put(0);
            }
        write_member_header(o, 16, "cpiotlr");
        const char trailer[16] = {};
        o.write(trailer, sizeof trailer);
        write_member_header(o, 0, "TRAILER!!!");
        o.seekp(header_at);
        // aeon's writer stores the record count in both count fields (src/cpio.cpp:268-271); readers take the number of
        // elements per record from the loader configuration, not from the file
        write_file_header(o, (uint32_t)records.size(), (uint32_t)records.size());
        if (!o)
            throw runtime_error("cache system: unable to write cache file");
    }

    vector<encoded_record> cpio_read_block(const string& path, size_t elements_per_record)
    {
        // One walk over the member headers finds where every element lies; the elements are then read straight into their
        // vectors by several threads (the page cache hands a block out at memcpy speed, one thread does not keep up with
        // the GPU).
        struct file
        {
            int fd;
            ~file()
            {
                if (fd >= 0)
                    close(fd);
            }
        } f{open(path.c_str(), O_RDONLY)};
        if (f.fd < 0)
            throw runtime_error("cache system: cache file missed");
        struct stat st;
        if (fstat(f.fd, &st) != 0)
            throw runtime_error("cache system: cache file missed");
        const size_t file_size = (size_t)st.st_size;
        auto read_at = [&](void* dst, size_t size, size_t at) {
            size_t done = 0;
            while (done < size)
            {
                const ssize_t got = pread(f.fd, static_cast<char*>(dst) + done, size - done, (off_t)(at + done));
                if (got <= 0)
                    throw runtime_error("cache system: cache file corrupted");
                done += (size_t)got;
            }
        };
        // returns the data offset of the member that starts at `at`, its size in `size`, and moves `at` past it
        auto member = [&](size_t& at, uint32_t& size) -> size_t {
            uint16_t h[13];
            read_at(h, sizeof h, at);
            if (h[0] != 070707)
                throw runtime_error("CPIO header magic incorrect");
            const size_t namesize = h[10];
            size                  = (uint32_t)h[11] << 16 | h[12];
            const size_t data_at  = at + sizeof h + namesize + namesize % 2;
            if (data_at + size > file_size)
                throw runtime_error("cache system: cache file corrupted");
            at                    = data_at + size + size % 2;
            return data_at;
        };
        size_t       at   = 0;
        uint32_t     size = 0;
        const size_t header_at = member(at, size);
        if (size != 64)
            throw runtime_error("unexpected header size.  expected 64 found " + to_string(size));
        char head[24];
        read_at(head, sizeof head, header_at);
        if (strncmp(head, "MACR", 4) != 0)
            throw runtime_error("Unrecognized format\n");
        uint32_t record_count = 0;
        memcpy(&record_count, head + 20, 4);
        if (record_count == 0)
            throw runtime_error("cache system: cache file corrupted");
        struct span
        {
            size_t   at;
            uint32_t size;
        };
        vector<span> spans((size_t)record_count * elements_per_record);
        for (span& sp : spans)
            sp.at = member(at, sp.size);
        vector<encoded_record> out(record_count);
        parallel_for(record_count, 16, [&](size_t r) {
            out[r].resize(elements_per_record);
            for (size_t e = 0; e < elements_per_record; ++e)
            {
                const span& sp = spans[r * elements_per_record + e];
                out[r][e].resize(sp.size);
                read_at(out[r][e].data(), sp.size, sp.at);
            }
        });
        return out;
    }

    // ------------------------------------------------------------------------------------------------

    block_cache::block_cache(uint32_t uid, size_t block_count, size_t elements_per_record, const string& root, bool shuffle, uint32_t seed)
        : m_block_count(block_count)
        , m_elements(elements_per_record)
        , m_shuffle(shuffle)
        , m_random(seed ? seed : random_device{}())
    {
        m_sequence.resize(block_count);
        for (size_t i = 0; i < block_count; ++i)
            m_sequence[i] = i;
        char name[32];
        snprintf(name, sizeof name, "aeon_cache_%08x", uid);
        m_dir = root.empty() || root.back() == '/' ? root + name : root + "/" + name;
        if (!exists(m_dir) && mkdir(m_dir.c_str(), 0777) != 0 && !exists(m_dir))
            throw runtime_error("error making directory " + m_dir);
        try_get_access();
    }

    block_cache::~block_cache()
    {
        if (is_ownership() && m_lock >= 0)
        {
            remove((m_dir + "/caching_in_progress").c_str());
            close(m_lock);
        }
    }

    void block_cache::try_get_access()
    {
        m_current = 0;
        m_stage   = stage::complete;
        if (exists(m_dir + "/cache_complete"))
            return;
        if (m_lock < 0)
        {
            const mode_t mask = umask(0);
            m_lock            = open((m_dir + "/caching_in_progress").c_str(), O_RDWR | O_CREAT, 0666);
            umask(mask);
            if (m_lock >= 0 && flock(m_lock, LOCK_EX | LOCK_NB) < 0)
            {
                close(m_lock);
                m_lock = -1;
            }
        }
        m_stage = m_lock >= 0 ? stage::ownership : stage::blocked;
    }

    string block_cache::block_path(size_t n) const { return m_dir + "/block_" + to_string(n) + ".cpio"; }

    vector<encoded_record> block_cache::load_block()
    {
        vector<encoded_record> block = cpio_read_block(block_path(m_sequence[m_current]), m_elements);
        if (m_shuffle)
            std::shuffle(block.begin(), block.end(), m_random);
        if (++m_current == m_block_count)
        {
            m_current = 0;
            if (m_shuffle)
                std::shuffle(m_sequence.begin(), m_sequence.end(), m_random);
        }
        return block;
    }

    void block_cache::store_block(const vector<encoded_record>& block)
    {
        cpio_write_block(block_path(m_current), block);
        if (++m_current == m_block_count)
        {
            m_current = 0;
            // the cache is whole: mark it and give the lock back
            ofstream mark(m_dir + "/cache_complete");
            mark.close();
            remove((m_dir + "/caching_in_progress").c_str());
            close(m_lock);
            m_lock  = -1;
            m_stage = stage::complete;
            if (m_shuffle)
                std::shuffle(m_sequence.begin(), m_sequence.end(), m_random);
        }
    }

    // ------------------------------------------------------------------------------------------------

    block_stream::block_stream(manifest& m, const string& cache_root, bool shuffle, uint32_t seed,
                               function<void(const vector<string>&, encoded_record&)> load)
        : m_manifest(m)
        , m_load(std::move(load))
        , m_shuffle(shuffle)
        , m_random(seed ? seed : random_device{}())
    {
        if (!cache_root.empty())
            m_cache.reset(new block_cache(m.crc, m.blocks.size(), m.types.size(), cache_root, shuffle, seed));
    }

    block_stream::~block_stream()
    {
        {
            lock_guard<mutex> lk(m_mutex);
            m_quit = true;
        }
        m_cv.notify_all();
        if (m_worker.joinable())
            m_worker.join();
    }

    // The worker loads one block ahead: asked for block k+1 at the moment block k is handed to the consumer (so the order
    // of loads, cache writes and shuffles -- and with it every generator's state -- is the same as without it).
    void block_stream::worker()
    {
        for (;;)
        {
            {
                unique_lock<mutex> lk(m_mutex);
                m_cv.wait(lk, [&] { return m_quit || m_state == ahead::wanted; });
                if (m_quit)
                    return;
            }
            vector<encoded_record> block;
            exception_ptr          failure;
            try
            {
                block = load_block();
            }
            catch (...)
            {
                failure = current_exception();
            }
            {
                lock_guard<mutex> lk(m_mutex);
                m_next       = std::move(block);
                m_next_error = failure;
                m_state      = ahead::ready;
            }
            m_cv.notify_all();
        }
    }

    void block_stream::request_block()
    {
        {
            lock_guard<mutex> lk(m_mutex);
            if (!m_worker.joinable())
                m_worker = thread([this] { worker(); });
            m_state = ahead::wanted;
        }
        m_cv.notify_all();
    }

    // Waits for the block being loaded, if any; what it produced (or threw) stays in m_next / m_next_error.
    void block_stream::settle()
    {
        unique_lock<mutex> lk(m_mutex);
        m_cv.wait(lk, [&] { return m_state != ahead::wanted; });
    }

    void block_stream::reset()
    {
        // every stage of aeon's chain starts over (src/async_manager.hpp:119-131): the manifest deals a new block order
        // when it shuffles, the block manager and the cache go back to block 0; the block loaded ahead is dropped
        settle();
        {
            lock_guard<mutex> lk(m_mutex);
            m_state = ahead::none;
        }
        m_next.clear();
        m_next_error = nullptr;
        m_manifest.reset();
        m_manifest_at  = 0;
        m_block_number = 0;
        if (m_cache)
            m_cache->restart();
        m_block.clear();
        m_at = 0;
    }

    // aeon block_manager::filler (src/block_manager.cpp:61-106); the records of a block are read by a few threads at once
    vector<encoded_record> block_stream::load_block()
    {
        if (m_cache && m_cache->is_complete())
            return m_cache->load_block();
        const auto             range = m_manifest.blocks[m_manifest.block_sequence[m_manifest_at++]];
        vector<encoded_record> block(range.second - range.first);
        parallel_for(block.size(), 16, [&](size_t i) { m_load(m_manifest.records[range.first + i], block[i]); });
        if (m_cache && m_cache->is_ownership())
            m_cache->store_block(block);
        if (++m_block_number == m_manifest.blocks.size())
        {
            // the record stream never ends: back to the start of the data set
            m_block_number = 0;
            m_manifest.reset();
            m_manifest_at = 0;
            if (m_cache)
                m_cache->try_get_access();
        }
        if (m_shuffle)
            std::shuffle(block.begin(), block.end(), m_random);
        return block;
    }

    void block_stream::next_block()
    {
        bool idle;
        {
            lock_guard<mutex> lk(m_mutex);
            idle = m_state == ahead::none;
        }
        if (idle)
            request_block(); // the very first block, or the first after a reset
        settle();
        {
            lock_guard<mutex> lk(m_mutex);
            m_state = ahead::none;
        }
        if (m_next_error)
        {
            exception_ptr e = m_next_error;
            m_next_error    = nullptr;
            rethrow_exception(e);
        }
        m_block = std::move(m_next);
        m_next.clear();
        m_at = 0;
        request_block();
    }

    encoded_record block_stream::next()
    {
        for (int guard = 0; guard < 4 && m_at >= m_block.size(); ++guard)
            next_block();
        if (m_at >= m_block.size())
            throw runtime_error("the record stream is empty");
        return std::move(m_block[m_at++]);
    }
}

aeonb_stream::~aeonb_stream() {}
