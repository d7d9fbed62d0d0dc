#include "block_stream.hpp"

#include <fcntl.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <fstream>
#include <sstream>
#include <stdexcept>

using namespace std;

namespace aeonb
{
    namespace
    {
        // ---- old binary cpio member header: thirteen 16-bit fields, name (with its NUL) and data each padded to even length
        void put16(ostream& o, uint16_t v) { o.write(reinterpret_cast<const char*>(&v), 2); }
        uint16_t get16(istream& i)
        {
            uint16_t v = 0;
            i.read(reinterpret_cast<char*>(&v), 2);
            return v;
        }

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

        uint32_t read_member_header(istream& i, string& name)
        {
            if (get16(i) != 070707 || !i)
                throw runtime_error("CPIO header magic incorrect");
            for (int k = 0; k < 9; ++k) // dev, ino, mode, uid, gid, nlink, rdev, mtime
                get16(i);
            const uint16_t namesize = get16(i);
            const uint32_t hi = get16(i), lo = get16(i);
            name.assign(namesize, '\0');
            i.read(&name[0], namesize);
            if (!name.empty())
                name.pop_back();
            if (namesize % 2)
                i.get();
            if (!i)
                throw runtime_error("cache system: cache file corrupted");
            return hi << 16 | lo;
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
        ifstream i(path, ios::binary);
        if (!i)
            throw runtime_error("cache system: cache file missed");
        string name;
        const uint32_t header_size = read_member_header(i, name);
        if (header_size != 64)
            throw runtime_error("unexpected header size.  expected 64 found " + to_string(header_size));
        char     magic[4];
        uint32_t versions[2], record_count = 0, elements_field = 0;
        char     skip[36];
        i.read(magic, 4);
        if (strncmp(magic, "MACR", 4) != 0)
            throw runtime_error("Unrecognized format\n");
        i.read(reinterpret_cast<char*>(versions), 8);
        i.read(skip, 8);
        i.read(reinterpret_cast<char*>(&record_count), 4);
        i.read(reinterpret_cast<char*>(&elements_field), 4);
        i.read(skip, 36);
        if (!i || record_count == 0)
            throw runtime_error("cache system: cache file corrupted");
        vector<encoded_record> out(record_count);
        for (encoded_record& rec : out)
        {
            rec.resize(elements_per_record);
            for (vector<char>& e : rec)
            {
                const uint32_t size = read_member_header(i, name);
                e.resize(size);
                i.read(e.data(), size);
                if (size % 2)
                    i.get();
                if (!i)
                    throw runtime_error("cache system: cache file corrupted");
            }
        }
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

    void block_stream::reset()
    {
        // every stage of aeon's chain starts over (src/async_manager.hpp:119-131): the manifest deals a new block order
        // when it shuffles, the block manager and the cache go back to block 0
        m_manifest.reset();
        m_manifest_at  = 0;
        m_block_number = 0;
        if (m_cache)
            m_cache->restart();
        m_block.clear();
        m_at = 0;
    }

    // aeon block_manager::filler (src/block_manager.cpp:61-106)
    void block_stream::next_block()
    {
        m_block.clear();
        m_at = 0;
        if (m_cache && m_cache->is_complete())
        {
            m_block = m_cache->load_block();
            return;
        }
        const auto range = m_manifest.blocks[m_manifest.block_sequence[m_manifest_at++]];
        m_block.resize(range.second - range.first);
        for (size_t i = range.first; i < range.second; ++i)
            m_load(m_manifest.records[i], m_block[i - range.first]);
        if (m_cache && m_cache->is_ownership())
            m_cache->store_block(m_block);
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
            std::shuffle(m_block.begin(), m_block.end(), m_random);
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
