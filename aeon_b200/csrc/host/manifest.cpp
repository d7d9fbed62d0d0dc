// TSV manifest, base64 and cpu-list parsing for the loader shell.
#include <algorithm>
#include <array>
#include <cmath>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "loader.hpp"

using namespace std;

namespace aeonb
{
    namespace
    {
        vector<string> split(const string& s, char delim)
        {
            vector<string> out;
            size_t         start = 0;
            for (;;)
            {
                size_t pos = s.find(delim, start);
                if (pos == string::npos)
                {
                    out.push_back(s.substr(start));
                    return out;
                }
                out.push_back(s.substr(start, pos - start));
                start = pos + 1;
            }
        }

        string path_join(const string& a, const string& b)
        {
            if (a.empty() || (!b.empty() && b[0] == '/'))
                return b;
            return a.back() == '/' ? a + b : a + "/" + b;
        }
    }

    vector<char> base64_decode(const string& in)
    {
        auto value = [](unsigned char c) -> int {
            if (c >= 'A' && c <= 'Z')
                return c - 'A';
            if (c >= 'a' && c <= 'z')
                return c - 'a' + 26;
            if (c >= '0' && c <= '9')
                return c - '0' + 52;
            if (c == '+')
                return 62;
            if (c == '/')
                return 63;
            return -1;
        };
        vector<char> out;
        unsigned     acc = 0;
        int          bits = 0;
        for (unsigned char c : in)
        {
            if (c == '=')
                break;
            int v = value(c);
            if (v < 0)
                continue;
            acc = (acc << 6) | (unsigned)v;
            bits += 6;
            if (bits >= 8)
            {
                bits -= 8;
                out.push_back((char)((acc >> bits) & 0xFF));
            }
        }
        return out;
    }

    vector<int> parse_cpu_list(const string& s)
    {
        vector<int> cpus;
        if (s.empty())
            return cpus;
        for (const string& part : split(s, ','))
        {
            if (part.empty())
                continue;
            size_t dash = part.find('-');
            if (dash == string::npos)
                cpus.push_back(stoi(part));
            else
                for (int i = stoi(part.substr(0, dash)); i <= stoi(part.substr(dash + 1)); ++i)
                    cpus.push_back(i);
        }
        sort(cpus.begin(), cpus.end());
        cpus.erase(unique(cpus.begin(), cpus.end()), cpus.end());
        return cpus;
    }

    void manifest::parse(istream& in, const string& root, float subset_fraction, bool shuffle, uint32_t seed, uint32_t node_id,
                         uint32_t node_count, int batch_size, int block_size)
    {
        string line;
        size_t line_number = 0;
        vector<vector<string>> list;
        while (getline(in, line))
        {
            if (!line.empty() && line.back() == '\r')
                line.pop_back();
            if (line.empty())
            {
            }
            else if (line[0] == '@')
            {
                if (!types.empty())
                    throw invalid_argument("metadata must be defined before any data"); // element types come first
                for (const string& t : split(line.substr(1), '\t'))
                {
                    if (t == "FILE")
                        types.push_back(element_t::FILE);
                    else if (t == "BINARY")
                        types.push_back(element_t::BINARY);
                    else if (t == "STRING")
                        types.push_back(element_t::STRING);
                    else if (t == "ASCII_INT")
                        types.push_back(element_t::ASCII_INT);
                    else if (t == "ASCII_FLOAT")
                        types.push_back(element_t::ASCII_FLOAT);
                    else
                    {
                        ostringstream ss;
                        ss << "invalid metadata type '" << t << "' at line " << line_number;
                        throw invalid_argument(ss.str());
                    }
                }
            }
            else if (line[0] == '#')
            {
            }
            else
            {
                vector<string> fields = split(line, '\t');
                if (types.empty())
                    throw invalid_argument("metadata must be defined before any data");
                if (fields.size() != types.size())
                {
                    ostringstream ss;
                    ss << "at line: " << line_number << ", manifest file has a line with differing number of elements ("
                       << fields.size() << ") vs (" << types.size() << "): ";
                    for (const string& f : fields)
                        ss << f << " ";
                    throw runtime_error(ss.str());
                }
                list.push_back(fields);
            }
            line_number++;
        }
        if (!(subset_fraction > 0.0 && subset_fraction <= 1.0))
            throw runtime_error("subset_fraction must be >= 0 and <= 1");
        if (subset_fraction < 1.0)
        {
            // aeon src/manifest_file.cpp:332-356: fixed-seed Bernoulli thinning with an exact target count
            bernoulli_distribution dist(subset_fraction);
            default_random_engine  gen(0);
            vector<vector<string>> tmp;
            tmp.swap(list);
            size_t needed = (size_t)(tmp.size() * subset_fraction);
            for (size_t i = 0; i < tmp.size() && needed; i++)
            {
                size_t remainder = tmp.size() - i;
                if (needed == remainder || dist(gen))
                {
                    list.push_back(tmp[i]);
                    needed--;
                }
            }
        }
        // cache identity: CRC32C over every field as written in the manifest, before the root is joined on
        // (src/manifest_file.cpp:208-219)
        {
            uint32_t c = 0xFFFFFFFFu;
            for (const auto& rec : list)
                for (const string& f : rec)
                    c = crc32c_update(c, f.data(), f.size());
            crc = ~c;
        }
        if (!root.empty())
            for (auto& rec : list)
                for (size_t i = 0; i < types.size(); i++)
                    if (types[i] == element_t::FILE)
                        rec[i] = path_join(root, rec[i]);
        m_all.swap(list);
        m_random.seed(seed ? seed : random_device{}());
        m_shuffle    = shuffle;
        m_node_id    = node_id;
        m_node_count = node_count;
        m_batch_size = batch_size;
        m_block_size = block_size;
        generate();
    }

    // Which records of the full list one node of a multi-node run reads (src/manifest_file.cpp:278-295): the list is
    // cut into rounds of node_count batches, node g takes batch g of every round; what is left after the last whole
    // round of this node's share is divided into node_count equal runs, node g taking run g.
    vector<size_t> node_record_indices(size_t total, uint32_t node_id, uint32_t node_count, int batch_size)
    {
        vector<size_t> out;
        if (node_count <= 1)
        {
            out.resize(total);
            for (size_t i = 0; i < total; ++i)
                out[i] = i;
            return out;
        }
        const size_t share  = total / node_count;        // records of this node
        const size_t rounds = share / (size_t)batch_size; // whole batches of this node
        out.reserve(share);
        for (size_t round = 0; round < rounds; ++round)
        {
            const size_t first = (round * node_count + node_id) * (size_t)batch_size;
            for (size_t k = 0; k < (size_t)batch_size; ++k)
                out.push_back(first + k);
        }
        const size_t run   = share - rounds * (size_t)batch_size;
        const size_t first = rounds * node_count * (size_t)batch_size + run * node_id;
        for (size_t k = 0; k < run; ++k)
            out.push_back(first + k);
        return out;
    }

    // aeon generate_block_list (src/block.cpp:23-44): about block_size records per block, all blocks but the last equal
    vector<pair<size_t, size_t>> block_ranges(size_t record_count, size_t block_size)
    {
        size_t count = (size_t)std::round((float)record_count / (float)block_size);
        count        = std::max<size_t>(count, 1);
        const size_t size = (size_t)std::ceil((float)record_count / (float)count);
        vector<pair<size_t, size_t>> out;
        for (size_t b = 0; b < count; ++b)
        {
            const size_t lo = size * b;
            if (lo + size > record_count)
            {
                out.emplace_back(lo, record_count);
                break;
            }
            out.emplace_back(lo, lo + size);
        }
        return out;
    }

    // aeon manifest_file::generate_blocks (src/manifest_file.cpp:270-318)
    void manifest::generate()
    {
        if (m_shuffle)
            std::shuffle(m_all.begin(), m_all.end(), m_random);
        const vector<size_t> mine = node_record_indices(m_all.size(), m_node_id, m_node_count, m_batch_size);
        records.clear();
        records.reserve(mine.size());
        for (size_t i : mine)
            records.push_back(m_all[i]);
        record_count = records.size();
        blocks       = block_ranges(record_count, (size_t)m_block_size);
        block_sequence.resize(blocks.size());
        for (size_t i = 0; i < blocks.size(); ++i)
            block_sequence[i] = i;
    }

    // aeon manifest_file::reset (src/manifest_file.cpp:320-329): with shuffle_manifest a new block order, and for a
    // multi-node run a new shuffle of the whole list
    void manifest::reset()
    {
        if (m_shuffle)
        {
            std::shuffle(block_sequence.begin(), block_sequence.end(), m_random);
            if (m_node_count > 1)
                generate();
        }
    }

    uint32_t crc32c_update(uint32_t crc, const void* data, size_t size)
    {
        static const auto table = [] {
            std::array<uint32_t, 256> t{};
            for (uint32_t i = 0; i < 256; ++i)
            {
                uint32_t c = i;
                for (int k = 0; k < 8; ++k)
                    c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1; // Castagnoli polynomial, reflected
                t[i] = c;
            }
            return t;
        }();
        const unsigned char* p = static_cast<const unsigned char*>(data);
        for (size_t i = 0; i < size; ++i)
            crc = table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
        return crc;
    }
}
