// TSV manifest, base64 and cpu-list parsing for the loader shell.
#include <algorithm>
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
                         uint32_t node_count, int batch_size)
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
        if (!root.empty())
            for (auto& rec : list)
                for (size_t i = 0; i < types.size(); i++)
                    if (types[i] == element_t::FILE)
                        rec[i] = path_join(root, rec[i]);
        if (shuffle)
        {
            minstd_rand0 rnd(seed ? seed : random_device{}());
            std::shuffle(list.begin(), list.end(), rnd);
        }
        record_count = list.size();
        if (node_count > 1)
        {
            // interleaved batch-sized slices per node (src/manifest_file.cpp:278-295)
            record_count = list.size() / node_count;
            int batches  = (int)(record_count / batch_size);
            records.resize(record_count);
            for (int i = 0; i < batches * batch_size; i++)
            {
                int batch_num = i / batch_size, in_batch = i % batch_size;
                records[i]    = list[(size_t)batch_num * batch_size * node_count + (size_t)batch_size * node_id + in_batch];
            }
            int tail_count = (int)record_count - batches * batch_size;
            int tail_src   = batches * batch_size * node_count + tail_count * node_id;
            for (int i = 0; i < tail_count; i++)
                records[i + batches * batch_size] = list[i + tail_src];
        }
        else
            records.swap(list);
    }
}
