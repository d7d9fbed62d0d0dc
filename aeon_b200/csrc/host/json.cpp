#include "json.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <sstream>

namespace aeonb
{
    const json* json::find(const std::string& key) const
    {
        if (m_kind != kind::object)
            return nullptr;
        for (const auto& kv : m_obj)
            if (kv.first == key)
                return &kv.second;
        return nullptr;
    }

    json* json::find(const std::string& key)
    {
        return const_cast<json*>(static_cast<const json*>(this)->find(key));
    }

    json& json::operator[](const std::string& key)
    {
        if (m_kind == kind::null)
            m_kind = kind::object;
        expect(kind::object, "object");
        if (json* p = find(key))
            return *p;
        m_obj.emplace_back(key, json());
        return m_obj.back().second;
    }

    void json::erase(const std::string& key)
    {
        if (m_kind != kind::object)
            return;
        for (auto it = m_obj.begin(); it != m_obj.end(); ++it)
            if (it->first == key)
            {
                m_obj.erase(it);
                return;
            }
    }

    bool json::as_bool() const
    {
        if (m_kind == kind::boolean || m_kind == kind::integer)
            return m_int != 0;
        throw std::invalid_argument("json value is not a boolean");
    }

    int64_t json::as_int() const
    {
        if (m_kind == kind::integer || m_kind == kind::boolean)
            return m_int;
        if (m_kind == kind::real)
            return static_cast<int64_t>(m_real);
        throw std::invalid_argument("json value is not a number");
    }

    double json::as_double() const
    {
        if (m_kind == kind::real)
            return m_real;
        if (m_kind == kind::integer || m_kind == kind::boolean)
            return static_cast<double>(m_int);
        throw std::invalid_argument("json value is not a number");
    }

    class json_reader
    {
    public:
        explicit json_reader(const std::string& s) : m_s(s) {}
        json run()
        {
            json v = value();
            skip();
            if (m_p != m_s.size())
                fail("trailing characters");
            return v;
        }

    private:
        [[noreturn]] void fail(const char* why) const
        {
            std::ostringstream ss;
            ss << "json parse error at offset " << m_p << ": " << why;
            throw std::invalid_argument(ss.str());
        }
        void skip()
        {
            while (m_p < m_s.size() && (m_s[m_p] == ' ' || m_s[m_p] == '\t' || m_s[m_p] == '\n' || m_s[m_p] == '\r'))
                ++m_p;
        }
        bool eat(const char* word)
        {
            size_t n = 0;
            while (word[n])
                ++n;
            if (m_s.compare(m_p, n, word) == 0)
            {
                m_p += n;
                return true;
            }
            return false;
        }
        json value()
        {
            skip();
            if (m_p >= m_s.size())
                fail("unexpected end");
            char c = m_s[m_p];
            if (c == '{')
                return object();
            if (c == '[')
                return array();
            if (c == '"')
                return json(string());
            if (eat("true"))
                return json(true);
            if (eat("false"))
                return json(false);
            if (eat("null"))
                return json();
            if (eat("NaN"))
                return json(std::nan(""));
            return number();
        }
        json object()
        {
            json o = json::make_object();
            ++m_p;
            skip();
            if (m_p < m_s.size() && m_s[m_p] == '}')
            {
                ++m_p;
                return o;
            }
            for (;;)
            {
                skip();
                if (m_p >= m_s.size() || m_s[m_p] != '"')
                    fail("expected a key");
                std::string k = string();
                skip();
                if (m_p >= m_s.size() || m_s[m_p] != ':')
                    fail("expected ':'");
                ++m_p;
                o[k] = value();
                skip();
                if (m_p < m_s.size() && m_s[m_p] == ',')
                {
                    ++m_p;
                    continue;
                }
                if (m_p < m_s.size() && m_s[m_p] == '}')
                {
                    ++m_p;
                    return o;
                }
                fail("expected ',' or '}'");
            }
        }
        json array()
        {
            json a = json::make_array();
            ++m_p;
            skip();
            if (m_p < m_s.size() && m_s[m_p] == ']')
            {
                ++m_p;
                return a;
            }
            for (;;)
            {
                a.push_back(value());
                skip();
                if (m_p < m_s.size() && m_s[m_p] == ',')
                {
                    ++m_p;
                    continue;
                }
                if (m_p < m_s.size() && m_s[m_p] == ']')
                {
                    ++m_p;
                    return a;
                }
                fail("expected ',' or ']'");
            }
        }
        static void utf8(std::string& out, unsigned cp)
        {
            if (cp < 0x80)
                out += static_cast<char>(cp);
            else if (cp < 0x800)
            {
                out += static_cast<char>(0xC0 | (cp >> 6));
                out += static_cast<char>(0x80 | (cp & 0x3F));
            }
            else
            {
                out += static_cast<char>(0xE0 | (cp >> 12));
                out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
                out += static_cast<char>(0x80 | (cp & 0x3F));
            }
        }
        std::string string()
        {
            std::string out;
            ++m_p;
            while (m_p < m_s.size())
            {
                char c = m_s[m_p++];
                if (c == '"')
                    return out;
                if (c != '\\')
                {
                    out += c;
                    continue;
                }
                if (m_p >= m_s.size())
                    break;
                char e = m_s[m_p++];
                switch (e)
                {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u':
                {
                    if (m_p + 4 > m_s.size())
                        fail("bad \\u escape");
                    unsigned cp = static_cast<unsigned>(std::strtoul(m_s.substr(m_p, 4).c_str(), nullptr, 16));
                    m_p += 4;
                    utf8(out, cp);
                    break;
                }
                default: out += e;
                }
            }
            fail("unterminated string");
        }
        json number()
        {
            size_t start = m_p;
            bool   real  = false;
            if (m_p < m_s.size() && (m_s[m_p] == '-' || m_s[m_p] == '+'))
                ++m_p;
            while (m_p < m_s.size())
            {
                char c = m_s[m_p];
                if (c >= '0' && c <= '9')
                    ++m_p;
                else if (c == '.' || c == 'e' || c == 'E' || c == '-' || c == '+')
                {
                    real = true;
                    ++m_p;
                }
                else
                    break;
            }
            if (m_p == start)
                fail("unexpected character");
            std::string tok = m_s.substr(start, m_p - start);
            if (real)
                return json(std::strtod(tok.c_str(), nullptr));
            return json(static_cast<int64_t>(std::strtoll(tok.c_str(), nullptr, 10)));
        }
        const std::string& m_s;
        size_t             m_p = 0;
    };

    json json::parse(const std::string& text) { return json_reader(text).run(); }

    static void dump_string(std::string& out, const std::string& s)
    {
        out += '"';
        for (unsigned char c : s)
        {
            switch (c)
            {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\t': out += "\\t"; break;
            case '\r': out += "\\r"; break;
            default:
                if (c < 0x20)
                {
                    char buf[8];
                    std::snprintf(buf, sizeof buf, "\\u%04x", c);
                    out += buf;
                }
                else
                    out += static_cast<char>(c);
            }
        }
        out += '"';
    }

    static void dump_value(std::string& out, const json& j)
    {
        switch (j.type())
        {
        case json::kind::null: out += "null"; break;
        case json::kind::boolean: out += j.as_bool() ? "true" : "false"; break;
        case json::kind::integer: out += std::to_string(j.as_int()); break;
        case json::kind::real:
        {
            char buf[40];
            std::snprintf(buf, sizeof buf, "%.17g", j.as_double());
            out += buf;
            break;
        }
        case json::kind::string: dump_string(out, j.as_string()); break;
        case json::kind::array:
        {
            out += '[';
            bool first = true;
            for (const json& e : j.elements())
            {
                if (!first)
                    out += ',';
                first = false;
                dump_value(out, e);
            }
            out += ']';
            break;
        }
        case json::kind::object:
        {
            out += '{';
            bool first = true;
            for (const auto& kv : j.items())
            {
                if (!first)
                    out += ',';
                first = false;
                dump_string(out, kv.first);
                out += ':';
                dump_value(out, kv.second);
            }
            out += '}';
            break;
        }
        }
    }

    std::string json::dump() const
    {
        std::string out;
        dump_value(out, *this);
        return out;
    }
}
