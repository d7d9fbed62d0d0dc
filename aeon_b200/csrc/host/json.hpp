// Minimal JSON document model, parser and writer for the aeon dataloader configuration.
//
// aeon configures every stage from one JSON object (loader keys, "etl" array,
// "augmentation" array).  This is a small self-contained implementation so the
// library has no third-party dependency; only the JSON subset a config needs is
// supported (objects, arrays, strings with the standard escapes, numbers, booleans, null).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace aeonb
{
    class json
    {
    public:
        enum class kind
        {
            null,
            boolean,
            integer,
            real,
            string,
            array,
            object
        };
        using array_t  = std::vector<json>;
        using object_t = std::vector<std::pair<std::string, json>>; // keeps insertion order

        json() = default;
        json(std::nullptr_t) {}
        json(bool v) : m_kind(kind::boolean), m_int(v) {}
        json(int v) : m_kind(kind::integer), m_int(v) {}
        json(int64_t v) : m_kind(kind::integer), m_int(v) {}
        json(uint64_t v) : m_kind(kind::integer), m_int(static_cast<int64_t>(v)) {}
        json(double v) : m_kind(kind::real), m_real(v) {}
        json(const char* v) : m_kind(kind::string), m_str(v) {}
        json(std::string v) : m_kind(kind::string), m_str(std::move(v)) {}
        static json make_array() { json j; j.m_kind = kind::array; return j; }
        static json make_object() { json j; j.m_kind = kind::object; return j; }

        static json parse(const std::string& text);
        std::string dump() const;

        kind type() const { return m_kind; }
        bool is_null() const { return m_kind == kind::null; }
        bool is_object() const { return m_kind == kind::object; }
        bool is_array() const { return m_kind == kind::array; }
        bool is_string() const { return m_kind == kind::string; }
        bool is_number() const { return m_kind == kind::integer || m_kind == kind::real; }
        bool is_boolean() const { return m_kind == kind::boolean; }

        // Object access.  find() returns nullptr when the key is absent.
        const json* find(const std::string& key) const;
        json*       find(const std::string& key);
        bool        contains(const std::string& key) const { return find(key) != nullptr; }
        json&       operator[](const std::string& key); // inserts null when absent
        void        erase(const std::string& key);
        const object_t& items() const { expect(kind::object, "object"); return m_obj; }

        // Array access.
        const array_t& elements() const { expect(kind::array, "array"); return m_arr; }
        array_t&       elements() { expect(kind::array, "array"); return m_arr; }
        void           push_back(json v) { expect(kind::array, "array"); m_arr.push_back(std::move(v)); }
        size_t         size() const { return m_kind == kind::array ? m_arr.size() : m_kind == kind::object ? m_obj.size() : 0; }

        // Scalar conversion with the narrowing rules a config reader needs.
        bool        as_bool() const;
        int64_t     as_int() const;
        double      as_double() const;
        const std::string& as_string() const { expect(kind::string, "string"); return m_str; }

    private:
        void expect(kind k, const char* what) const
        {
            if (m_kind != k)
                throw std::invalid_argument(std::string("json value is not a ") + what);
        }
        kind        m_kind = kind::null;
        int64_t     m_int  = 0;
        double      m_real = 0;
        std::string m_str;
        array_t     m_arr;
        object_t    m_obj;
        friend class json_reader;
    };
}
