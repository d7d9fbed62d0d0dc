// aeon_b200.hpp -- aeon's C++ loader API (namespace nervana) as a header-only layer over the C ABI of
// libaeon_b200 (include/aeon_b200.h).  A program written against aeon's `aeon.hpp`
//
//     nervana::loader_factory factory;
//     auto train_set = factory.get_loader(config);          // JSON text, or any JSON object with dump()
//     for (const nervana::fixed_buffer_map& batch : *train_set)
//         const char* first = batch["image"]->get_item(0);
//
// compiles against this header with only the include line changed.  The classes keep the names, members and
// error behaviour (std::invalid_argument / std::runtime_error with aeon's messages) of
//   loader, loader::iterator, loader_factory   aeon src/loader.hpp:112-175, src/loader.cpp:197-268
//   fixed_buffer_map, buffer_fixed_size_elements   aeon src/buffer_batch.hpp:154-283
//   shape_type, output_type                         aeon src/typemap.hpp:55-212
// Differences, all forced by leaving nlohmann::json and OpenCV out of the interface: get_current_config() returns
// the JSON text; get_item_as_mat() does not exist; buffers are views of the loader's batch memory (pinned host
// memory, or device memory when the configuration sets "device_output": true -- data() is then a device pointer),
// valid until the iterator moves on, exactly as in aeon (src/async_manager.hpp:96-107).
#ifndef AEON_B200_HPP
#define AEON_B200_HPP

#include <algorithm>
#include <cstddef>
#include <iterator>
#include <map>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "aeon_b200.h"

namespace nervana
{
    typedef std::vector<size_t> shape_t;

    // aeon src/typemap.hpp:55-112 (numpy / OpenCV type numbers are not carried)
    class output_type
    {
    public:
        output_type() {}
        explicit output_type(const std::string& r)
        {
            static const std::map<std::string, size_t> all = {{"int8_t", 1},  {"uint8_t", 1}, {"int16_t", 2}, {"uint16_t", 2}, {"int32_t", 4},
                                                              {"uint32_t", 4}, {"float", 4},  {"double", 8},  {"char", 1}};
            auto it = all.find(r);
            if (it == all.end())
                throw std::runtime_error("Unable to map output type " + r);
            m_tp_name = r;
            m_size    = it->second;
        }
        bool               valid() const { return m_tp_name.size() > 0; }
        size_t             get_size() const { return m_size; }
        const std::string& get_name() const { return m_tp_name; }
        bool               operator==(const output_type& o) const { return m_size == o.m_size && m_tp_name == o.m_tp_name; }
        bool               operator!=(const output_type& o) const { return !(*this == o); }

        std::string m_tp_name;
        size_t      m_size = 0;
    };

    // aeon src/typemap.hpp:114-212
    class shape_type
    {
    public:
        shape_type() {}
        shape_type(const std::vector<size_t>& shape, const output_type& otype)
            : m_shape{shape}
            , m_otype{otype}
        {
            m_byte_size = m_otype.get_size() * get_element_count();
        }
        size_t get_element_count() const { return std::accumulate(m_shape.begin(), m_shape.end(), (size_t)1, std::multiplies<size_t>()); }
        size_t get_byte_size() const { return m_byte_size; }
        const std::vector<size_t>& get_shape() const { return m_shape; }
        const output_type&         get_otype() const { return m_otype; }
        void set_names(const std::vector<std::string>& names)
        {
            if (m_shape.size() != names.size())
                throw std::runtime_error("naming shape dimensions: number of names does not match number of dimensions");
            m_names = names;
        }
        std::vector<std::string> get_names() const
        {
            if (!m_names.empty())
                return m_names;
            std::vector<std::string> res;
            for (size_t i = 0; i < m_shape.size(); ++i)
                res.push_back(std::to_string(i));
            return res;
        }
        bool operator==(const shape_type& o) const
        {
            return m_byte_size == o.m_byte_size && m_otype == o.m_otype && m_shape == o.m_shape && m_names == o.m_names;
        }
        bool operator!=(const shape_type& o) const { return !(*this == o); }

    private:
        std::vector<size_t>      m_shape;
        output_type              m_otype;
        size_t                   m_byte_size = 0;
        std::vector<std::string> m_names;
    };

    // aeon src/buffer_batch.hpp:154-188: one named output of a batch, `batch_size` items of `stride` bytes.  Here a
    // view: the memory belongs to the loader.
    class buffer_fixed_size_elements
    {
    public:
        buffer_fixed_size_elements() {}
        buffer_fixed_size_elements(const shape_type& shp_tp, size_t batch_size)
            : m_shape_type{shp_tp}
            , m_size{shp_tp.get_byte_size() * batch_size}
            , m_batch_size{batch_size}
            , m_stride{shp_tp.get_byte_size()}
        {
        }
        const char* get_item(size_t index) const
        {
            if (index >= m_batch_size)
                throw std::invalid_argument("buffer_fixed_size: index out-of-range");
            return &m_data[index * m_stride];
        }
        char* get_item(size_t index) { return const_cast<char*>(static_cast<const buffer_fixed_size_elements*>(this)->get_item(index)); }
        char*             data() const { return m_data; }
        size_t            get_item_count() const { return m_stride ? m_size / m_stride : 0; }
        size_t            size() const { return m_size; }
        size_t            get_stride() const { return m_stride; }
        const shape_type& get_shape_type() const { return m_shape_type; }
        void              rebind(void* p) { m_data = static_cast<char*>(p); } // used by the loader when a new batch arrives

    protected:
        char*      m_data = nullptr;
        shape_type m_shape_type;
        size_t     m_size = 0, m_batch_size = 0, m_stride = 0;
    };

    // aeon src/buffer_batch.hpp:190-283
    class fixed_buffer_map
    {
    public:
        fixed_buffer_map() {}
        fixed_buffer_map(const std::vector<std::pair<std::string, shape_type>>& write_sizes, size_t batch_size)
        {
            for (const auto& sz : write_sizes)
            {
                m_names.push_back(sz.first);
                m_data.emplace_back(sz.first, std::unique_ptr<buffer_fixed_size_elements>(new buffer_fixed_size_elements(sz.second, batch_size)));
            }
        }
        const std::vector<std::string>&   get_names() const { return m_names; }
        const buffer_fixed_size_elements* operator[](const std::string& name) const
        {
            for (const auto& v : m_data)
                if (v.first == name)
                    return v.second.get();
            return nullptr;
        }
        buffer_fixed_size_elements* operator[](const std::string& name)
        {
            return const_cast<buffer_fixed_size_elements*>((*static_cast<const fixed_buffer_map*>(this))[name]);
        }
        size_t size() const { return m_data.size(); }

    private:
        fixed_buffer_map(const fixed_buffer_map&) = delete;
        const buffer_fixed_size_elements* operator[](int) const = delete; // map[0] would otherwise pick the string overload
        buffer_fixed_size_elements*       operator[](int)       = delete;

        std::vector<std::string> m_names;
        std::vector<std::pair<std::string, std::unique_ptr<buffer_fixed_size_elements>>> m_data;
    };

    // aeon src/loader.hpp:112-175
    class loader
    {
    public:
        enum class BatchMode
        {
            INFINITE,
            ONCE,
            COUNT
        };

        class iterator : public std::iterator<std::input_iterator_tag, fixed_buffer_map>
        {
        public:
            explicit iterator(loader& ld, bool is_end)
                : m_current_loader(ld)
                , m_is_end{is_end}
            {
            }
            iterator(const iterator& o)
                : m_current_loader{o.m_current_loader}
                , m_is_end{o.m_is_end}
            {
            }
            iterator& operator++()
            {
                m_current_loader.increment_position();
                return *this;
            }
            iterator& operator++(int) { return ++(*this); }
            bool      operator==(const iterator& other) const
            {
                bool res = &m_current_loader == &other.m_current_loader;
                res &= (other.m_is_end && positional_end()) || (m_is_end && other.positional_end());
                return res;
            }
            bool operator!=(const iterator& other) const { return !(*this == other); }
            const fixed_buffer_map& operator*() const
            {
                if (m_current_loader.get_output_buffer())
                    return *m_current_loader.get_output_buffer();
                throw std::runtime_error("empty buffer");
            }
            const size_t& position() const { return m_current_loader.position(); }
            bool          positional_end() const { return !m_is_end && (position() >= (size_t)m_current_loader.batch_count()); }

        private:
            iterator() = delete;
            loader&    m_current_loader;
            const bool m_is_end;
        };

        virtual ~loader() {}
        virtual const std::vector<std::string>& get_buffer_names() const = 0;
        virtual const std::vector<std::pair<std::string, shape_type>>& get_names_and_shapes() const = 0;
        virtual const shape_t& get_shape(const std::string& name) const = 0;
        virtual int            record_count() const = 0;
        virtual int            batch_size() const   = 0;
        virtual int            batch_count() const  = 0;
        virtual iterator       begin()              = 0;
        virtual iterator       end()                = 0;
        virtual iterator&      get_current_iter()   = 0;
        virtual iterator&      get_end_iter()       = 0;
        virtual const fixed_buffer_map* get_output_buffer() const  = 0;
        virtual const size_t&           position()                 = 0;
        virtual void                    reset()                    = 0;
        virtual std::string             get_current_config() const = 0; // JSON text (aeon: nlohmann::json)

    protected:
        friend class iterator;
        virtual void increment_position() = 0;
    };

    // aeon's loader_local (src/loader.hpp:177-240) on the B200 library: manifest, batching, decoding and augmentation
    // run behind aeonb_loader; `device` picks the GPU.
    class loader_local final : public loader
    {
    public:
        explicit loader_local(const std::string& config_json, int device = 0)
            : m_current_iter(*this, false)
            , m_end_iter(*this, true)
        {
            check(aeonb_loader_create(config_json.c_str(), device, &m_handle));
            m_batch_size        = aeonb_loader_batch_size(m_handle);
            m_batch_count_value = aeonb_loader_batch_count(m_handle);
            m_current_config    = aeonb_loader_config(m_handle);
            m_infinite          = m_current_config.find("\"iteration_mode\":\"INFINITE\"") != std::string::npos ||
                         m_current_config.find("\"iteration_mode\": \"INFINITE\"") != std::string::npos;
            static const char* type_names[] = {"uint8_t", "int8_t", "int16_t", "uint16_t", "int32_t", "float", "double"};
            const int          n            = aeonb_loader_output_count(m_handle);
            for (int i = 0; i < n; ++i)
            {
                int64_t dims[8];
                int32_t dtype = 0;
                const int           rank = aeonb_loader_output_shape(m_handle, i, dims, &dtype);
                std::vector<size_t> shape(dims, dims + rank);
                shape_type          st(shape, output_type(type_names[dtype]));
                const std::string   axes = aeonb_loader_axis_names(m_handle, i);
                if (!axes.empty())
                {
                    std::vector<std::string> names;
                    size_t                   at = 0;
                    while (at <= axes.size())
                    {
                        const size_t comma = std::min(axes.find(',', at), axes.size());
                        names.push_back(axes.substr(at, comma - at));
                        at = comma + 1;
                    }
                    if (names.size() == shape.size())
                        st.set_names(names);
                }
                const std::string name = aeonb_loader_output_name(m_handle, i);
                m_names.push_back(name);
                m_names_and_shapes.emplace_back(name, st);
            }
            m_buffers.reset(new fixed_buffer_map(m_names_and_shapes, (size_t)m_batch_size));
            m_pointers.resize(n);
            fetch(); // aeon primes the pipeline in the constructor (src/loader.cpp:179)
        }
        ~loader_local() override { aeonb_loader_destroy(m_handle); }

        const std::vector<std::string>& get_buffer_names() const override { return m_names; }
        const std::vector<std::pair<std::string, shape_type>>& get_names_and_shapes() const override { return m_names_and_shapes; }
        const shape_t& get_shape(const std::string& name) const override
        {
            for (const auto& v : m_names_and_shapes)
                if (v.first == name)
                    return v.second.get_shape();
            throw std::runtime_error("key '" + name + "' not found");
        }
        int      record_count() const override { return aeonb_loader_record_count(m_handle); }
        int      batch_size() const override { return m_batch_size; }
        int      batch_count() const override { return m_batch_count_value; }
        iterator begin() override
        {
            reset();
            return m_current_iter;
        }
        iterator  end() override { return m_end_iter; }
        iterator& get_current_iter() override { return m_current_iter; }
        iterator& get_end_iter() override { return m_end_iter; }
        const fixed_buffer_map* get_output_buffer() const override { return m_output_buffer_ptr; }
        const size_t&           position() override { return m_position; }
        void                    reset() override
        {
            check(aeonb_loader_reset(m_handle));
            fetch();
            m_position = 0;
        }
        std::string get_current_config() const override { return m_current_config; }

    private:
        loader_local() = delete;
        static void check(int status)
        {
            if (status == AEONB_ERR_INVALID)
                throw std::invalid_argument(aeonb_last_error());
            if (status < 0)
                throw std::runtime_error(aeonb_last_error());
        }
        // Takes the next batch from the library and points the buffer views at it.  Past the end of a finite
        // iteration the views keep the last batch (aeon's stream never ends; its position counter ends the loop).
        void fetch()
        {
            const int status = aeonb_loader_next(m_handle, m_pointers.data());
            check(status);
            if (status == AEONB_END)
                return;
            for (size_t i = 0; i < m_names.size(); ++i)
                (*m_buffers)[m_names[i]]->rebind(m_pointers[i]);
            m_output_buffer_ptr = m_buffers.get();
        }
        void increment_position() override
        {
            fetch();
            m_position++;
            if (m_infinite && m_position == (size_t)m_batch_count_value) // wrap around if this is an infinite iterator
                m_position = 0;
        }

        aeonb_loader* m_handle = nullptr;
        iterator      m_current_iter;
        iterator      m_end_iter;
        int           m_batch_size = 0, m_batch_count_value = 0;
        bool          m_infinite = false;
        size_t        m_position{0};
        std::vector<std::string>                        m_names;
        std::vector<std::pair<std::string, shape_type>> m_names_and_shapes;
        std::unique_ptr<fixed_buffer_map>               m_buffers;
        std::vector<void*>                              m_pointers;
        fixed_buffer_map*                               m_output_buffer_ptr{nullptr};
        std::string                                     m_current_config;
    };

    // aeon src/loader.hpp:171-175
    class loader_factory
    {
    public:
        std::unique_ptr<loader> get_loader(const std::string& config) { return std::unique_ptr<loader>(new loader_local(config)); }
        std::unique_ptr<loader> get_loader(const char* config) { return get_loader(std::string(config)); }
        // any JSON object with a dump() member (nlohmann::json, as aeon's callers hold)
        template <typename Json>
        auto get_loader(const Json& config) -> decltype(config.dump(), std::unique_ptr<loader>())
        {
            return get_loader(std::string(config.dump()));
        }
    };
}

#endif // AEON_B200_HPP
