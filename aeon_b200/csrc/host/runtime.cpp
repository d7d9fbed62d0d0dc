#include "runtime.hpp"

#include <algorithm>

namespace aeonb
{
    int default_worker_count()
    {
        const int hw = std::max(1u, std::thread::hardware_concurrency());
        return std::max(1, hw - std::min(2, hw / 8));
    }

    worker_pool::worker_pool(int threads)
    {
        threads = std::max(1, threads);
        for (int i = 0; i < threads; ++i)
            m_threads.emplace_back([this] { loop(); });
    }

    worker_pool::~worker_pool()
    {
        {
            std::lock_guard<std::mutex> lk(m_mutex);
            m_stop = true;
        }
        m_wake.notify_all();
        for (auto& t : m_threads)
            t.join();
    }

    void worker_pool::start(int count, std::function<void(int)> fn)
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        m_fn     = std::move(fn);
        m_count  = count;
        m_next   = 0;
        m_active = (int)m_threads.size();
        m_error  = nullptr;
        ++m_epoch;
        m_wake.notify_all();
    }

    void worker_pool::wait()
    {
        std::unique_lock<std::mutex> lk(m_mutex);
        m_done.wait(lk, [this] { return m_active == 0; });
        if (m_error)
        {
            auto e  = m_error;
            m_error = nullptr;
            std::rethrow_exception(e);
        }
    }

    void worker_pool::loop()
    {
        uint64_t seen = 0;
        for (;;)
        {
            {
                std::unique_lock<std::mutex> lk(m_mutex);
                m_wake.wait(lk, [&] { return m_stop || m_epoch != seen; });
                if (m_stop)
                    return;
                seen = m_epoch;
            }
            for (;;)
            {
                const int i = m_next.fetch_add(1);
                if (i >= m_count)
                    break;
                try
                {
                    m_fn(i);
                }
                catch (...)
                {
                    std::lock_guard<std::mutex> lk(m_mutex);
                    if (!m_error)
                        m_error = std::current_exception(); // the first failure wins, as in aeon's pool
                }
            }
            {
                std::lock_guard<std::mutex> lk(m_mutex);
                if (--m_active == 0)
                    m_done.notify_all();
            }
        }
    }
}
