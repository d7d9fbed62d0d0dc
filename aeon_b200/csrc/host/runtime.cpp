#include <cstdlib>
#include "runtime.hpp"

#include <algorithm>
#include <atomic>

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
            m_threads.emplace_back([this, i] { loop(i); });
    }

    worker_pool::~worker_pool()
    {
        {
            std::lock_guard<std::mutex> lk(m_mutex);
            m_stop = true;
        }
        m_wake.notify_all();
        m_wake_rest.notify_all();
        for (auto& t : m_threads)
            t.join();
    }

    int worker_pool::light_threads()
    {
        static const int value = [] {
            const char* e = std::getenv("AEONB_LIGHT_THREADS");
            const int   v = e ? std::atoi(e) : 3;
            return v < 1 ? 1 : v > 64 ? 64 : v;
        }();
        return value;
    }

    void worker_pool::start(int count, std::function<void(int)> fn, bool light)
    {
        const int all = (int)m_threads.size();
        const int k   = light ? std::min(k_light, all) : all;
        {
            std::lock_guard<std::mutex> lk(m_mutex);
            m_fn      = std::move(fn);
            m_count   = count;
            m_next    = 0;
            m_active  = k;
            m_tickets = k;
            m_error   = nullptr;
            ++m_epoch;
        }
        // Exactly k threads take a ticket and work.  Every thread of the first group is woken, so k tickets are always
        // taken; a thread of the other group that is still on its way back to its wait may take one instead, and the
        // thread that then finds none sleeps on.
        m_wake.notify_all();
        if (!light)
            m_wake_rest.notify_all();
    }

    int worker_pool::help()
    {
        int ran = 0;
        for (;;)
        {
            const int i = m_next.fetch_add(1);
            if (i >= m_count)
                return ran;
            try
            {
                m_fn(i);
            }
            catch (...)
            {
                std::lock_guard<std::mutex> lk(m_mutex);
                if (!m_error)
                    m_error = std::current_exception();
            }
            ++ran;
        }
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

    void worker_pool::loop(int index)
    {
        uint64_t                 seen = 0;
        std::condition_variable& wake = index < k_light ? m_wake : m_wake_rest;
        for (;;)
        {
            {
                std::unique_lock<std::mutex> lk(m_mutex);
                wake.wait(lk, [&] { return m_stop || m_epoch != seen; });
                if (m_stop)
                    return;
                seen = m_epoch;
                if (m_tickets == 0)
                    continue;
                --m_tickets;
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

// Self-test hook of the pool (host only): `rounds` dispatches of 1..300 jobs, every seventh on the whole pool and the rest
// on the light group; returns the sum of all job indices run, which the caller can predict.
extern "C" int64_t aeonb_selftest_worker_pool(int threads, int rounds)
{
    try
    {
        aeonb::worker_pool  pool(threads);
        std::atomic<int64_t> sum{0};
        for (int it = 0; it < rounds; ++it)
        {
            const int n = 1 + it % 300;
            pool.start(n, [&](int i) { sum += i; }, it % 7 != 0);
            pool.wait();
        }
        return sum.load();
    }
    catch (...)
    {
        return -1;
    }
}
