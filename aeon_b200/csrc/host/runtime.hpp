// Small host runtime pieces shared by the provider and the loader: a worker pool with
// dynamic index hand-out (aeon's thread_pool, src/thread_pool.hpp:82-175), and grow-only
// pinned / device buffers.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <exception>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "../context.hpp"

namespace aeonb
{
    class worker_pool
    {
    public:
        explicit worker_pool(int threads);
        ~worker_pool();
        int size() const { return (int)m_threads.size(); }
        // Starts fn(i) for i in [0,count) on the workers (indices handed out in increasing order) and
        // returns at once; wait() blocks until all are done and rethrows the first exception.
        // `light` wakes only the first k_light threads: a few hundred small copies finish sooner on three threads than on
        // a whole pool whose wake-up competes with the calling thread for the cores.
        static int light_threads(); // AEONB_LIGHT_THREADS or 3
        const int k_light = light_threads();
        void start(int count, std::function<void(int)> fn, bool light = false);
        void wait();
        // The calling thread takes part in the job started last: runs fn(i) for indices it draws from the same counter until
        // none is left.  Returns how many it ran.  (The workers' wake-up takes tens of microseconds; the caller is already awake.)
        int help();
        void run(int count, std::function<void(int)> fn)
        {
            start(count, std::move(fn));
            wait();
        }

    private:
        void loop(int index);
        std::vector<std::thread>  m_threads;
        std::mutex                m_mutex;
        std::condition_variable   m_wake, m_wake_rest, m_done; // the first k_light threads wait on m_wake, the others on m_wake_rest
        std::function<void(int)>  m_fn;
        std::atomic<int>          m_next{0};
        int                       m_count   = 0;
        int                       m_active  = 0;
        int                       m_tickets = 0; // threads still to join the current job
        uint64_t                  m_epoch   = 0;
        bool                      m_stop    = false;
        std::exception_ptr        m_error;
    };

    // aeon's default worker count: hardware threads minus min(2, hw/8) (src/util.cpp:360-370).
    int default_worker_count();

    struct pinned_buffer
    {
        void*  p   = nullptr;
        size_t cap = 0;
        void   reserve(size_t bytes)
        {
            if (bytes <= cap)
                return;
            release();
            bytes += bytes / 4; // head room: batch sizes wander with the drawn crop boxes, and growing stalls the pipeline
            AEONB_CUDA(cudaMallocHost(&p, bytes));
            cap = bytes;
        }
        void release()
        {
            if (p)
                cudaFreeHost(p);
            p   = nullptr;
            cap = 0;
        }
        ~pinned_buffer() { release(); }
    };

    struct device_buffer
    {
        void*  p   = nullptr;
        size_t cap = 0;
        // Growing frees the old allocation: the caller makes sure no kernel still uses it.
        void reserve(size_t bytes)
        {
            if (bytes <= cap)
                return;
            release();
            bytes += bytes / 4; // head room, as above (cudaFree waits for the whole device)
            AEONB_CUDA(cudaMalloc(&p, bytes));
            cap = bytes;
        }
        void release()
        {
            if (p)
                cudaFree(p);
            p   = nullptr;
            cap = 0;
        }
        ~device_buffer() { release(); }
    };

    inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}
