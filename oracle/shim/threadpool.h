// threadpool.h - portable stand-in for the reference's Apple-only thread pool,
// used ONLY to compile the reference's own matmul sources on a Linux host for
// the oracle / CPU baseline (the real header needs IOKit and Apple futexes).
//
// It keeps the one property of the original that affects results and timing
// of the matmul path: parallel_for(n, body) splits [0, n) into contiguous
// chunks of ceil(n / T) items, thread t takes chunk t, and the caller is
// thread 0 (reference: src/threadpool.h:228-258, 310-320). The power/QoS
// policy of the original is not modelled. T comes from LAPLACE_THREADS
// (as in the original, src/threadpool.h:118) or the hardware concurrency,
// and can be changed between calls with set_threads().
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <mutex>
#include <thread>
#include <type_traits>
#include <vector>

namespace Laplace {

class ThreadPool {
public:
    static ThreadPool& get() {
        static ThreadPool pool;
        return pool;
    }

    int threads() const { return active_; }

    void set_threads(int t) {
        if (t < 1) t = 1;
        if (t > max_) t = max_;
        active_ = t;
    }

    template <typename F>
    void parallel_for(int n, F&& body) {
        if (n <= 0) return;
        const int T = active_;
        if (T <= 1) {
            for (int i = 0; i < n; i++) body(i);
            return;
        }
        using Fd = std::decay_t<F>;
        call_ = [](void* c, int i) { (*static_cast<Fd*>(c))(i); };
        ctx_ = &body;
        n_ = n;
        team_ = T;
        pending_.store(T - 1, std::memory_order_relaxed);
        {
            std::lock_guard<std::mutex> lk(mu_);
            epoch_.fetch_add(1, std::memory_order_release);
        }
        cv_.notify_all();
        run_chunk(0);
        while (pending_.load(std::memory_order_acquire) != 0) std::this_thread::yield();
    }

    ~ThreadPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
            epoch_.fetch_add(1, std::memory_order_release);
        }
        cv_.notify_all();
        for (auto& w : workers_) w.join();
    }

private:
    ThreadPool() {
        int hw = static_cast<int>(std::thread::hardware_concurrency());
        if (hw < 1) hw = 1;
        max_ = hw;
        active_ = hw;
        if (const char* e = std::getenv("LAPLACE_THREADS")) {
            int v = std::atoi(e);
            if (v >= 1) active_ = v < hw ? v : hw;
        }
        for (int t = 1; t < max_; t++) workers_.emplace_back([this, t] { worker(t); });
    }

    void run_chunk(int t) {
        const int chunk = (n_ + team_ - 1) / team_;
        int b = t * chunk, e = b + chunk;
        if (e > n_) e = n_;
        for (int i = b; i < e; i++) call_(ctx_, i);
    }

    void worker(int t) {
        unsigned seen = 0;
        for (;;) {
            // brief spin for back-to-back matmuls, then sleep
            unsigned now = seen;
            for (int spin = 0; spin < 20000; spin++) {
                now = epoch_.load(std::memory_order_acquire);
                if (now != seen) break;
            }
            if (now == seen) {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return epoch_.load(std::memory_order_acquire) != seen; });
                now = epoch_.load(std::memory_order_acquire);
            }
            seen = now;
            if (stop_) return;
            if (t < team_) {
                run_chunk(t);
                pending_.fetch_sub(1, std::memory_order_release);
            }
        }
    }

    using call_t = void (*)(void*, int);
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::atomic<unsigned> epoch_{0};
    std::atomic<int> pending_{0};
    call_t call_ = nullptr;
    void* ctx_ = nullptr;
    int n_ = 0, team_ = 1, max_ = 1, active_ = 1;
    bool stop_ = false;
};

} // namespace Laplace
