// Minimal stand-in for oneTBB, which the reference includes but does not vendor: the range classes and a
// parallel_for that cuts a range into chunks and runs them on a small pool of host threads (at most the parallelism
// the reference asks for through tbb::global_control, 21, and never more than the machine has).  TBB only schedules
// the reference's output tiles and packing loops; every output element is computed by the same sequence of operations
// whatever the schedule, so the results are the reference's bits.
#pragma once
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>
namespace tbb {
template <class T>
class blocked_range {
    T b_, e_;
   public:
    blocked_range(T b, T e, size_t = 1) : b_(b), e_(e) {}
    T begin() const { return b_; }
    T end() const { return e_; }
    size_t size() const { return e_ > b_ ? size_t(e_ - b_) : 0; }
};
template <class T>
class blocked_range2d {
    blocked_range<T> r_, c_;
   public:
    blocked_range2d(T rb, T re, T cb, T ce) : r_(rb, re), c_(cb, ce) {}
    blocked_range2d(T rb, T re, size_t, T cb, T ce, size_t) : r_(rb, re), c_(cb, ce) {}
    const blocked_range<T>& rows() const { return r_; }
    const blocked_range<T>& cols() const { return c_; }
};
template <class T>
class blocked_range3d {
    blocked_range<T> p_, r_, c_;
   public:
    blocked_range3d(T pb, T pe, T rb, T re, T cb, T ce) : p_(pb, pe), r_(rb, re), c_(cb, ce) {}
    blocked_range3d(T pb, T pe, size_t, T rb, T re, size_t, T cb, T ce, size_t) : p_(pb, pe), r_(rb, re), c_(cb, ce) {}
    const blocked_range<T>& pages() const { return p_; }
    const blocked_range<T>& rows() const { return r_; }
    const blocked_range<T>& cols() const { return c_; }
};

namespace detail {
inline std::atomic<size_t>& parallelism_limit() {
    static std::atomic<size_t> limit{0};   // 0: not set
    return limit;
}
// Runs job(i) for i in [0, n) on the pool's threads and the caller; returns when all are done.
class Pool {
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable wake_, done_;
    const std::function<void(size_t)>* job_ = nullptr;
    size_t n_ = 0, active_ = 0;
    unsigned long generation_ = 0;
    std::atomic<size_t> next_{0};
    bool stop_ = false;
    void work() {
        unsigned long seen = 0;
        for (;;) {
            const std::function<void(size_t)>* job;
            size_t n;
            {
                std::unique_lock<std::mutex> lk(mu_);
                wake_.wait(lk, [&] { return stop_ || generation_ != seen; });
                if (stop_) return;
                seen = generation_;
                job = job_;
                n = n_;
            }
            for (size_t i; (i = next_.fetch_add(1)) < n;) (*job)(i);
            std::unique_lock<std::mutex> lk(mu_);
            if (--active_ == 0) done_.notify_all();
        }
    }
   public:
    explicit Pool(size_t threads) {
        for (size_t t = 1; t < threads; ++t) workers_.emplace_back([this] { work(); });
    }
    ~Pool() {
        {
            std::unique_lock<std::mutex> lk(mu_);
            stop_ = true;
        }
        wake_.notify_all();
        for (auto& w : workers_) w.join();
    }
    size_t threads() const { return workers_.size() + 1; }
    void run(size_t n, const std::function<void(size_t)>& job) {
        if (n == 0) return;
        {
            std::unique_lock<std::mutex> lk(mu_);
            job_ = &job;
            n_ = n;
            next_.store(0);
            active_ = workers_.size();
            ++generation_;
        }
        wake_.notify_all();
        for (size_t i; (i = next_.fetch_add(1)) < n;) job(i);
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [&] { return active_ == 0; });
    }
    static Pool& instance() {
        static Pool pool([] {
            size_t hw = std::max<size_t>(1, std::thread::hardware_concurrency());
            const size_t want = parallelism_limit().load();
            return want ? std::min(hw, want) : std::min<size_t>(hw, 21);
        }());
        return pool;
    }
};
}  // namespace detail

template <class T, class Body>
void parallel_for(const blocked_range<T>& range, const Body& body) {
    detail::Pool& pool = detail::Pool::instance();
    const size_t n = range.size(), chunks = std::min(n, pool.threads() * 4);
    if (chunks <= 1) { body(range); return; }
    const std::function<void(size_t)> job = [&](size_t c) {
        body(blocked_range<T>(range.begin() + T(n * c / chunks), range.begin() + T(n * (c + 1) / chunks)));
    };
    pool.run(chunks, job);
}
template <class T, class Body>
void parallel_for(const blocked_range2d<T>& range, const Body& body) {
    detail::Pool& pool = detail::Pool::instance();
    const size_t nr = range.rows().size(), nc = range.cols().size();
    const size_t want = pool.threads() * 4;
    const size_t cr = std::min(nr, want), cc = cr >= want ? 1 : std::min(nc, (want + std::max<size_t>(cr, 1) - 1) / std::max<size_t>(cr, 1));
    if (cr * cc <= 1) { body(range); return; }
    const std::function<void(size_t)> job = [&](size_t c) {
        const size_t ri = c / cc, ci = c % cc;
        body(blocked_range2d<T>(range.rows().begin() + T(nr * ri / cr), range.rows().begin() + T(nr * (ri + 1) / cr),
                                range.cols().begin() + T(nc * ci / cc), range.cols().begin() + T(nc * (ci + 1) / cc)));
    };
    pool.run(cr * cc, job);
}
template <class T, class Body>
void parallel_for(const blocked_range3d<T>& range, const Body& body) {
    detail::Pool& pool = detail::Pool::instance();
    const size_t np = range.pages().size();
    if (np <= 1) { body(range); return; }
    const std::function<void(size_t)> job = [&](size_t c) {
        body(blocked_range3d<T>(range.pages().begin() + T(c), range.pages().begin() + T(c + 1), range.rows().begin(), range.rows().end(),
                                range.cols().begin(), range.cols().end()));
    };
    pool.run(np, job);
}
class global_control {
   public:
    enum parameter { max_allowed_parallelism };
    global_control(parameter, size_t n) { detail::parallelism_limit().store(n); }
};
class task_group {
   public:
    template <class F> void run(F&& f) { f(); }
    void wait() {}
};
}  // namespace tbb
