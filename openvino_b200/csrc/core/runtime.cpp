#include "runtime.hpp"

namespace ovc {

TaskExecutor::TaskExecutor(int n, std::string name) : name_(std::move(name)) {
    if (n <= 0) n = 1;
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { loop(); });
}
TaskExecutor::~TaskExecutor() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        stop_ = true;
    }
    cv_.notify_all();
    for (auto& w : workers_) if (w.joinable()) w.join();
}
void TaskExecutor::run(Task t) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        queue_.push_back(std::move(t));
    }
    cv_.notify_one();
}
void TaskExecutor::loop() {
    for (;;) {
        Task t;
        {
            std::unique_lock<std::mutex> lk(mu_);
            cv_.wait(lk, [&] { return stop_ || !queue_.empty(); });
            if (queue_.empty()) return;   // stop requested and nothing left to do
            t = std::move(queue_.front());
            queue_.pop_front();
        }
        t();
    }
}

// ------------------------------------------------------------------------------------ AsyncRequest
void AsyncRequest::begin() {
    std::lock_guard<std::mutex> lk(mu_);
    if (state_ == BUSY) throw BusyError();
    if (state_ == STOPPED) throw Error("Infer Request was stopped");
    state_ = BUSY;
    done_ = false;
    error_ = nullptr;
    t0_ = std::chrono::steady_clock::now();
}

void AsyncRequest::finish(std::exception_ptr e) {
    std::function<void(std::exception_ptr)> cb;
    {
        std::lock_guard<std::mutex> lk(mu_);
        latency_ms_ = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0_).count();
        if (state_ == CANCELLED && !e) e = std::make_exception_ptr(CancelledError());
        error_ = e;
        cb = callback_;
        // the request is IDLE again before the callback runs, so that the callback may start it anew
        if (state_ != STOPPED) state_ = IDLE;
    }
    if (cb) {
        try {
            cb(e);
        } catch (...) {
            std::lock_guard<std::mutex> lk(mu_);
            if (!error_) error_ = std::current_exception();
        }
    }
    {
        std::lock_guard<std::mutex> lk(mu_);
        done_ = true;
    }
    cv_.notify_all();
}

void AsyncRequest::run_stage(size_t i) {
    if (i >= pipeline_.size()) { finish(nullptr); return; }
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (state_ == CANCELLED) { /* fallthrough to finish below */ }
        else if (state_ != BUSY) return;
        if (state_ == CANCELLED) {
            // do not start further stages of a cancelled request
        }
    }
    if (state() == CANCELLED) { finish(nullptr); return; }
    auto self = shared_from_this();
    auto body = [self, i] {
        try {
            self->pipeline_[i].second();
        } catch (...) {
            self->finish(std::current_exception());
            return;
        }
        self->run_stage(i + 1);
    };
    if (pipeline_[i].first) pipeline_[i].first->run(body); else body();
}

void AsyncRequest::infer() {
    begin();
    std::exception_ptr e;
    try {
        for (auto& st : pipeline_) {
            if (state() == CANCELLED) break;
            st.second();
        }
    } catch (...) {
        e = std::current_exception();
    }
    finish(e);
    wait();
}

void AsyncRequest::start_async() {
    begin();
    run_stage(0);
}

void AsyncRequest::wait() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return done_; });
    if (error_) {
        auto e = error_;
        error_ = nullptr;
        std::rethrow_exception(e);
    }
}

bool AsyncRequest::wait_for(int64_t ms) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, std::chrono::milliseconds(ms), [&] { return done_; })) return false;
    if (error_) {
        auto e = error_;
        error_ = nullptr;
        std::rethrow_exception(e);
    }
    return true;
}

void AsyncRequest::cancel() {
    Task hook;
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (state_ == BUSY) { state_ = CANCELLED; hook = cancel_hook_; }
    }
    if (hook) hook();
}

void AsyncRequest::stop_and_wait() {
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return done_; });
        state_ = STOPPED;
    }
}

// ------------------------------------------------------------------------------------ IdleQueue
IdleQueue::IdleQueue(size_t n) : n_(n) { for (size_t i = 0; i < n; ++i) idle_.push_back(i); }
bool IdleQueue::is_ready() {
    std::lock_guard<std::mutex> lk(mu_);
    if (error_) { auto e = error_; error_ = nullptr; std::rethrow_exception(e); }
    return !idle_.empty();
}
size_t IdleQueue::get_idle() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !idle_.empty() || error_; });
    if (error_) { auto e = error_; error_ = nullptr; std::rethrow_exception(e); }
    return idle_.front();
}
size_t IdleQueue::acquire() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !idle_.empty() || error_; });
    if (error_) { auto e = error_; error_ = nullptr; std::rethrow_exception(e); }
    const size_t i = idle_.front();
    idle_.pop_front();
    return i;
}
void IdleQueue::release(size_t i) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        idle_.push_back(i);
    }
    cv_.notify_all();
}
void IdleQueue::wait_all() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return idle_.size() == n_; });
    if (error_) { auto e = error_; error_ = nullptr; std::rethrow_exception(e); }
}
void IdleQueue::set_error(std::exception_ptr e) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (!error_) error_ = e;
    }
    cv_.notify_all();
}
void IdleQueue::rethrow_if_error() {
    std::lock_guard<std::mutex> lk(mu_);
    if (error_) { auto e = error_; error_ = nullptr; std::rethrow_exception(e); }
}

}  // namespace ovc
