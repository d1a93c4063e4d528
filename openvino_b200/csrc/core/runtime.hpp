// Native runtime pieces shared by every device plugin: task executors (streams), the asynchronous
// infer-request state machine, the pool-based async queue, per-node profiling records.
//
// Roles covered: ITaskExecutor / CPUStreamsExecutor (src/inference/src/dev/threading/
// cpu_streams_executor.cpp:28-579), IAsyncInferRequest (src/inference/src/dev/iasync_infer_request.cpp:
// pipeline of (executor, task) stages :43-64, wait :66, cancel :100, start_async :194, Busy/Cancelled
// states iasync_infer_request.hpp:229-270), AsyncInferQueue (src/bindings/python/src/pyopenvino/core/
// async_infer_queue.cpp:20-178), ProfilingInfo (src/inference/include/openvino/runtime/profiling_info.hpp).
#pragma once
#include <condition_variable>
#include <deque>
#include <future>
#include <thread>

#include "graph.hpp"

namespace ovc {

struct BusyError : Error { BusyError() : Error("Infer Request is busy") {} };
struct CancelledError : Error { CancelledError() : Error("Infer Request was canceled") {} };

using Task = std::function<void()>;

class TaskExecutor {
public:
    explicit TaskExecutor(int num_threads, std::string name = "executor");
    ~TaskExecutor();
    void run(Task t);
    int num_threads() const { return (int)workers_.size(); }
    const std::string& name() const { return name_; }
private:
    void loop();
    std::string name_;
    std::vector<std::thread> workers_;
    std::deque<Task> queue_;
    std::mutex mu_;
    std::condition_variable cv_;
    bool stop_ = false;
};

// Runs tasks on the calling thread (the executor of synchronous infer()).
struct ImmediateExecutor {
    static void run(const Task& t) { t(); }
};

struct ProfilingInfo {
    enum Status { NOT_RUN, OPTIMIZED_OUT, EXECUTED } status = EXECUTED;
    double real_time_us = 0, cpu_time_us = 0;
    std::string node_name, exec_type, node_type;
};

// One asynchronous request: a pipeline of stages, each run on an executor; a user callback at the end.
class AsyncRequest : public std::enable_shared_from_this<AsyncRequest> {
public:
    using Stage = std::pair<std::shared_ptr<TaskExecutor>, Task>;   // null executor = run inline
    enum State { IDLE, BUSY, CANCELLED, STOPPED };

    void set_pipeline(std::vector<Stage> stages) { pipeline_ = std::move(stages); }
    void set_callback(std::function<void(std::exception_ptr)> cb) { std::lock_guard<std::mutex> lk(mu_); callback_ = std::move(cb); }
    void set_cancel_hook(Task t) { cancel_hook_ = std::move(t); }

    void infer();                       // run every stage on the calling thread; throws BusyError when running
    void start_async();                 // throws BusyError when running
    void wait();                        // rethrows the stage/callback exception
    bool wait_for(int64_t timeout_ms);  // true when the result is ready
    void cancel();
    void stop_and_wait();
    State state() const { std::lock_guard<std::mutex> lk(mu_); return state_; }
    double last_latency_ms() const { return latency_ms_; }

private:
    void begin();
    void run_stage(size_t i);
    void finish(std::exception_ptr e);
    std::vector<Stage> pipeline_;
    std::function<void(std::exception_ptr)> callback_;
    Task cancel_hook_;
    mutable std::mutex mu_;
    std::condition_variable cv_;
    State state_ = IDLE;
    bool done_ = true;
    std::exception_ptr error_;
    std::chrono::steady_clock::time_point t0_;
    double latency_ms_ = 0;
};

// Pool of request slots with an idle queue (the native half of AsyncInferQueue).
class IdleQueue {
public:
    explicit IdleQueue(size_t n);
    size_t size() const { return n_; }
    bool is_ready();                       // any slot idle
    size_t get_idle();                     // blocks until a slot is idle, returns its index (does not remove it)
    size_t acquire();                      // blocks, removes and returns an idle slot
    void release(size_t i);                // slot becomes idle again
    void wait_all();                       // blocks until every slot is idle
    void set_error(std::exception_ptr e);  // first error wins; rethrown by wait_all / acquire
    void rethrow_if_error();
private:
    size_t n_;
    std::deque<size_t> idle_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::exception_ptr error_;
};

}  // namespace ovc
