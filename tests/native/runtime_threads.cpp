// The thread-heavy part of the native runtime under ThreadSanitizer: task executors, the asynchronous request state
// machine (start / wait / cancel / busy), the idle queue behind AsyncInferQueue, and the scheduler driven from a second
// thread the way a serving loop hands steps to a worker. Links runtime.cpp, sched.cpp and types.cpp only.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "runtime.hpp"
#include "sched.hpp"

using namespace ovc;

static void fail(const char* what) {
    std::fprintf(stderr, "runtime_threads: %s\n", what);
    std::exit(2);
}

int main() {
    // several requests share two executors; every request runs a two-stage pipeline and a callback
    auto ex_a = std::make_shared<TaskExecutor>(3, "stage-a");
    auto ex_b = std::make_shared<TaskExecutor>(2, "stage-b");
    constexpr int kRequests = 6, kRounds = 40;
    std::vector<std::shared_ptr<AsyncRequest>> reqs;
    std::vector<int> counters(kRequests, 0);
    std::atomic<int> callbacks{0};
    IdleQueue idle(kRequests);
    for (int r = 0; r < kRequests; ++r) {
        auto q = std::make_shared<AsyncRequest>();
        q->set_pipeline({{ex_a, [&counters, r] { counters[r] += 1; }}, {ex_b, [&counters, r] { counters[r] += 10; }}, {nullptr, [&counters, r] { counters[r] += 100; }}});
        q->set_callback([&callbacks, &idle, r](std::exception_ptr) { callbacks.fetch_add(1); idle.release((size_t)r); });
        reqs.push_back(q);
    }
    for (int round = 0; round < kRounds; ++round)
        for (int k = 0; k < kRequests; ++k) {
            const size_t slot = idle.acquire();
            reqs[slot]->start_async();
        }
    idle.wait_all();
    for (auto& q : reqs) q->wait();
    int total = 0;
    for (int c : counters) total += c;
    if (total != kRounds * kRequests * 111 || callbacks.load() != kRounds * kRequests) fail("lost or duplicated stage executions");

    // a request that is busy refuses a second start; cancel() lets wait() return with the cancellation error
    std::atomic<bool> release_stage{false};
    auto slow = std::make_shared<AsyncRequest>();
    slow->set_pipeline({{ex_a, [&release_stage] { while (!release_stage.load()) std::this_thread::yield(); }}, {ex_b, [] {}}});
    slow->start_async();
    bool busy = false;
    try { slow->start_async(); } catch (const BusyError&) { busy = true; }
    if (!busy) fail("second start_async on a running request did not throw");
    slow->cancel();
    release_stage.store(true);
    bool cancelled = false;
    try { slow->wait(); } catch (const CancelledError&) { cancelled = true; } catch (...) {}
    if (!cancelled) fail("wait() after cancel() did not report the cancellation");
    // a failing stage reaches wait() as its exception and the request is reusable afterwards
    auto bad = std::make_shared<AsyncRequest>();
    bad->set_pipeline({{ex_a, [] { throw Error("stage failed"); }}});
    bad->start_async();
    bool threw = false;
    try { bad->wait(); } catch (const Error&) { threw = true; }
    if (!threw) fail("stage exception was lost");
    bad->set_pipeline({{ex_b, [] {}}});
    bad->start_async();
    bad->wait();

    // scheduler: one thread schedules and commits, another patches token values one step behind (look-ahead of one)
    SchedulerConfig cfg;
    cfg.max_num_batched_tokens = 32;
    cfg.max_num_seqs = 4;
    cfg.num_kv_blocks = 12;
    cfg.block_size = 4;
    Scheduler sched(cfg);
    std::mutex mu;
    for (int r = 0; r < 8; ++r) sched.add(r, std::vector<int32_t>((size_t)(5 + r), 1 + r), 6, -1, true);
    std::vector<std::vector<Produced>> pending;
    std::atomic<bool> done{false};
    std::thread patcher([&] {
        while (!done.load() || [&] { std::lock_guard<std::mutex> lk(mu); return !pending.empty(); }()) {
            std::vector<Produced> p;
            {
                std::lock_guard<std::mutex> lk(mu);
                if (pending.empty()) { std::this_thread::yield(); continue; }
                p = std::move(pending.front());
                pending.erase(pending.begin());
                std::vector<int32_t> toks(8, 7);
                sched.patch(p, toks.data());
            }
        }
    });
    int steps = 0;
    for (;;) {
        std::lock_guard<std::mutex> lk(mu);
        if (!sched.has_unfinished()) break;
        ScheduledStep st;
        if (!sched.schedule(st)) fail("scheduler stalled");
        pending.push_back(sched.commit(st, nullptr));
        if (++steps > 1000) fail("scheduler does not terminate");
    }
    done.store(true);
    patcher.join();
    std::printf("RUNTIME_THREADS_OK\n");
    return 0;
}
