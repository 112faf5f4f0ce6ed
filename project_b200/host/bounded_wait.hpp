// The host-side wait of the exchange layer, kept free of CUDA and NCCL so that the give-up path can be
// exercised on a machine without a GPU: the caller supplies "is the stream drained?" and "tear the
// exchange down" as callables.  The reference has no counterpart (it is a single-process prover); the
// shape follows the usual collective watchdog: poll, and after the limit abort instead of blocking.
#pragma once
#include <chrono>
#include <thread>

namespace gzk
{
    enum class WaitState
    {
        Ready,     // the queued work completed
        Pending,   // still running
        Failed     // the query itself reported an error
    };

    enum class WaitResult
    {
        Completed,
        QueryFailed,
        TimedOut   // the limit ran out; on_timeout ran exactly once
    };

    // Polls query() until it stops answering Pending, for at most limit_seconds of wall clock.  When the
    // limit runs out on_timeout() is called once (it must end whatever the queue is stuck on, e.g. abort
    // the communicator) and TimedOut is returned.  `polls`, when given, receives the number of queries made.
    template <typename Query, typename OnTimeout>
    WaitResult bounded_wait(Query&& query, OnTimeout&& on_timeout, double limit_seconds, unsigned sleep_microseconds = 50,
                            unsigned long long* polls = nullptr)
    {
        const auto start = std::chrono::steady_clock::now();
        unsigned long long made = 0;
        for (;;)
        {
            const WaitState state = query();
            ++made;
            if (polls != nullptr) *polls = made;
            if (state == WaitState::Ready) return WaitResult::Completed;
            if (state == WaitState::Failed) return WaitResult::QueryFailed;
            const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
            if (waited > limit_seconds)
            {
                on_timeout();
                return WaitResult::TimedOut;
            }
            if (sleep_microseconds != 0) std::this_thread::sleep_for(std::chrono::microseconds(sleep_microseconds));
        }
    }
}
