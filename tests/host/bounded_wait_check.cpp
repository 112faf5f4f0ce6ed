// CPU check of the exchange layer's host-side wait (project_b200/host/bounded_wait.hpp): a peer that
// never posts is modelled by a query that stays Pending; the wait must give up after the limit, call the
// abort hook exactly once and report TimedOut.  No GPU and no NCCL are involved.
#include <atomic>
#include <cstdio>
#include <thread>

#include "../../project_b200/host/bounded_wait.hpp"

static int failures = 0;
#define CHECK(cond, what)                                   \
    do                                                      \
    {                                                       \
        if (!(cond))                                        \
        {                                                   \
            std::printf("FAIL: %s\n", what);                \
            ++failures;                                     \
        }                                                   \
    } while (0)

int main()
{
    using namespace gzk;
    // 1. the peer never posts
    {
        int aborts = 0;
        unsigned long long polls = 0;
        const auto t0 = std::chrono::steady_clock::now();
        const WaitResult r = bounded_wait([] { return WaitState::Pending; }, [&] { ++aborts; }, 0.05, 50, &polls);
        const double took = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        CHECK(r == WaitResult::TimedOut, "a query that stays pending times out");
        CHECK(aborts == 1, "the abort hook runs exactly once");
        CHECK(took >= 0.05 && took < 2.0, "the wait ends shortly after the limit");
        CHECK(polls > 1, "the stream was polled more than once");
    }
    // 2. the peer posts late, but inside the limit (another thread flips the flag)
    {
        std::atomic<bool> posted{false};
        int aborts = 0;
        std::thread peer([&] {
            std::this_thread::sleep_for(std::chrono::milliseconds(20));
            posted.store(true);
        });
        const WaitResult r = bounded_wait([&] { return posted.load() ? WaitState::Ready : WaitState::Pending; }, [&] { ++aborts; }, 5.0);
        peer.join();
        CHECK(r == WaitResult::Completed, "a late post inside the limit completes");
        CHECK(aborts == 0, "no abort when the work completes");
    }
    // 3. already drained: one query, no sleep
    {
        unsigned long long polls = 0;
        const WaitResult r = bounded_wait([] { return WaitState::Ready; }, [] {}, 1.0, 50, &polls);
        CHECK(r == WaitResult::Completed && polls == 1, "a drained queue answers on the first query");
    }
    // 4. the query reports an error: returned as such, the abort hook does not run
    {
        int aborts = 0;
        int calls = 0;
        const WaitResult r = bounded_wait([&] { return ++calls < 3 ? WaitState::Pending : WaitState::Failed; }, [&] { ++aborts; }, 5.0);
        CHECK(r == WaitResult::QueryFailed && aborts == 0 && calls == 3, "a failing query ends the wait without an abort");
    }
    std::printf(failures == 0 ? "OK\n" : "FAILED %d\n", failures);
    return failures == 0 ? 0 : 1;
}
