// Host waits with a deadline: the MD loop never blocks for ever on a GPU or on a neighbour rank that has stopped
// answering (the reference's behaviour on a failed rank is an exception caught in main and MPI_Abort,
// src/main.cpp:85-93; here the wait returns a status and the caller aborts its communicator).
#pragma once

#include <chrono>
#include <thread>

namespace dsmd::host {

enum class WaitResult { kReady, kTimedOut, kFailed };

// Polls `query` (returns 1: done, 0: not yet, negative: failed) until it is done, fails, or `limit_s` seconds have
// passed. Spins for the first polls (the usual wait is microseconds), then yields the core between polls.
template <class Query>
WaitResult poll_until(Query query, double limit_s) {
    const auto start = std::chrono::steady_clock::now();
    for (unsigned long long polls = 0;; ++polls) {
        const int state = query();
        if (state > 0) return WaitResult::kReady;
        if (state < 0) return WaitResult::kFailed;
        if (polls >= 256) {
            if ((polls & 63) == 0) {
                const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
                if (waited > limit_s) return WaitResult::kTimedOut;
            }
            std::this_thread::yield();
        }
    }
}

}  // namespace dsmd::host
