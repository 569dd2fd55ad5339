// Host-side meeting point of the ranks of an in-process group (one host thread per GPU).
//
// Before a rank enqueues a collective, every rank must know that all the others will enqueue it too: a rank that
// failed a local check (bad input, an allocation that did not fit) and returned would leave the GPUs of its peers
// waiting inside the collective.  So every phase that can fail locally ends with agree(): the ranks meet here, on
// the host, and either all go on or all give up.  A rank that dies outside such a point calls abandon(), which
// releases the waiting ranks with a failure.  A rank that never arrives is noticed by the time limit.
//
// Plain C++ (no CUDA, no NCCL) so that the logic can be exercised by CPU threads.
#pragma once
#include <chrono>
#include <condition_variable>
#include <mutex>

namespace tgbm {

class HostGroup {
public:
    HostGroup(int world, double timeout_s) : world_(world), timeout_s_(timeout_s) {}

    // Called by every rank with its own status.  true: all ranks arrived and all passed ok = true.
    // false: some rank reported a failure, left the group, or did not arrive within the time limit; from then on
    // the group is broken and every later call returns false at once.
    bool agree(bool ok) {
        std::unique_lock<std::mutex> lk(m_);
        if (broken_) return false;
        if (!ok) round_failed_ = true;
        const long my_round = round_;
        if (++arrived_ == world_) {
            result_ = !round_failed_;
            if (round_failed_) broken_ = true;
            arrived_ = 0;
            round_failed_ = false;
            ++round_;
            cv_.notify_all();
            return result_;
        }
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s_);
        while (round_ == my_round && !broken_) {
            if (cv_.wait_until(lk, deadline) == std::cv_status::timeout && round_ == my_round && !broken_) {
                broken_ = true;  // a rank is missing: nobody may enqueue the next collective
                cv_.notify_all();
                return false;
            }
        }
        return round_ != my_round ? result_ : false;
    }

    void abandon() {
        std::lock_guard<std::mutex> lk(m_);
        broken_ = true;
        cv_.notify_all();
    }

    bool broken() {
        std::lock_guard<std::mutex> lk(m_);
        return broken_;
    }
    int world() const { return world_; }

private:
    std::mutex m_;
    std::condition_variable cv_;
    const int world_;
    const double timeout_s_;
    int arrived_ = 0;
    long round_ = 0;
    bool round_failed_ = false, result_ = true, broken_ = false;
};

}  // namespace tgbm
