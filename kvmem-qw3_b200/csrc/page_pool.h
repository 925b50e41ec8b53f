// Physical K/V page pool shared by the sequences of a batch (the role of GlobalKvPagePool,
// src/qwen_native_backend.cpp:1155-1265: one pool of pool_pages pages per cache tensor, a LIFO free stack that hands out
// page 0 first, pages of a cached prompt prefix kept alive while something still refers to them, a mutex because
// server threads release pages).  Here a page carries a holder count instead of a pin flag plus an "owned" flag: a
// sequence that allocates a page holds it once, a prefix entry or a second sequence sharing it holds it once more, and
// the page returns to the free stack when its last holder drops it.  Host-side only; the device sees page ids through
// the batch's page table.
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>

class QbPagePool {
public:
    explicit QbPagePool(uint32_t total) : holders_(total, 0) {
        free_.reserve(total);
        for (uint32_t i = 0; i < total; ++i) free_.push_back((int32_t)(total - 1 - i));      // page 0 on top
    }
    // A free page with one holder, or -1 when the pool is exhausted.
    int32_t alloc() {
        std::lock_guard<std::mutex> lk(mu_);
        if (free_.empty()) return -1;
        const int32_t p = free_.back();
        free_.pop_back();
        holders_[(size_t)p] = 1;
        return p;
    }
    // One more holder of a page that is in use; false for a page id that is free or out of range.
    bool share(int32_t p) {
        std::lock_guard<std::mutex> lk(mu_);
        if (p < 0 || (size_t)p >= holders_.size() || holders_[(size_t)p] == 0) return false;
        ++holders_[(size_t)p];
        return true;
    }
    // One holder less; the page goes back on top of the free stack with the last one.  Returns the holders left,
    // -1 for a page id that is free or out of range (nothing changes then).
    int32_t drop(int32_t p) {
        std::lock_guard<std::mutex> lk(mu_);
        if (p < 0 || (size_t)p >= holders_.size() || holders_[(size_t)p] == 0) return -1;
        if (--holders_[(size_t)p] == 0) free_.push_back(p);
        return (int32_t)holders_[(size_t)p];
    }
    uint32_t free_count() const { std::lock_guard<std::mutex> lk(mu_); return (uint32_t)free_.size(); }
    uint32_t total() const { return (uint32_t)holders_.size(); }
    uint32_t holders(int32_t p) const {
        std::lock_guard<std::mutex> lk(mu_);
        return p < 0 || (size_t)p >= holders_.size() ? 0 : holders_[(size_t)p];
    }
    // Whole-pool state for batch snapshots.
    struct State { std::vector<int32_t> free; std::vector<uint32_t> holders; };
    State save() const { std::lock_guard<std::mutex> lk(mu_); return State{free_, holders_}; }
    void load(const State &s) { std::lock_guard<std::mutex> lk(mu_); free_ = s.free; holders_ = s.holders; }

private:
    mutable std::mutex mu_;
    std::vector<int32_t> free_;
    std::vector<uint32_t> holders_;
};
