// Device arena: one contiguous address range, sub-allocated on the host.
//
// Stands where the reference keeps its host allocators (utility/mempool.h:23-71,
// CommonMemPool / PrivateMemPool, and _mm_malloc in utility/common.cpp:26-39).
// The class only does address arithmetic on [base, base+capacity): it never
// dereferences the range, so the same code manages a cudaMalloc'd slab in the
// library and a fake range in the CPU unit tests.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>

namespace fc {

class Arena {
public:
    static constexpr size_t kAlign = 256;

    Arena() : base_(0), capacity_(0), in_use_(0), peak_(0) {}

    void reset(uintptr_t base, size_t capacity) {
        base_ = base;
        capacity_ = capacity - capacity % kAlign;
        in_use_ = peak_ = 0;
        used_.clear();
        free_.clear();
        if (capacity_ > 0) free_[0] = capacity_;
    }

    static size_t round_up(size_t bytes) { return (bytes + kAlign - 1) / kAlign * kAlign; }

    // Best-fit allocation; returns 0 when no free block is large enough.
    uintptr_t alloc(size_t bytes) {
        if (bytes == 0) bytes = 1;
        const size_t need = round_up(bytes);
        auto best = free_.end();
        for (auto it = free_.begin(); it != free_.end(); ++it)
            if (it->second >= need && (best == free_.end() || it->second < best->second)) best = it;
        if (best == free_.end()) return 0;
        const size_t off = best->first, len = best->second;
        free_.erase(best);
        if (len > need) free_[off + need] = len - need;
        used_[off] = need;
        in_use_ += need;
        if (in_use_ > peak_) peak_ = in_use_;
        return base_ + off;
    }

    bool owns(uintptr_t ptr) const { return ptr >= base_ && used_.count(ptr - base_) != 0; }

    size_t size_of(uintptr_t ptr) const {
        if (ptr < base_) return 0;
        auto it = used_.find(ptr - base_);
        return it == used_.end() ? 0 : it->second;
    }

    // Returns false for a pointer this arena did not hand out (or a double free).
    bool release(uintptr_t ptr) {
        if (ptr < base_) return false;
        auto it = used_.find(ptr - base_);
        if (it == used_.end()) return false;
        size_t off = it->first, len = it->second;
        used_.erase(it);
        in_use_ -= len;
        auto next = free_.lower_bound(off);
        if (next != free_.end() && off + len == next->first) {  // merge with the block after
            len += next->second;
            next = free_.erase(next);
        }
        if (next != free_.begin()) {  // merge with the block before
            auto prev = next;
            --prev;
            if (prev->first + prev->second == off) {
                prev->second += len;
                return true;
            }
        }
        free_[off] = len;
        return true;
    }

    void release_all() {
        used_.clear();
        free_.clear();
        in_use_ = 0;
        if (capacity_ > 0) free_[0] = capacity_;
    }

    size_t capacity() const { return capacity_; }
    size_t in_use() const { return in_use_; }
    size_t peak() const { return peak_; }
    size_t blocks() const { return used_.size(); }
    size_t free_fragments() const { return free_.size(); }
    size_t largest_free() const {
        size_t m = 0;
        for (auto &kv : free_)
            if (kv.second > m) m = kv.second;
        return m;
    }

private:
    uintptr_t base_;
    size_t capacity_, in_use_, peak_;
    std::map<size_t, size_t> used_;  // offset -> length
    std::map<size_t, size_t> free_;  // offset -> length
};

}  // namespace fc
