// Device-memory pools with the method names of the reference's host pools (utility/mempool.h:23-71).
//
// CommonMemPool  - scratch shared by layers that never run at the same time: every layer Requests its
//                  need under an id, Alloc() materialises max(requests) per id once, GetPtr hands it out.
// PrivateMemPool - per-object allocations that live until freed.
// Both sub-allocate the fc_context arena (one cudaMalloc'd slab); PTR_TYPE pointers are DEVICE pointers.
#pragma once

#include <stdio.h>

#include <map>

#include "fastconv_b200.h"

#define MEMPOOL_CHECK_RETURN(var)                                                \
    {                                                                            \
        if (!(var)) {                                                            \
            fprintf(stderr, "Err in file %s line %d: %s\n", __FILE__, __LINE__, fc_last_error()); \
            return false;                                                        \
        }                                                                        \
    }

template <typename PTR_TYPE>
class CommonMemPool {
public:
    explicit CommonMemPool(fc_context *ctx) : ctx_(ctx) {}
    ~CommonMemPool() { FreeAll(); }

    // default pool = id 0
    bool Request(size_t size_byte) { return Request(size_byte, 0); }
    bool GetPtr(PTR_TYPE **ptr) { return GetPtr(ptr, 0); }
    bool Free() { return Free(0); }

    bool Request(size_t size_byte, size_t id) {
        MEMPOOL_CHECK_RETURN(fc_arena_common_request(ctx_, size_byte, id) == FC_OK);
        ids_[id] = true;
        return true;
    }
    bool GetPtr(PTR_TYPE **ptr, size_t id) {
        void *p = NULL;
        MEMPOOL_CHECK_RETURN(fc_arena_common_ptr(ctx_, id, &p) == FC_OK);
        *ptr = static_cast<PTR_TYPE *>(p);
        return true;
    }
    bool Free(size_t id) {
        MEMPOOL_CHECK_RETURN(fc_arena_common_free(ctx_, id) == FC_OK);
        ids_.erase(id);
        return true;
    }
    bool Alloc() {
        MEMPOOL_CHECK_RETURN(fc_arena_common_commit(ctx_) == FC_OK);
        return true;
    }
    bool Alloc(size_t size_byte) { return Request(size_byte, 0) && Alloc(); }
    bool FreeAll() {
        bool ok = true;
        while (!ids_.empty()) ok = Free(ids_.begin()->first) && ok;
        return ok;
    }
    void PrintStats() {
        size_t cap = 0, use = 0, peak = 0, blocks = 0;
        fc_arena_stats(ctx_, &cap, &use, &peak, &blocks);
        printf("Common pools: %zu ids; arena %zu / %zu bytes in use (peak %zu, %zu blocks)\n", ids_.size(), use, cap,
               peak, blocks);
    }

private:
    fc_context *ctx_;
    std::map<size_t, bool> ids_;
};

template <typename PTR_TYPE>
class PrivateMemPool {
public:
    explicit PrivateMemPool(fc_context *ctx) : ctx_(ctx) {}
    ~PrivateMemPool() { FreeAll(); }

    bool Alloc(PTR_TYPE **ptr, size_t size_byte) {
        void *p = NULL;
        MEMPOOL_CHECK_RETURN(fc_arena_alloc(ctx_, size_byte, &p) == FC_OK);
        *ptr = static_cast<PTR_TYPE *>(p);
        private_map_[*ptr] = size_byte;
        return true;
    }
    bool GetSize(PTR_TYPE *ptr, size_t *size_byte) {
        typename std::map<PTR_TYPE *, size_t>::iterator it = private_map_.find(ptr);
        MEMPOOL_CHECK_RETURN(it != private_map_.end());
        *size_byte = it->second;
        return true;
    }
    bool Free(PTR_TYPE **ptr) {
        typename std::map<PTR_TYPE *, size_t>::iterator it = private_map_.find(*ptr);
        MEMPOOL_CHECK_RETURN(it != private_map_.end());
        MEMPOOL_CHECK_RETURN(fc_arena_free(ctx_, *ptr) == FC_OK);
        private_map_.erase(it);
        *ptr = NULL;
        return true;
    }
    bool FreeAll() {
        bool ok = true;
        while (!private_map_.empty()) {
            PTR_TYPE *p = private_map_.begin()->first;
            ok = Free(&p) && ok;
        }
        return ok;
    }
    void PrintStats() {
        size_t total = 0;
        for (typename std::map<PTR_TYPE *, size_t>::iterator it = private_map_.begin(); it != private_map_.end(); ++it)
            total += it->second;
        printf("Private pool: %zu blocks, %zu bytes\n", private_map_.size(), total);
    }

private:
    fc_context *ctx_;
    std::map<PTR_TYPE *, size_t> private_map_;
};
