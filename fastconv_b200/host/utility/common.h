// Small host helpers the layer classes use (reference: utility/common.h:36-40).
#pragma once

#include <stddef.h>
#include <stdlib.h>

inline int align_ceil(int num, int align) { return (num + align - 1) / align * align; }
inline int min(int a, int b) { return a < b ? a : b; }

// Host allocations of the harness itself (inputs, outputs).  Device workspaces never come from here:
// they are carved from the GPU arena (utility/mempool.h).
inline void *_mm_malloc(size_t sz, size_t align = 64) {
    void *p = NULL;
    return posix_memalign(&p, align, sz) == 0 ? p : NULL;
}
inline void _mm_free(void *p) { free(p); }
