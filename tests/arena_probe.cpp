// CPU probe of the device arena's bookkeeping (fastconv_b200/csrc/fc_arena.h) over a fake address
// range; built and driven by tests/test_arena_cpu.py.
#include "../fastconv_b200/csrc/fc_arena.h"

static fc::Arena g_arena;

extern "C" {
void probe_reset(unsigned long long base, unsigned long long cap) { g_arena.reset(base, cap); }
unsigned long long probe_alloc(unsigned long long bytes) { return g_arena.alloc(bytes); }
int probe_release(unsigned long long p) { return g_arena.release(p) ? 1 : 0; }
unsigned long long probe_size_of(unsigned long long p) { return g_arena.size_of(p); }
unsigned long long probe_in_use() { return g_arena.in_use(); }
unsigned long long probe_peak() { return g_arena.peak(); }
unsigned long long probe_blocks() { return g_arena.blocks(); }
unsigned long long probe_fragments() { return g_arena.free_fragments(); }
unsigned long long probe_largest_free() { return g_arena.largest_free(); }
void probe_release_all() { g_arena.release_all(); }
}
