// TensorGEMM on the 5th-generation tensor cores (tcgen05 + TMEM), operands fed by TMA.
//
// For every Winograd position p the GEMM  M_p[oc][tile] = sum_ic U_p[oc][ic] * V_p[tile][ic]  has both
// operands K-major in global memory, which is exactly what a K-major UMMA shared-memory descriptor
// with 128-byte swizzle and a TMA box of 32 floats x rows want.  A work item is one 128(oc) x BN(tile)
// block of one position; the kernel is persistent: CTA b handles items b, b + gridDim.x, ... with
//
//   warp 0      TMA producer: cp.async.bulk.tensor 3-D boxes (ic, row, p) of U and V into a ring of
//               shared-memory stages that runs on across work items, one mbarrier per stage
//   warp 1      allocates TMEM (two accumulators of BN columns), then one elected lane issues
//               tcgen05.mma.cta_group::1.kind::tf32 (M=128, N=BN, K=8) four times per stage;
//               tcgen05.commit releases the stage and, after the last one, publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator (lane = oc row), hand the TMEM buffer back,
//               store to M -- while the MMA warp already fills the other accumulator.
//               In 3xTF32 mode the same warps first split every landed stage in place into
//               hi = tf32(x) and lo = x - hi, so each k-step becomes lo*hi + hi*lo + hi*hi with fp32
//               accumulation: fp32-class accuracy without touching HBM twice.
//
// Layers with at most 64 output channels run with the operand roles exchanged (kSwap): the 128 accumulator rows
// are 128 TILES and the N columns are the output channels, M_p^T[tile][oc] = sum_ic V_p[tile][ic] * U_p[oc][ic].
// Both operands are K-major either way, so only the descriptors trade places; no accumulator row is padding, and
// the epilogue's stores (lane = tile) are full 128-byte lines of M[p][oc][tile..].
//
// U is constant, so the producer fills the ring's U halves before griddepcontrol.wait (the kernel may
// have been launched while the input transform is still running) and adds V afterwards.
// The tensor core's fp32 accumulate rounds toward zero, so a sum kept in TMEM drifts by a bias that grows with the
// number of accumulation steps.  In the 3xTF32 mode (the accuracy mode) a long reduction is therefore cut into chunks
// of kb_chunk k-blocks: each chunk accumulates in one of the two TMEM buffers from zero, and the epilogue warps add the
// finished chunk to a running sum in registers with ordinary round-to-nearest additions while the MMA warp already
// fills the other buffer.  The bias then stops growing with the reduction length.
// Reduced-precision filter (kMode 2): the transformed filter is kept in HBM as fp16 -- the significand TF32 reads
// anyway -- scaled per position by a power of two, so the dominant stream of a single-image layer is half as long.
// The producer lands a box of 128 x 32 halves (8 KB) beside the stage, the four helper warps expand it into the
// swizzled fp32 operand slot (exact), the MMAs are the single-pass TF32 ones, and the epilogue multiplies the
// accumulator by the position's scale (exact).
// Every wait on an mbarrier is bounded: after the limit the kernel records FC_ERR_TIMEOUT in the
// context's status word, all roles drain, TMEM is released and the kernel returns.
#include <cstdlib>

#include <cuda_fp16.h>

#include "fc_tc_common.cuh"

namespace fc {

namespace {

using namespace tc;

struct TcParams {
    float *M;
    int *status;
    int oc, tp, bn, num_kb, stages, acc_cols;
    int n_tile_blk, n_oc_blk, n_items;
    int n_kb_u;  // boxes per (position, oc block) of the packed filter
    int n_oc_items;  // work items along the output channels: n_oc_blk blocks of 128, or blocks of `bn` with exchanged roles
    int b_bytes;     // bytes of the second operand slot of a stage
    int u_loads;     // exchanged roles: 128-row boxes of U per stage (1 or 2)
    int kb_chunk;    // k-blocks accumulated in TMEM before the sum is taken over into registers (>= num_kb: never)
    const float *scales;  // fp16 filter: the power of two every position's values were divided by, [64]
};

// row coordinate of U box (p, ocb, kb) in the packed filter viewed as a [boxes*128][32] matrix
__device__ __forceinline__ int u_box_row(const TcParams &P, int p, int oc0, int kb) {
    return ((p * P.n_oc_blk + (oc0 >> 7)) * P.n_kb_u + kb) * U_BOX_ROWS;
}

template <bool kSwap>
__device__ __forceinline__ void item_coords(const TcParams &P, int item, int &p, int &oc0, int &t0) {
    // tile block fastest, then oc block, then position: CTAs next to each other share the same U box
    const int tb = item % P.n_tile_blk;
    const int rest = item / P.n_tile_blk;
    t0 = tb * (kSwap ? BM : P.bn);  // exchanged roles: a block is 128 tiles (rows) x bn output channels (columns)
    oc0 = (rest % P.n_oc_items) * (kSwap ? P.bn : BM);
    p = rest / P.n_oc_items;
}

// two fp16 values in one 32-bit word -> two floats (exact)
__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t v) {
    float2 f;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
        : "=f"(f.x), "=f"(f.y)
        : "r"(v));
    return f;
}

constexpr int TC_SPLIT_THREADS = TC_THREADS + 128;  // 3xTF32 / fp16 filter: four more warps that only prepare stages
constexpr int A16_BYTES = BM * BK * 2;               // a filter box in fp16

// kMode: 0 = one TF32 pass, 1 = 3xTF32 (hi/lo split of every landed stage), 2 = one TF32 pass over an fp16 filter
template <int kMode, bool kSwap>
__global__ void __launch_bounds__(kMode != 0 ? TC_SPLIT_THREADS : TC_THREADS) wino_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmU,
                                                                  const __grid_constant__ CUtensorMap tmV,
                                                                  const TcParams P) {
    constexpr bool kSplit = kMode == 1, kU16 = kMode == 2, kHelpers = kMode != 0;
    static_assert(!(kU16 && kSwap), "the fp16 filter is built for rows = channels");
    extern __shared__ uint8_t smem_raw[];
    // carve: [barriers + flags | 1024-aligned stage ring]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[8] empty[8] split[8] acc_full[2] acc_empty[2]
    const int S = P.stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 28);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t ring = (smem_u32(smem_raw) + 512 + 1023) & ~1023u;
    const uint32_t b_bytes = (uint32_t)P.b_bytes;
    const uint32_t part_bytes = A_BYTES + b_bytes;  // one (A,B) pair
    const uint32_t stage_bytes = kSplit ? 2 * part_bytes : kU16 ? part_bytes + A16_BYTES : part_bytes;
    const uint32_t tx_bytes = kU16 ? b_bytes + A16_BYTES : part_bytes;  // what the producer lands per stage

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    auto bar_full = [&](int s) { return smem_u32(bars + s); };
    auto bar_empty = [&](int s) { return smem_u32(bars + 8 + s); };
    auto bar_split = [&](int s) { return smem_u32(bars + 16 + s); };
    auto bar_acc_full = [&](int a) { return smem_u32(bars + 24 + a); };
    auto bar_acc_empty = [&](int a) { return smem_u32(bars + 26 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
            mbar_init(bar_split(s), 128);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)(2 * P.acc_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // the first slot of a stage (A operand, 128 rows) and the second (B operand, bn rows): U, V or V, U
            auto load_u = [&](uint32_t stage, uint32_t bar, int p, int oc0, int kb) {
                if (kU16) {  // the fp16 box lands behind the operand slots; the helper warps expand it into slot A
                    tma_load_3d(stage + part_bytes, &tmU, bar, 0, u_box_row(P, p, oc0, kb), 0);
                    return;
                }
                tma_load_3d(stage + (kSwap ? A_BYTES : 0), &tmU, bar, 0, u_box_row(P, p, oc0, kb), 0);
                if (kSwap && P.u_loads == 2)  // channels oc0+128.. of a 256-wide block: the next packed box
                    tma_load_3d(stage + 2 * A_BYTES, &tmU, bar, 0, u_box_row(P, p, oc0 + BM, kb), 0);
            };
            auto load_v = [&](uint32_t stage, uint32_t bar, int p, int t0, int kb) {
                tma_load_3d(stage + (kSwap ? 0 : A_BYTES), &tmV, bar, kb * BK, t0, p);
            };
            int g = 0;  // k-blocks issued so far by this CTA, over all its items
            bool first = true, ok = true;
            for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
                int p, oc0, t0;
                item_coords<kSwap>(P, item, p, oc0, t0);
                int kb = 0;
                if (first) {
                    // the ring is empty: fill it with U boxes before waiting for the producer of V
                    const int pre = P.num_kb < S ? P.num_kb : S;
                    for (; kb < pre; ++kb) {
                        mbar_expect_tx(bar_full(kb), tx_bytes);
                        load_u(ring + kb * stage_bytes, bar_full(kb), p, oc0, kb);
                    }
                    pdl_wait();
                    for (int j = 0; j < pre; ++j) load_v(ring + j * stage_bytes, bar_full(j), p, t0, j);
                    g = pre;
                    first = false;
                }
                for (; kb < P.num_kb; ++kb, ++g) {
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, P.status);
                    if (!ok) break;
                    const uint32_t a_dst = ring + s * stage_bytes;
                    mbar_expect_tx(bar_full(s), tx_bytes);
                    load_u(a_dst, bar_full(s), p, oc0, kb);
                    load_v(a_dst, bar_full(s), p, t0, kb);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_tf32(BM, P.bn);
            int g = 0, it = 0;  // it counts accumulator hand-overs: one per chunk of a work item
            bool ok = true;
            for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
                uint32_t d_tmem = 0;
                int acc = 0;
                for (int kb = 0; kb < P.num_kb; ++kb, ++g) {
                    const bool chunk_start = kb % P.kb_chunk == 0;
                    if (chunk_start) {
                        acc = it & 1;
                        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                        ok = mbar_wait(bar_acc_empty(acc), acc_ph ^ 1u, abort_flag, P.status);  // epilogue drained it
                        if (!ok) break;
                        tc_fence_after();
                        d_tmem = tmem_base + (uint32_t)(acc * P.acc_cols);
                    }
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(kHelpers ? bar_split(s) : bar_full(s), ph, abort_flag, P.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_hi = ring + s * stage_bytes, b_hi = a_hi + A_BYTES;
                    const uint32_t a_lo = a_hi + part_bytes, b_lo = a_lo + A_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) {
                        const uint32_t koff = ks * 32;  // 8 tf32 = 32 bytes further along K inside the swizzle span
                        const uint32_t accum = (chunk_start && ks == 0) ? 0u : 1u;
                        if (kSplit) {
                            tc_mma_tf32(d_tmem, umma_desc_k_sw128(a_lo + koff), umma_desc_k_sw128(b_hi + koff), idesc, accum);
                            tc_mma_tf32(d_tmem, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_lo + koff), idesc, 1u);
                            tc_mma_tf32(d_tmem, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_hi + koff), idesc, 1u);
                        } else {
                            tc_mma_tf32(d_tmem, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_hi + koff), idesc, accum);
                        }
                    }
                    tc_commit(bar_empty(s));  // arrives once the MMAs above have finished reading the stage
                    if ((kb + 1) % P.kb_chunk == 0 || kb + 1 == P.num_kb) {  // the chunk is complete: hand it over
                        tc_commit(bar_acc_full(acc));
                        ++it;
                    }
                }
            }
        }
    } else if (warp >= 6) {
        // ---------------- splitters (3xTF32 only): warps 6..9 ----------------
        // hi = tf32(x) stays in place, lo = x - hi goes to the second half of the stage; the MMA warp waits for
        // bar_split instead of bar_full.  Warps of their own, so that splitting never queues behind an epilogue.
        const int et = threadIdx.x - TC_THREADS;  // 0..127
        int g = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
            if constexpr (kU16) {
                for (int kb = 0; kb < P.num_kb; ++kb, ++g) {
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(bar_full(s), ph, abort_flag, P.status);
                    if (!ok) break;
                    uint8_t *a32 = smem_raw + (ring - smem_u32(smem_raw)) + s * stage_bytes;
                    const uint8_t *a16 = a32 + part_bytes;  // 128 rows x 32 halves, rows of 64 bytes
                    for (int c = et; c < BM * 4; c += 128) {  // 16 bytes = 8 halves = two 16-byte pieces of floats
                        const int r = c >> 2, q = c & 3;
                        const uint4 raw = *reinterpret_cast<const uint4 *>(a16 + (size_t)c * 16);
                        const float2 f0 = half2_bits_to_float2(raw.x), f1 = half2_bits_to_float2(raw.y);
                        const float2 f2 = half2_bits_to_float2(raw.z), f3 = half2_bits_to_float2(raw.w);
                        // K-major, 128-byte swizzle: 16-byte piece index XOR row-in-group
                        const uint32_t row_off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
                        const uint32_t sw = (uint32_t)(r & 7);
                        *reinterpret_cast<float4 *>(a32 + row_off + ((((uint32_t)(2 * q)) ^ sw) << 4)) =
                            make_float4(f0.x, f0.y, f1.x, f1.y);
                        *reinterpret_cast<float4 *>(a32 + row_off + ((((uint32_t)(2 * q + 1)) ^ sw) << 4)) =
                            make_float4(f2.x, f2.y, f3.x, f3.y);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
                    mbar_arrive(bar_split(s));
                }
            } else {
                const int all_chunks = (int)(part_bytes / 16);
                for (int kb = 0; kb < P.num_kb; ++kb, ++g) {
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(bar_full(s), ph, abort_flag, P.status);
                    if (!ok) break;
                    float4 *hi = reinterpret_cast<float4 *>(smem_raw + (ring - smem_u32(smem_raw)) + s * stage_bytes);
                    float4 *lo = reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(hi) + part_bytes);
                    // element-wise at identical offsets: the swizzled placement of hi and lo stays that of TMA
                    for (int i = et; i < all_chunks; i += 128) {
                        const float4 v = hi[i];
                        float4 h, l;
                        h.x = to_tf32(v.x); h.y = to_tf32(v.y); h.z = to_tf32(v.z); h.w = to_tf32(v.w);
                        l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
                        hi[i] = h;
                        lo[i] = l;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
                    mbar_arrive(bar_split(s));
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int it = 0;
        bool ok = true, waited = false;
        const int n_chunks = (P.num_kb + P.kb_chunk - 1) / P.kb_chunk;
        for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
            int p, oc0, t0;
            item_coords<kSwap>(P, item, p, oc0, t0);
            if (!waited) {  // M may still be read by the output transform of the forward before this one
                pdl_wait();
                waited = true;
            }
            if constexpr (kSplit) {
                if (n_chunks > 1) {
                    // running sum of the chunks in registers: accumulator row of this lane, up to 128 columns
                    float sum[128];
#pragma unroll
                    for (int j = 0; j < 128; ++j) sum[j] = 0.0f;
                    for (int c = 0; c < n_chunks; ++c, ++it) {
                        const int acc = it & 1;
                        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                        ok = mbar_wait(bar_acc_full(acc), acc_ph, abort_flag, P.status);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * P.acc_cols);
#pragma unroll
                        for (int c0 = 0; c0 < 128; c0 += 16) {
                            if (c0 < P.bn) {
                                float va[16];
                                tc_ld16(t_addr + (uint32_t)c0, va);
                                // (the first chunk is added to +0, which leaves its bits alone)
#pragma unroll
                                for (int j = 0; j < 16; ++j) sum[c0 + j] = __fadd_rn(sum[c0 + j], va[j]);
                            }
                        }
                        tc_fence_before();
                        mbar_arrive(bar_acc_empty(acc));  // the MMA warp may start the chunk after next in this buffer
                    }
                    if (!ok) break;
                    if constexpr (kSwap) {
                        const int tile = t0 + q * 32 + lane;
                        float *dst = P.M + ((size_t)p * P.oc + oc0) * P.tp + tile;
                        if (tile < P.tp) {
#pragma unroll
                            for (int j = 0; j < 128; ++j)
                                if (j < P.bn && oc0 + j < P.oc) dst[(size_t)j * P.tp] = sum[j];
                        }
                    } else {
                        const int row = oc0 + q * 32 + lane;
                        float *dst = P.M + ((size_t)p * P.oc + row) * P.tp + t0;
                        if (row < P.oc) {
#pragma unroll
                            for (int j = 0; j < 128; j += 4)
                                if (j < P.bn && t0 + j < P.tp)  // tp is a multiple of 8: a float4 never straddles the end
                                    *reinterpret_cast<float4 *>(dst + j) = make_float4(sum[j], sum[j + 1], sum[j + 2], sum[j + 3]);
                        }
                    }
                    continue;
                }
            }
            const int acc = it & 1;
            const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
            ok = mbar_wait(bar_acc_full(acc), acc_ph, abort_flag, P.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * P.acc_cols);
            if constexpr (kSwap) {
                // accumulator row = tile, column = output channel: for every channel a warp stores 32 consecutive tiles
                const int tile = t0 + q * 32 + lane;
                float *dst = P.M + ((size_t)p * P.oc + oc0) * P.tp + tile;
                for (int c0 = 0; c0 < P.bn; c0 += 16) {
                    float va[16];
                    tc_ld16(t_addr + (uint32_t)c0, va);
                    if (c0 + 16 >= P.bn) {  // last columns read: the MMA warp may overwrite this accumulator
                        tc_fence_before();
                        mbar_arrive(bar_acc_empty(acc));
                    }
                    if (tile < P.tp) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (oc0 + c0 + j < P.oc) dst[(size_t)(c0 + j) * P.tp] = va[j];
                    }
                }
            } else {
                const int row = oc0 + q * 32 + lane;
                float *dst = P.M + ((size_t)p * P.oc + row) * P.tp + t0;
                const float scale = kU16 ? __ldg(P.scales + p) : 1.0f;  // a power of two: the product is exact
                for (int c0 = 0; c0 < P.bn; c0 += 32) {
                    float va[16], vb[16];
                    tc_ld16(t_addr + (uint32_t)c0, va);
                    const bool second = c0 + 16 < P.bn;
                    if (second) tc_ld16(t_addr + (uint32_t)(c0 + 16), vb);
                    if (kU16) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            va[j] *= scale;
                            if (second) vb[j] *= scale;
                        }
                    }
                    if (c0 + 32 >= P.bn) {  // last columns read: the MMA warp may overwrite this accumulator
                        tc_fence_before();
                        mbar_arrive(bar_acc_empty(acc));
                    }
                    if (row < P.oc) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            if (t0 + c0 + j < P.tp)  // tp is a multiple of 8: a float4 never straddles the end
                                *reinterpret_cast<float4 *>(dst + c0 + j) = make_float4(va[j], va[j + 1], va[j + 2], va[j + 3]);
                        if (second) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                if (t0 + c0 + 16 + j < P.tp)
                                    *reinterpret_cast<float4 *>(dst + c0 + 16 + j) =
                                        make_float4(vb[j], vb[j + 1], vb[j + 2], vb[j + 3]);
                        }
                    }
                }
            }
            ++it;
        }
    }

    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)(2 * P.acc_cols))
                     : "memory");
    }
}

}  // namespace

// The fp16 filter as a matrix [boxes*128][32 halves]; box = 128 rows x 32 halves, no swizzle (the helper warps place
// the expanded floats themselves).
static int make_map_u16(CUtensorMap *map, const void *base, size_t rows) {
    EncodeTiledFn enc;
    FC_PROPAGATE(get_encoder(&enc));
    cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)BK * 2, (cuuint64_t)BK * 2 * rows};
    cuuint32_t box[3] = {BK, (cuuint32_t)BM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FC_REQUIRE(r == CUDA_SUCCESS, FC_ERR_CUDA, "cuTensorMapEncodeTiled (fp16 filter) failed with %d", (int)r);
    return FC_OK;
}

// rows = channels, columns = tiles: the layout the fp16 filter is built for
bool wino_gemm_tc_rows_are_channels(const WinoGeom &g) { return !(g.oc <= 64 || g.tp >= 128); }

int launch_wino_gemm_tc(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g, int mode,
                        const KernelCfg *cfg, const float *d_scales) {
    const bool split = mode == FC_MATH_3XTF32, u16 = mode == FC_MATH_TF32_U16;
    FC_REQUIRE(!u16 || (d_scales != nullptr && wino_gemm_tc_rows_are_channels(g)), FC_ERR_INVALID_ARG,
               "the fp16 filter needs its scales and a layer whose accumulator rows are channels");
    // Exchanged roles (rows = 128 tiles, columns = a block of at most 128 output channels, a multiple of 16) when no
    // accumulator row is left empty by it: at most 64 channels, or at least 128 tiles.  Measured on the batch-8
    // VGG-16 stack: TF32 1.233 ms with rows = channels everywhere, 1.143 ms with this rule (3xTF32: 1.624 -> 1.577 ms);
    // 256-wide channel blocks (one CTA per SM, all of TMEM) were slower (1.197 ms).
    // Otherwise rows = 128 channels and tile blocks of at most 128 tiles (or the tuned width), balanced, a multiple
    // of 16 (UMMA N granularity at M=128).
    constexpr int swap_block = 128;
    const bool swap = g.oc <= 64 || g.tp >= 128;
    const int max_bn = cfg && cfg->bn >= 16 && cfg->bn <= 256 ? cfg->bn : 128;
    int n_blk, bn, n_oc_items, b_bytes, u_loads = 1;
    if (swap) {
        n_blk = (g.tp + BM - 1) / BM;
        n_oc_items = (g.oc + swap_block - 1) / swap_block;
        bn = round_up((g.oc + n_oc_items - 1) / n_oc_items, 16);       // balanced blocks of channels
        if (bn > BM) bn = round_up(bn, BM);                             // wider than one packed box: whole boxes
        u_loads = bn > BM ? 2 : 1;
        b_bytes = bn * BK * 4;
    } else {
        n_blk = (g.tp + max_bn - 1) / max_bn;
        bn = round_up((g.tp + n_blk - 1) / n_blk, 16);
        n_oc_items = g.n_ocb;
        b_bytes = bn * BK * 4;
    }
    TcParams P;
    P.M = d_M;
    P.status = ctx->d_status;
    P.oc = g.oc;
    P.tp = g.tp;
    P.bn = bn;
    P.num_kb = (g.icp + BK - 1) / BK;
    P.acc_cols = pow2_at_least(bn, 32);  // two accumulators: 2 * acc_cols TMEM columns (<= 512)
    P.n_tile_blk = n_blk;
    P.n_oc_blk = g.n_ocb;
    P.n_kb_u = g.n_kb;
    P.n_oc_items = n_oc_items;
    P.b_bytes = b_bytes;
    P.u_loads = u_loads;
    P.scales = d_scales;
    // 3xTF32: at most four k-blocks (128 input channels, 48 accumulation steps) per TMEM chunk; accumulator blocks wider
    // than 128 columns (a tuned configuration) keep the whole reduction in TMEM, their sum would not fit the registers
    P.kb_chunk = split && bn <= 128 ? 4 : P.num_kb;
    if (P.kb_chunk < 1) P.kb_chunk = 1;
    P.n_items = P.n_tile_blk * P.n_oc_items * 64;
    const size_t stage_bytes = split ? (size_t)2 * (A_BYTES + b_bytes) : (size_t)(A_BYTES + b_bytes) + (u16 ? A16_BYTES : 0);
    // More work items than SMs: size the ring so that two CTAs share an SM (one CTA's loads then overlap the
    // other's epilogue); otherwise one CTA takes the whole SM.  512 TMEM columns cannot be shared.
    const bool two_per_sm = P.n_items > ctx->sm_count && 2 * P.acc_cols <= 256;
    const size_t budget = cfg && cfg->smem_kb ? (size_t)cfg->smem_kb * 1024 : (two_per_sm ? 104 * 1024 : 200 * 1024);
    int stages = (int)(budget / stage_bytes);
    if (stages < 2) stages = 2;
    // a ring that no longer lets two CTAs share an SM (3xTF32 stages are twice as large) takes the whole SM instead
    if (!(cfg && cfg->smem_kb) && 512 + 1024 + stages * stage_bytes > 113 * 1024) stages = (int)((200 * 1024) / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    P.stages = stages;
    const size_t smem = 512 + 1024 + stages * stage_bytes;
    FC_REQUIRE(smem <= 227 * 1024, FC_ERR_UNSUPPORTED, "tile block of %d does not fit the shared-memory ring", bn);
    const int per_sm = (2 * P.acc_cols > 256 || smem > 113 * 1024) ? 1 : 2;
    int ctas = ctx->sm_count * per_sm;
    if (ctas > P.n_items) ctas = P.n_items;
    // FASTCONV_TC_MAX_CTAS caps the persistent grid (experiments: how fast a given number of SMs can pull the filter
    // stream -- the question a kernel that needs all 64 positions of a tile block in ONE CTA has to answer)
    static const int cta_cap = [] {
        const char *e = getenv("FASTCONV_TC_MAX_CTAS");
        return e && atoi(e) > 0 ? atoi(e) : 0;
    }();
    if (cta_cap > 0 && ctas > cta_cap) ctas = cta_cap;

    CUtensorMap tmU, tmV;  // box rows: the 128-row operand and the bn-row operand
    if (u16)
        FC_PROPAGATE(make_map_u16(&tmU, d_U, (size_t)64 * g.n_ocb * g.n_kb * U_BOX_ROWS));
    else
        FC_PROPAGATE(make_map_3d(&tmU, d_U, U_BOX_COLS, 64 * g.n_ocb * g.n_kb * U_BOX_ROWS, 1, swap && bn < U_BOX_ROWS ? bn : U_BOX_ROWS));
    FC_PROPAGATE(make_map_3d(&tmV, d_V, g.icp, g.tp, 64, swap ? BM : bn));

    dim3 grid((unsigned)ctas), block(split || u16 ? TC_SPLIT_THREADS : TC_THREADS);
    auto launch = [&](auto kernel) -> int {
        FC_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FC_CHECK_CUDA(launch_pdl(kernel, grid, block, smem, ctx->stream, tmU, tmV, P));
        return FC_OK;
    };
    if (u16) FC_PROPAGATE(launch(wino_gemm_tc_kernel<2, false>));
    else if (split) FC_PROPAGATE(swap ? launch(wino_gemm_tc_kernel<1, true>) : launch(wino_gemm_tc_kernel<1, false>));
    else FC_PROPAGATE(swap ? launch(wino_gemm_tc_kernel<0, true>) : launch(wino_gemm_tc_kernel<0, false>));
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
