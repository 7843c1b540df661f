// TensorGEMM, fp32 "mirrored" mode: 64 independent GEMMs
//     M_p[oc][tile] = sum_ic U_p[ic][oc] * V_p[ic][tile]
// on the FP32 pipes, with the reference's accumulation chain kept exactly: every output element
// owns ONE accumulator that starts at 0 and takes one fused multiply-add per input channel, in
// ascending channel order (TensorGEMMInnerKernel4x4x5_v1, winoF63ZC/TensorGEMMZC.cpp:585-697;
// ic blocks of the reference continue the same chain through gemmBuf).  No split-K, no pairwise
// sums, no reordering -- that is what makes the layer bit-identical to the reference.
//
// Operands arrive in the row-major layouts U[p][icp][ocp] / V[p][icp][tp] (row index contiguous), so a
// BK x BM slab of U and a BK x BN slab of V are sets of contiguous runs: they go to shared memory as [k][row]
// and the inner product reads 128-bit rows without bank conflicts.  No register staging, no transposition, two
// CTAs per SM.  Behind a context the slabs are TMA boxes in a ring of mbarrier-guarded stages
// (wino_gemm_ffma_tma_kernel, further down); callers without one get the same blocks on 16-byte asynchronous
// copies (cp.async, zero-filled past the edges) through a 4-stage ring with a block-wide barrier per slab.  The
// FMAs of two neighbouring tiles are issued as one packed instruction (fma.rn.f32x2): each half rounds like a
// scalar FMA, so the chains are unchanged.
#include <cstdlib>

#include "fc_tc_common.cuh"

namespace fc {

namespace {

constexpr int BK = 16;
constexpr int THREADS = 256;
constexpr int STAGES = 4;

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Packed fp32 arithmetic of sm_100: one instruction, two independent IEEE fused multiply-adds (lo and hi halves of
// 64-bit register pairs).  Each half rounds exactly like a scalar fma.rn, so the accumulation chains are unchanged;
// what changes is that the same math needs half the issue slots.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int BM, int BN, int MAP = 0, int BK = 16, int STAGES = 4>
__global__ void __launch_bounds__(THREADS, 2) wino_gemm_ffma_kernel(const float *__restrict__ U,
                                                                    const float *__restrict__ V, float *__restrict__ M,
                                                                    int oc, int ocp, int tp, int icp) {
    constexpr int TM = BM / 16, TN = BN / 16;  // outputs per thread: TM output channels x TN tiles
    constexpr int A_CHUNKS = BK * BM / 4 / THREADS, B_CHUNKS = BK * BN / 4 / THREADS;
    static_assert(A_CHUNKS >= 1 && B_CHUNKS >= 1 && TM % 4 == 0 && TN % 4 == 0, "block shape");
    extern __shared__ __align__(16) float smem[];
    float(*As)[BK][BM] = reinterpret_cast<float(*)[BK][BM]>(smem);
    float(*Bs)[BK][BN] = reinterpret_cast<float(*)[BK][BN]>(smem + STAGES * BK * BM);

    const int p = blockIdx.z, oc0 = blockIdx.y * BM, t0 = blockIdx.x * BN;
    const float *Up = U + (size_t)p * icp * ocp;
    const float *Vp = V + (size_t)p * icp * tp;
    const int tid = threadIdx.x;
    // MAP 0: a warp is 16 tile columns x 2 channel rows; MAP 1: 8 x 4, so that each 128-bit operand read of a warp
    // is one 128-byte wavefront (measured 2 % faster on the 128 x 128 block, no gain on the 64-row blocks)
    const int tx = MAP == 0 ? tid % 16 : (tid / 32 % 2) * 8 + tid % 8;
    const int ty = MAP == 0 ? tid / 16 : (tid / 64) * 4 + tid % 32 / 8;

    auto load_stage = [&](int stage, int k0) {
#pragma unroll
        for (int i = 0; i < A_CHUNKS; ++i) {
            const int idx = tid + i * THREADS;
            const int kr = idx / (BM / 4), c4 = (idx % (BM / 4)) * 4;
            const int k = k0 + kr, col = oc0 + c4;
            const bool ok = k < icp && col < ocp;
            cp_async_16(&As[stage][kr][c4], Up + (ok ? (size_t)k * ocp + col : 0), ok);
        }
#pragma unroll
        for (int i = 0; i < B_CHUNKS; ++i) {
            const int idx = tid + i * THREADS;
            const int kr = idx / (BN / 4), c4 = (idx % (BN / 4)) * 4;
            const int k = k0 + kr, col = t0 + c4;
            const bool ok = k < icp && col < tp;
            cp_async_16(&Bs[stage][kr][c4], Vp + (ok ? (size_t)k * tp + col : 0), ok);
        }
    };

    // accumulators as pairs of neighbouring tiles: one packed FMA per pair (same rounding per element as a scalar FMA)
    uint64_t acc2[TM][TN / 2];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc2[i][j] = 0ull;  // (+0.0f, +0.0f)

    pdl_trigger();
    pdl_wait();  // V comes from the input transform launched just before

    const int n_slabs = (icp + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_slabs) load_stage(s, s * BK);
        cp_async_commit();
    }
    for (int kt = 0; kt < n_slabs; ++kt) {
        cp_async_wait<STAGES - 2>();  // slab kt has landed (for this thread's copies) ...
        __syncthreads();              // ... and for everyone's; everyone is also done with slab kt-1
        const int next = kt + STAGES - 1;
        if (next < n_slabs) load_stage(next % STAGES, next * BK);  // overwrites the stage slab kt-1 used
        cp_async_commit();
        const int buf = kt % STAGES;
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
            // rows are taken in float4 groups strided by 64 (16 threads x 4), so a warp's 128-bit reads
            // of one k-row touch consecutive banks
#pragma unroll
            for (int g = 0; g < TM / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&As[buf][k][g * 64 + ty * 4]);
                a[g * 4 + 0] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < TN / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&Bs[buf][k][g * 64 + tx * 4]);
                b[g * 4 + 0] = v.x; b[g * 4 + 1] = v.y; b[g * 4 + 2] = v.z; b[g * 4 + 3] = v.w;
            }
            uint64_t bp[TN / 2];
#pragma unroll
            for (int j = 0; j < TN / 2; ++j) bp[j] = pack2(b[2 * j], b[2 * j + 1]);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const uint64_t ap = pack2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < TN / 2; ++j) acc2[i][j] = fma2(ap, bp[j], acc2[i][j]);
            }
        }
    }
    cp_async_wait<0>();

    float *Mp = M + (size_t)p * oc * tp;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = oc0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= oc) continue;
#pragma unroll
        for (int g = 0; g < TN / 4; ++g) {
            const int c = t0 + g * 64 + tx * 4;
            if (c < tp) {  // tp is a multiple of 8, so a float4 never straddles the end
                float4 v;
                unpack2(acc2[i][g * 2 + 0], v.x, v.y);
                unpack2(acc2[i][g * 2 + 1], v.z, v.w);
                *reinterpret_cast<float4 *>(Mp + (size_t)r * tp + c) = v;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Tile counts between the block widths: 72 tiles (14x14 maps of 8 images) fill 56 % of two 64-wide blocks, 200 tiles
// (28x28 of 8 images) 78 % of two 128-wide ones.  Here a thread owns 8 output channels x TN tiles with TN = 5, 6 or 7,
// so a block is 128 x 80, 96 or 112 and the launcher picks the width that pads least.  The tiles of a thread are
// 16 apart (tx, tx + 16, ...), read from shared memory one float at a time (a half-warp reads 16 consecutive floats,
// the other half the same ones: one wavefront); everything else -- cp.async ring, one accumulator per output, one
// fused multiply-add per input channel in ascending order, packed pairs -- is the kernel above.
// ---------------------------------------------------------------------------------------------
template <int TN>
__global__ void __launch_bounds__(THREADS, 2) wino_gemm_ffma_flex_kernel(const float *__restrict__ U,
                                                                         const float *__restrict__ V, float *__restrict__ M,
                                                                         int oc, int ocp, int tp, int icp) {
    constexpr int BM = 128, BN = 16 * TN, TM = 8;
    constexpr int A_CHUNKS = BK * BM / 4 / THREADS, B_TOTAL = BK * BN / 4, TP2 = TN / 2;
    extern __shared__ __align__(16) float smem[];
    float(*As)[BK][BM] = reinterpret_cast<float(*)[BK][BM]>(smem);
    float(*Bs)[BK][BN] = reinterpret_cast<float(*)[BK][BN]>(smem + STAGES * BK * BM);

    const int p = blockIdx.z, oc0 = blockIdx.y * BM, t0 = blockIdx.x * BN;
    const float *Up = U + (size_t)p * icp * ocp;
    const float *Vp = V + (size_t)p * icp * tp;
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;

    auto load_stage = [&](int stage, int k0) {
#pragma unroll
        for (int i = 0; i < A_CHUNKS; ++i) {
            const int idx = tid + i * THREADS;
            const int kr = idx / (BM / 4), c4 = (idx % (BM / 4)) * 4;
            const int k = k0 + kr, col = oc0 + c4;
            const bool ok = k < icp && col < ocp;
            cp_async_16(&As[stage][kr][c4], Up + (ok ? (size_t)k * ocp + col : 0), ok);
        }
        for (int idx = tid; idx < B_TOTAL; idx += THREADS) {
            const int kr = idx / (BN / 4), c4 = (idx % (BN / 4)) * 4;
            const int k = k0 + kr, col = t0 + c4;
            const bool ok = k < icp && col < tp;  // tp is a multiple of 8 and so is t0: a 16-byte piece never straddles
            cp_async_16(&Bs[stage][kr][c4], Vp + (ok ? (size_t)k * tp + col : 0), ok);
        }
    };

    uint64_t acc2[TM][TP2 > 0 ? TP2 : 1];
    float acc1[TM];  // the odd tile of a thread, when TN is odd
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        acc1[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < TP2; ++j) acc2[i][j] = 0ull;
    }

    pdl_trigger();
    pdl_wait();  // V comes from the input transform launched just before

    const int n_slabs = (icp + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_slabs) load_stage(s, s * BK);
        cp_async_commit();
    }
    for (int kt = 0; kt < n_slabs; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        const int next = kt + STAGES - 1;
        if (next < n_slabs) load_stage(next % STAGES, next * BK);
        cp_async_commit();
        const int buf = kt % STAGES;
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int g = 0; g < TM / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&As[buf][k][g * 64 + ty * 4]);
                a[g * 4 + 0] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[buf][k][tx + 16 * j];
            uint64_t bp[TP2 > 0 ? TP2 : 1];
#pragma unroll
            for (int j = 0; j < TP2; ++j) bp[j] = pack2(b[2 * j], b[2 * j + 1]);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const uint64_t ap = pack2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < TP2; ++j) acc2[i][j] = fma2(ap, bp[j], acc2[i][j]);
                if constexpr (TN % 2 == 1) acc1[i] = __fmaf_rn(a[i], b[TN - 1], acc1[i]);
            }
        }
    }
    cp_async_wait<0>();

    float *Mp = M + (size_t)p * oc * tp;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = oc0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= oc) continue;
        float res[TN];
#pragma unroll
        for (int j = 0; j < TP2; ++j) unpack2(acc2[i][j], res[2 * j], res[2 * j + 1]);
        if constexpr (TN % 2 == 1) res[TN - 1] = acc1[i];
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int c = t0 + tx + 16 * j;
            if (c < tp) Mp[(size_t)r * tp + c] = res[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Few tiles (small feature maps at batch 1: 28x28 -> 25 tiles, 14x14 -> 9, 7x7 -> 4).  The GEMM is a
// stream over U with a short N, so the blocked kernel above would multiply mostly padding.  Here a CTA
// owns 128 output channels and all tiles of one position.  A producer warp keeps a ring of stages in
// flight with TMA, each stage a 32(ic) x 128(oc) box of U and the matching 32(ic) x tp box of V, so
// neither HBM nor L2 latency is waited for by the math warps.  There are four consumer warps, one per
// scheduler of the SM, each covering 32 channels x 4*TT tiles as 8 x 4 lanes: a lane owns 4 channels (one
// 128-bit read of the landed U row, shared by the 4 lanes of its column) and TT consecutive tiles (read
// from the V row, shared by the 8 lanes of its row).  Both operands are thus reused across lanes inside
// one shared-memory read, which is what keeps the kernel off the shared-memory bandwidth limit: a lane
// per channel with broadcast V reads measured 0.34 issue slots used and 61 us for 512->512 at 25 tiles.
// Operands of k-step kk+1 are read while the FMAs of kk issue.  The chain per output element is
// unchanged: one accumulator, one FMA per input channel, ascending.
// ---------------------------------------------------------------------------------------------
constexpr int ST_STAGES = 5;
constexpr int ST_BOX = 128 * 32 * 4;         // bytes of a U box
constexpr int ST_VBOX = 32 * 32 * 4;         // room for a V box (32 k-rows of tp <= 32 floats)
constexpr int ST_STAGE = ST_BOX + ST_VBOX;
constexpr int ST_THREADS = 160;              // 4 consumer warps + 1 producer warp

template <int TT>
__global__ void __launch_bounds__(ST_THREADS, 2)
    wino_gemm_ffma_skinny_tma_kernel(const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmV,
                                     float *__restrict__ M, int *status, int oc, int tp, int icp) {
    using namespace tc;
    static_assert(TT == 1 || TT == 2 || TT == 4 || TT == 8, "tiles per lane");
    extern __shared__ uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[ST_STAGES], empty[ST_STAGES]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * ST_STAGES);
    const uint32_t ring = (smem_u32(smem_raw) + 128 + 127) & ~127u;
    const uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = blockIdx.y, oc0 = blockIdx.x * 128;
    const int num_kb = (icp + 31) / 32;
    const uint32_t stage_bytes = ST_BOX + 32u * (uint32_t)tp * 4u;
    auto bar_full = [&](int s) { return smem_u32(bars + s); };
    auto bar_empty = [&](int s) { return smem_u32(bars + ST_STAGES + s); };

    if (tid == 0) {
        for (int s = 0; s < ST_STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    if (warp == 4) {
        if (lane == 0) {
            // U is constant, so the first ring of U boxes is requested before the input transform that writes V
            // is known to be complete; V boxes follow after the wait
            const int head = num_kb < ST_STAGES ? num_kb : ST_STAGES;
            for (int kb = 0; kb < head; ++kb) {
                mbar_expect_tx(bar_full(kb), stage_bytes);
                tma_load_3d(ring + kb * ST_STAGE, &tmU, bar_full(kb), oc0, kb * 32, p);  // box: 128 oc x 32 ic
            }
            pdl_wait();
            for (int kb = 0; kb < head; ++kb)
                tma_load_3d(ring + kb * ST_STAGE + ST_BOX, &tmV, bar_full(kb), 0, kb * 32, p);  // box: tp tiles x 32 ic
            for (int kb = head; kb < num_kb; ++kb) {
                const int s = kb % ST_STAGES;
                const uint32_t ph = (uint32_t)(kb / ST_STAGES) & 1u;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, status)) break;
                mbar_expect_tx(bar_full(s), stage_bytes);
                tma_load_3d(ring + s * ST_STAGE, &tmU, bar_full(s), oc0, kb * 32, p);
                tma_load_3d(ring + s * ST_STAGE + ST_BOX, &tmV, bar_full(s), 0, kb * 32, p);
            }
        }
    } else {
        const int ocl = warp * 32 + (lane & 7) * 4;  // first of this lane's 4 channels within the box
        const int j0 = (lane >> 3) * TT;             // first of this lane's TT tiles
        // accumulators: pairs of neighbouring tiles in one 64-bit register (one packed FMA updates both); a single
        // tile per lane stays scalar
        constexpr int TP = TT >= 2 ? TT / 2 : 1;
        uint64_t acc2[4][TP];
        float acc1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc1[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < TP; ++j) acc2[i][j] = 0ull;  // (+0.0f, +0.0f)
        }
        // TT floats of a V row; lanes past the last real tile read whatever follows inside the stage and never store
        auto load_v = [&](const float *src, float (&b)[TT]) {
            if constexpr (TT == 8) {
                const float4 lo = *reinterpret_cast<const float4 *>(src), hi = *reinterpret_cast<const float4 *>(src + 4);
                b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w; b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
            } else if constexpr (TT == 4) {
                const float4 t = *reinterpret_cast<const float4 *>(src);
                b[0] = t.x; b[1] = t.y; b[2] = t.z; b[3] = t.w;
            } else if constexpr (TT == 2) {
                const float2 t = *reinterpret_cast<const float2 *>(src);
                b[0] = t.x; b[1] = t.y;
            } else {
                b[0] = *src;
            }
        };
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % ST_STAGES;
            const uint32_t ph = (uint32_t)(kb / ST_STAGES) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_full(s), ph, abort_flag, status));
            if (!ok) break;
            const float *a = reinterpret_cast<const float *>(ring_ptr + (size_t)s * ST_STAGE) + ocl;
            const float *vk = reinterpret_cast<const float *>(ring_ptr + (size_t)s * ST_STAGE + ST_BOX) + j0;
            float4 u = *reinterpret_cast<const float4 *>(a);
            float b[TT];
            load_v(vk, b);
#pragma unroll 8
            for (int kk = 0; kk < 32; ++kk) {
                // the row after the last one of the box is still inside the stage or the slack: read, never used
                const float4 un = *reinterpret_cast<const float4 *>(a + (kk + 1) * 128);
                float bn[TT];
                load_v(vk + (kk + 1) * tp, bn);
                const float uu[4] = {u.x, u.y, u.z, u.w};
                if constexpr (TT >= 2) {
                    uint64_t bp[TP];
#pragma unroll
                    for (int j = 0; j < TP; ++j) bp[j] = pack2(b[2 * j], b[2 * j + 1]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint64_t up = pack2(uu[i], uu[i]);
#pragma unroll
                        for (int j = 0; j < TP; ++j) acc2[i][j] = fma2(up, bp[j], acc2[i][j]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc1[i] = __fmaf_rn(uu[i], b[0], acc1[i]);
                }
                u = un;
#pragma unroll
                for (int j = 0; j < TT; ++j) b[j] = bn[j];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(s));  // this warp no longer reads the stage
        }
        if (ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = oc0 + ocl + i;
                if (row >= oc) continue;
                float *dst = M + ((size_t)p * oc + row) * tp + j0;
                float res[TT];
                if constexpr (TT >= 2) {
#pragma unroll
                    for (int j = 0; j < TP; ++j) unpack2(acc2[i][j], res[2 * j], res[2 * j + 1]);
                } else {
                    res[0] = acc1[i];
                }
#pragma unroll
                for (int j = 0; j < TT; ++j)
                    if (j0 + j < tp) dst[j] = res[j];
            }
        }
    }
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let boxes still in flight land before the CTA goes
    }
}

// The same computation with plain loads (no mbarriers, no status word), for callers that have no
// context: consecutive threads read consecutive output channels of U[p][k][.], one coalesced line per k.
constexpr int SK_THREADS = 128;
constexpr int SK_KC = 256;

template <int TN>
__global__ void __launch_bounds__(SK_THREADS) wino_gemm_ffma_skinny_kernel(const float *__restrict__ U,
                                                                           const float *__restrict__ V,
                                                                           float *__restrict__ M, int oc, int ocp,
                                                                           int tp, int icp) {
    constexpr int TNP = (TN + 3) / 4 * 4;
    __shared__ __align__(16) float Vs[SK_KC * TNP];
    const int tid = threadIdx.x;
    const int p = blockIdx.y;
    const int row = blockIdx.x * SK_THREADS + tid;
    const int row_ld = row < ocp ? row : ocp - 1;
    const float *up = U + (size_t)p * icp * ocp + row_ld;
    const float *Vp = V + (size_t)p * icp * tp;

    float acc[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[j] = 0.0f;
    pdl_trigger();
    pdl_wait();

    for (int k0 = 0; k0 < icp; k0 += SK_KC) {
        const int kc = min(SK_KC, icp - k0);
        __syncthreads();
        for (int idx = tid; idx < kc * (TNP / 4); idx += SK_THREADS) {
            const int k = idx / (TNP / 4), t4 = (idx % (TNP / 4)) * 4;
            *reinterpret_cast<float4 *>(&Vs[k * TNP + t4]) =
                t4 < tp ? __ldg(reinterpret_cast<const float4 *>(Vp + (size_t)(k0 + k) * tp + t4))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncthreads();
        float u_next[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) u_next[q] = q < kc ? __ldg(up + (size_t)(k0 + q) * ocp) : 0.0f;
        for (int k = 0; k < kc; k += 4) {
            float uu[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) uu[q] = u_next[q];
#pragma unroll
            for (int q = 0; q < 4; ++q) u_next[q] = k + 4 + q < kc ? __ldg(up + (size_t)(k0 + k + 4 + q) * ocp) : 0.0f;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                if (k + kk >= kc) break;
                const float4 *b4 = reinterpret_cast<const float4 *>(&Vs[(k + kk) * TNP]);
#pragma unroll
                for (int g = 0; g < TNP / 4; ++g) {
                    const float4 b = b4[g];
                    if (g * 4 + 0 < TN) acc[g * 4 + 0] = __fmaf_rn(uu[kk], b.x, acc[g * 4 + 0]);
                    if (g * 4 + 1 < TN) acc[g * 4 + 1] = __fmaf_rn(uu[kk], b.y, acc[g * 4 + 1]);
                    if (g * 4 + 2 < TN) acc[g * 4 + 2] = __fmaf_rn(uu[kk], b.z, acc[g * 4 + 2]);
                    if (g * 4 + 3 < TN) acc[g * 4 + 3] = __fmaf_rn(uu[kk], b.w, acc[g * 4 + 3]);
                }
            }
        }
    }
    if (row < oc) {
        float *dst = M + ((size_t)p * oc + row) * tp;
#pragma unroll
        for (int j = 0; j < TN; ++j)
            if (j < tp) dst[j] = acc[j];
    }
}

// U[p][icp][ocp] as a 3-D tensor (oc, ic, p), box = 128 oc x 32 ic, no swizzle, zero fill outside
int make_map_u_rowmajor(CUtensorMap *map, const float *base, int ocp, int icp, int box_oc = 128, int box_ic = 32) {
    tc::EncodeTiledFn enc;
    FC_PROPAGATE(tc::get_encoder(&enc));
    cuuint64_t dims[3] = {(cuuint64_t)ocp, (cuuint64_t)icp, 64};
    cuuint64_t strides[2] = {(cuuint64_t)ocp * 4, (cuuint64_t)ocp * icp * 4};
    cuuint32_t box[3] = {(cuuint32_t)box_oc, (cuuint32_t)box_ic, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FC_REQUIRE(r == CUDA_SUCCESS, FC_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (ocp %d icp %d)", (int)r, ocp, icp);
    return FC_OK;
}

// V[p][icp][tp] as a 3-D tensor (tile, ic, p), box = tp tiles x 32 ic, no swizzle, zero fill outside
int make_map_v_rowmajor(CUtensorMap *map, const float *base, int tp, int icp, int box_t = 0, int box_ic = 32) {
    tc::EncodeTiledFn enc;
    FC_PROPAGATE(tc::get_encoder(&enc));
    cuuint64_t dims[3] = {(cuuint64_t)tp, (cuuint64_t)icp, 64};
    cuuint64_t strides[2] = {(cuuint64_t)tp * 4, (cuuint64_t)tp * icp * 4};
    cuuint32_t box[3] = {(cuuint32_t)(box_t ? box_t : tp), (cuuint32_t)box_ic, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FC_REQUIRE(r == CUDA_SUCCESS, FC_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (tp %d icp %d)", (int)r, tp, icp);
    return FC_OK;
}


// ---------------------------------------------------------------------------------------------
// The blocked kernel fed by TMA.  Same block, same thread tile, same inner product as wino_gemm_ffma_kernel; what
// changes is how the slabs arrive and how the warps meet.  One thread asks for a whole BK x BM box of U and a BK x BN
// box of V per slab (cp.async.bulk.tensor, zero fill past the edges), the boxes land in a ring of TB_STAGES stages and
// complete the stage's "full" mbarrier; each warp waits for that barrier by itself, multiplies, and arrives on the
// stage's "empty" barrier.  No thread issues per-slab copy instructions, and no block-wide barrier sits in the loop:
// a warp may run a slab ahead of its neighbours.  The stage refilled while slab kt is multiplied is the one slab kt-2
// used, so the requesting warp waits only for warps that are two slabs behind.
// ---------------------------------------------------------------------------------------------
// FLEX = 0: a thread owns TM channels x TN tiles read as 128-bit rows (BN a multiple of 64).  FLEX = 1: BN = 80, 96 or
// 112 and a thread's TN = BN / 16 tiles are 16 apart, read one float at a time (wino_gemm_ffma_flex_kernel's form).
template <int BM, int BN, int MAP, int BK, int TB_STAGES, int FLEX>
__device__ __forceinline__ void tma_block_body(const CUtensorMap *tmU_p, const CUtensorMap *tmV_p, float *__restrict__ M,
                                               int *status, int oc, int tp, int icp, int oc0, int t0, int p) {
    using namespace tc;
    constexpr int TM = BM / 16, TN = BN / 16, TP2 = TN / 2;
    static_assert(FLEX == 1 || (TM % 4 == 0 && TN % 4 == 0), "block shape");
    constexpr uint32_t A_STAGE = BK * BM * 4, B_STAGE = BK * BN * 4, STAGE = A_STAGE + B_STAGE;
    static_assert(STAGE % 128 == 0, "stages stay 128-byte aligned");
    static_assert(2 * TB_STAGES * 8 + 4 <= 128, "barriers and the abort flag live in the 128 bytes ahead of the ring");
    extern __shared__ uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[TB_STAGES], empty[TB_STAGES]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * TB_STAGES);
    const uint32_t ring = (smem_u32(smem_raw) + 128 + 127) & ~127u;
    const uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    auto bar_full = [&](int s) { return smem_u32(bars + s); };
    auto bar_empty = [&](int s) { return smem_u32(bars + TB_STAGES + s); };

    const int tid = threadIdx.x, lane = tid & 31;
    const int tx = MAP == 0 ? tid % 16 : (tid / 32 % 2) * 8 + tid % 8;
    const int ty = MAP == 0 ? tid / 16 : (tid / 64) * 4 + tid % 32 / 8;
    const int n_slabs = (icp + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < TB_STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), THREADS / 32);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();
    if (tid == 0) {
        // U is constant: its first boxes are requested before the input transform that writes V is known to be complete
        const int head = n_slabs < TB_STAGES - 1 ? n_slabs : TB_STAGES - 1;
        for (int kt = 0; kt < head; ++kt) {
            mbar_expect_tx(bar_full(kt), STAGE);
            tma_load_3d(ring + kt * STAGE, tmU_p, bar_full(kt), oc0, kt * BK, p);
        }
        pdl_wait();
        for (int kt = 0; kt < head; ++kt) tma_load_3d(ring + kt * STAGE + A_STAGE, tmV_p, bar_full(kt), t0, kt * BK, p);
    }

    uint64_t acc2[TM][TP2];
    float acc1[TM];  // FLEX with an odd TN: the last tile of a thread
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        acc1[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < TP2; ++j) acc2[i][j] = 0ull;  // (+0.0f, +0.0f)
    }

    bool ok = true;
    for (int kt = 0; kt < n_slabs; ++kt) {
        const int s = kt % TB_STAGES;
        if (tid == 0 && kt >= 1) {  // request slab kt + TB_STAGES - 2 into the stage slab kt - 2 used
            const int kn = kt + TB_STAGES - 2;
            if (kn < n_slabs) {
                const int sn = kn % TB_STAGES;
                bool free_stage = true;
                if (kt >= 2) free_stage = mbar_wait(bar_empty(sn), (uint32_t)((kt - 2) / TB_STAGES) & 1u, abort_flag, status);
                if (free_stage) {
                    mbar_expect_tx(bar_full(sn), STAGE);
                    tma_load_3d(ring + sn * STAGE, tmU_p, bar_full(sn), oc0, kn * BK, p);
                    tma_load_3d(ring + sn * STAGE + A_STAGE, tmV_p, bar_full(sn), t0, kn * BK, p);
                }
            }
        }
        __syncwarp();
        ok = __all_sync(0xffffffffu, mbar_wait(bar_full(s), (uint32_t)(kt / TB_STAGES) & 1u, abort_flag, status));
        if (!ok) break;
        const float(*As)[BM] = reinterpret_cast<const float(*)[BM]>(ring_ptr + (size_t)s * STAGE);
        const float(*Bs)[BN] = reinterpret_cast<const float(*)[BN]>(ring_ptr + (size_t)s * STAGE + A_STAGE);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int g = 0; g < TM / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&As[k][g * 64 + ty * 4]);
                a[g * 4 + 0] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
            }
            if constexpr (FLEX == 0) {
#pragma unroll
                for (int g = 0; g < TN / 4; ++g) {
                    const float4 v = *reinterpret_cast<const float4 *>(&Bs[k][g * 64 + tx * 4]);
                    b[g * 4 + 0] = v.x; b[g * 4 + 1] = v.y; b[g * 4 + 2] = v.z; b[g * 4 + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx + 16 * j];
            }
            uint64_t bp[TP2];
#pragma unroll
            for (int j = 0; j < TP2; ++j) bp[j] = pack2(b[2 * j], b[2 * j + 1]);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const uint64_t ap = pack2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < TP2; ++j) acc2[i][j] = fma2(ap, bp[j], acc2[i][j]);
                if constexpr (TN % 2 == 1) acc1[i] = __fmaf_rn(a[i], b[TN - 1], acc1[i]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty(s));  // this warp no longer reads the stage
    }
    if (ok) {
        float *Mp = M + (size_t)p * oc * tp;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = oc0 + (i / 4) * 64 + ty * 4 + (i % 4);
            if (r >= oc) continue;
            if constexpr (FLEX == 0) {
#pragma unroll
                for (int g = 0; g < TN / 4; ++g) {
                    const int c = t0 + g * 64 + tx * 4;
                    if (c < tp) {  // tp is a multiple of 8, so a float4 never straddles the end
                        float4 v;
                        unpack2(acc2[i][g * 2 + 0], v.x, v.y);
                        unpack2(acc2[i][g * 2 + 1], v.z, v.w);
                        *reinterpret_cast<float4 *>(Mp + (size_t)r * tp + c) = v;
                    }
                }
            } else {
                float res[TN];
#pragma unroll
                for (int j = 0; j < TP2; ++j) unpack2(acc2[i][j], res[2 * j], res[2 * j + 1]);
                if constexpr (TN % 2 == 1) res[TN - 1] = acc1[i];
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const int c = t0 + tx + 16 * j;
                    if (c < tp) Mp[(size_t)r * tp + c] = res[j];
                }
            }
        }
    }
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let boxes still in flight land before the CTA goes
    }
}

template <int BM, int BN, int MAP, int BK = 16, int TB_STAGES = 5, int FLEX = 0>
__global__ void __launch_bounds__(THREADS, 2)
    wino_gemm_ffma_tma_kernel(const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmV,
                              float *__restrict__ M, int *status, int oc, int tp, int icp) {
    tma_block_body<BM, BN, MAP, BK, TB_STAGES, FLEX>(&tmU, &tmV, M, status, oc, tp, icp, blockIdx.y * BM, blockIdx.x * BN,
                                                     blockIdx.z);
}

// Tile counts that are not a multiple of 128: the first n_main block columns are 128 tiles wide, the last one only as
// wide as the rest needs (32 ... 112 tiles), so that almost nothing but real tiles is multiplied -- 200 tiles (28x28 maps
// of 8 images) are 128 + 80 instead of 2 x 128, 576 (14x14 of 64 images) are 4 x 128 + 64.  One launch, two block shapes:
// the branch is uniform per block.
template <int TAIL_BN, int TAIL_FLEX>
__global__ void __launch_bounds__(THREADS, 2)
    wino_gemm_ffma_tma_mixed_kernel(const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmV,
                                    const __grid_constant__ CUtensorMap tmVtail, float *__restrict__ M, int *status, int oc,
                                    int tp, int icp, int n_main) {
    if ((int)blockIdx.x < n_main)
        tma_block_body<128, 128, 1, 32, 3, 0>(&tmU, &tmV, M, status, oc, tp, icp, blockIdx.y * 128, blockIdx.x * 128,
                                              blockIdx.z);
    else
        tma_block_body<128, TAIL_BN, 0, 32, 3, TAIL_FLEX>(&tmU, &tmVtail, M, status, oc, tp, icp, blockIdx.y * 128,
                                                          n_main * 128, blockIdx.z);
}

// $FASTCONV_FFMA_TMA=0 keeps the blocked kernel on per-thread asynchronous copies (for comparisons).
static bool tma_blocked_enabled() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_FFMA_TMA");
        state = (e && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

// $FASTCONV_FFMA_MIXED=0 keeps every block column 128 tiles wide (for comparisons).
static bool mixed_enabled() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_FFMA_MIXED");
        state = (e && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

template <int BM, int BN, int MAP, int BKT = 16, int NST = 5, int FLEX = 0>
int launch_blocked_tma(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    CUtensorMap tmU, tmV;
    FC_PROPAGATE(make_map_u_rowmajor(&tmU, d_U, g.ocp, g.icp, BM, BKT));
    FC_PROPAGATE(make_map_v_rowmajor(&tmV, d_V, g.tp, g.icp, BN, BKT));
    const size_t smem = 128 + 128 + (size_t)NST * BKT * (BM + BN) * sizeof(float);
    auto kern = wino_gemm_ffma_tma_kernel<BM, BN, MAP, BKT, NST, FLEX>;
    FC_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(g.tp, BN), (unsigned)ceil_div(g.oc, BM), 64), block(THREADS);
    FC_CHECK_CUDA((launch_pdl(kern, grid, block, smem, ctx->stream, tmU, tmV, d_M, ctx->d_status, g.oc, g.tp, g.icp)));
    return FC_OK;
}

template <int TAIL_BN, int TAIL_FLEX>
int launch_blocked_tma_mixed(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    CUtensorMap tmU, tmV, tmVtail;
    FC_PROPAGATE(make_map_u_rowmajor(&tmU, d_U, g.ocp, g.icp, 128, 32));
    FC_PROPAGATE(make_map_v_rowmajor(&tmV, d_V, g.tp, g.icp, 128, 32));
    FC_PROPAGATE(make_map_v_rowmajor(&tmVtail, d_V, g.tp, g.icp, TAIL_BN, 32));
    const size_t smem = 128 + 128 + (size_t)3 * 32 * (128 + 128) * sizeof(float);
    auto kern = wino_gemm_ffma_tma_mixed_kernel<TAIL_BN, TAIL_FLEX>;
    FC_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int n_main = g.tp / 128;
    dim3 grid((unsigned)n_main + 1, (unsigned)ceil_div(g.oc, 128), 64), block(THREADS);
    FC_CHECK_CUDA((launch_pdl(kern, grid, block, smem, ctx->stream, tmU, tmV, tmVtail, d_M, ctx->d_status, g.oc, g.tp, g.icp,
                              n_main)));
    return FC_OK;
}


template <int TN>
int launch_skinny(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    if (ctx->d_status == nullptr) {  // no context behind the call: the plain-load kernel
        dim3 grid((unsigned)ceil_div(g.oc, SK_THREADS), 64), block(SK_THREADS);
        FC_CHECK_CUDA(launch_pdl(wino_gemm_ffma_skinny_kernel<TN>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.ocp,
                                 g.tp, g.icp));
        return FC_OK;
    }
    FC_REQUIRE(g.tp <= 32, FC_ERR_INVALID_ARG, "skinny TensorGEMM needs at most 32 tiles, got %d", g.tp);
    constexpr int TT = TN <= 4 ? 1 : TN <= 8 ? 2 : TN <= 16 ? 4 : 8;  // tiles per lane: a warp covers 4*TT tiles
    CUtensorMap tmU, tmV;
    FC_PROPAGATE(make_map_u_rowmajor(&tmU, d_U, g.ocp, g.icp));
    FC_PROPAGATE(make_map_v_rowmajor(&tmV, d_V, g.tp, g.icp));
    // 256 B of barriers and flag, alignment slack, the ring, and 4.5 KB that the look-ahead reads of the last k-step
    // of the last stage run into (one V row past the box, one U row past that)
    const size_t smem = 128 + 128 + (size_t)ST_STAGES * ST_STAGE + 4608;
    FC_CHECK_CUDA(cudaFuncSetAttribute(wino_gemm_ffma_skinny_tma_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    dim3 grid((unsigned)ceil_div(g.oc, 128), 64), block(ST_THREADS);
    FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_skinny_tma_kernel<TT>, grid, block, smem, ctx->stream, tmU, tmV, d_M,
                              ctx->d_status, g.oc, g.tp, g.icp)));
    return FC_OK;
}

// FASTCONV_FFMA_FLEX=0 in the environment keeps the heuristic on the 64- and 128-wide blocks (for comparisons).
bool flex_enabled() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_FFMA_FLEX");
        state = (e && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

template <int TN>
int launch_flex(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    constexpr int BN = 16 * TN;
    const size_t smem = (size_t)STAGES * BK * (128 + BN) * sizeof(float);
    FC_CHECK_CUDA(cudaFuncSetAttribute(wino_gemm_ffma_flex_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(g.tp, BN), (unsigned)ceil_div(g.oc, 128), 64), block(THREADS);
    FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_flex_kernel<TN>, grid, block, smem, ctx->stream, d_U, d_V, d_M, g.oc, g.ocp,
                              g.tp, g.icp)));
    return FC_OK;
}

template <int BM, int BN, int MAP = 0>
int launch_blocked(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    const size_t smem = (size_t)STAGES * BK * (BM + BN) * sizeof(float);
    auto kern = wino_gemm_ffma_kernel<BM, BN, MAP>;
    FC_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(g.tp, BN), (unsigned)ceil_div(g.oc, BM), 64), block(THREADS);
    FC_CHECK_CUDA((launch_pdl(kern, grid, block, smem, ctx->stream, d_U, d_V, d_M, g.oc, g.ocp, g.tp, g.icp)));
    return FC_OK;
}

}  // namespace

int launch_wino_gemm_ffma(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g,
                          const KernelCfg *cfg) {
    const int force = cfg ? cfg->skinny : 0;
    if (g.tiles <= 32 && force != 2) {  // every real tile in one thread's registers
        const int t = g.tiles;
        if (t <= 4) return launch_skinny<4>(ctx, d_U, d_V, d_M, g);
        if (t <= 8) return launch_skinny<8>(ctx, d_U, d_V, d_M, g);
        if (t <= 9) return launch_skinny<9>(ctx, d_U, d_V, d_M, g);
        if (t <= 12) return launch_skinny<12>(ctx, d_U, d_V, d_M, g);
        if (t <= 16) return launch_skinny<16>(ctx, d_U, d_V, d_M, g);
        if (t <= 20) return launch_skinny<20>(ctx, d_U, d_V, d_M, g);
        if (t <= 25) return launch_skinny<25>(ctx, d_U, d_V, d_M, g);
        if (t <= 28) return launch_skinny<28>(ctx, d_U, d_V, d_M, g);
        return launch_skinny<32>(ctx, d_U, d_V, d_M, g);
    }
    // 64 is the float4-group stride of the thread mapping, so BM and BN are 64 or 128.  Without a tuned
    // configuration: the largest block that still gives every SM about one and a half CTAs (at batch 1 the
    // GEMMs are small and a 128x128 grid would leave the machine half empty), else the one with most CTAs.
    bool wide_m = g.oc > 64, wide_n = g.tp > 64;
    // block widths of 80, 96 and 112 tiles: by name (bn), or where they pad at least a fifth less than 64 / 128 do.
    // Their inner loop is slower per multiplication (scalar operand reads): measured on 8 images, 72 tiles in one
    // 80-wide block 0.074 ms against 0.096 ms in two 64-wide ones, but 200 tiles in two 112-wide blocks 0.188 ms
    // against 0.184 ms in two 128-wide ones.  (Keeping 8 x 8 outputs per thread and dropping thread columns instead --
    // blocks of 128 x 72 ... 120 with 144 ... 240 threads -- measured slower than both: too few warps per SM.)
    int flex = 0;
    if (cfg && (cfg->bn == 80 || cfg->bn == 96 || cfg->bn == 112)) {
        flex = cfg->bn;
    } else if (!(cfg && (cfg->bm || cfg->bn)) && g.oc > 64 && flex_enabled()) {
        auto padded = [&](int bn) { return (double)ceil_div(g.tp, bn) * bn; };
        double best = padded(128) < padded(64) ? padded(128) : padded(64);
        const int widths[3] = {112, 96, 80};
        for (int bn : widths)
            if (padded(bn) * 1.25 < best) { best = padded(bn) * 1.25; flex = bn; }
    }
    if (flex && ctx->d_status != nullptr && tma_blocked_enabled()) {
        if (flex == 80) return launch_blocked_tma<128, 80, 0, 16, 5, 1>(ctx, d_U, d_V, d_M, g);
        if (flex == 96) return launch_blocked_tma<128, 96, 0, 16, 5, 1>(ctx, d_U, d_V, d_M, g);
        if (flex == 112) return launch_blocked_tma<128, 112, 0, 16, 5, 1>(ctx, d_U, d_V, d_M, g);
    }
    if (flex == 80) return launch_flex<5>(ctx, d_U, d_V, d_M, g);
    if (flex == 96) return launch_flex<6>(ctx, d_U, d_V, d_M, g);
    if (flex == 112) return launch_flex<7>(ctx, d_U, d_V, d_M, g);
    if (cfg && (cfg->bm || cfg->bn)) {
        if (cfg->bm) wide_m = cfg->bm == 128;
        if (cfg->bn) wide_n = cfg->bn >= 128;
    } else {
        const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
        const int shapes[4][2] = {{128, 128}, {128, 64}, {64, 128}, {64, 64}};
        size_t best_ctas = 0;
        for (const auto &sh : shapes) {
            if ((sh[0] == 128 && g.oc <= 64) || (sh[1] == 128 && g.tp <= 64)) continue;
            const size_t ctas = ceil_div(g.oc, sh[0]) * ceil_div(g.tp, sh[1]) * 64;
            if (2 * ctas >= 3 * (size_t)sms) {
                wide_m = sh[0] == 128;
                wide_n = sh[1] == 128;
                break;
            }
            if (ctas > best_ctas) {
                best_ctas = ctas;
                wide_m = sh[0] == 128;
                wide_n = sh[1] == 128;
            }
        }
    }
    // at most 64 output channels: a 256-wide block gives a thread 4 channels x 16 tiles, the 64 outputs of the 128 x 128
    // block (measured 7 % faster than 64 x 128 on 64 -> 64 channels at 224 x 224, 64 images), once there are blocks
    // enough for several waves
    const bool named = cfg && cfg->bn;
    // The TMA-fed kernel wherever a context stands behind the call (its waits report into the context's status word); a
    // box may be wider than the tensor, what lies outside reads as zero.  Slabs of 32
    // channels in a ring of 3 measured 1 % faster than 16 x 5 or 16 x 6 on the 128 x 128 block; the 64 x 256 block keeps
    // 16 x 5 so that two CTAs fit an SM.
    const bool tma = ctx->d_status != nullptr && tma_blocked_enabled();
    const bool wide256 = !wide_m && wide_n && (named ? cfg->bn == 256 : ceil_div(g.tp, 256) * ceil_div(g.oc, 64) * 64 >= (size_t)8 * 148);
    if (tma) {
        if (wide_m && wide_n) {
            const int tail = g.tp % 128;  // a multiple of 8
            if (tail == 0 || g.tp < 128 || named || !mixed_enabled()) return launch_blocked_tma<128, 128, 1, 32, 3>(ctx, d_U, d_V, d_M, g);
            if (tail <= 32) return launch_blocked_tma_mixed<32, 1>(ctx, d_U, d_V, d_M, g);
            if (tail <= 48) return launch_blocked_tma_mixed<48, 1>(ctx, d_U, d_V, d_M, g);
            if (tail <= 64) return launch_blocked_tma_mixed<64, 0>(ctx, d_U, d_V, d_M, g);
            if (tail <= 80) return launch_blocked_tma_mixed<80, 1>(ctx, d_U, d_V, d_M, g);
            if (tail <= 96) return launch_blocked_tma_mixed<96, 1>(ctx, d_U, d_V, d_M, g);
            if (tail <= 112) return launch_blocked_tma_mixed<112, 1>(ctx, d_U, d_V, d_M, g);
            return launch_blocked_tma<128, 128, 1, 32, 3>(ctx, d_U, d_V, d_M, g);
        }
        if (wide_m && !wide_n) return launch_blocked_tma<128, 64, 0, 32, 3>(ctx, d_U, d_V, d_M, g);
        if (wide256) return launch_blocked_tma<64, 256, 0, 16, 5>(ctx, d_U, d_V, d_M, g);
        if (!wide_m && wide_n && !wide256) return launch_blocked_tma<64, 128, 0, 32, 3>(ctx, d_U, d_V, d_M, g);
        if (!wide_m && !wide_n) return launch_blocked_tma<64, 64, 0, 32, 3>(ctx, d_U, d_V, d_M, g);
    }
    if (wide_m && wide_n) return launch_blocked<128, 128, 1>(ctx, d_U, d_V, d_M, g);
    if (wide_m) return launch_blocked<128, 64>(ctx, d_U, d_V, d_M, g);
    if (wide256) return launch_blocked<64, 256>(ctx, d_U, d_V, d_M, g);
    if (wide_n) return launch_blocked<64, 128>(ctx, d_U, d_V, d_M, g);
    return launch_blocked<64, 64>(ctx, d_U, d_V, d_M, g);
}

}  // namespace fc
