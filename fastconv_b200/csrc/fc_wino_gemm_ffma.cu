// TensorGEMM, fp32 "mirrored" mode: 64 independent GEMMs
//     M_p[oc][tile] = sum_ic U_p[oc][ic] * V_p[tile][ic]
// on the FP32 pipes, with the reference's accumulation chain kept exactly: every output element
// owns ONE accumulator that starts at 0 and takes one fused multiply-add per input channel, in
// ascending channel order (TensorGEMMInnerKernel4x4x5_v1, winoF63ZC/TensorGEMMZC.cpp:585-697;
// ic blocks of the reference continue the same chain through gemmBuf).  No split-K, no pairwise
// sums, no reordering -- that is what makes the layer bit-identical to the reference.
//
// Both operands are K-major in global memory (ic contiguous).  A CTA stages a BM x BK slab of U
// and a BN x BK slab of V into shared memory transposed ([k][row], padded) so that the inner
// product reads 128-bit rows without bank conflicts; global loads of the next slab are issued
// before the math of the current one (register-staged double buffering).
#include "fc_tc_common.cuh"

namespace fc {

namespace {

constexpr int BK = 16;
constexpr int THREADS = 256;

template <int BM, int BN>
struct FfmaCfg {
    static constexpr int TM = BM / 16;  // rows (oc) per thread
    static constexpr int TN = BN / 16;  // columns (tiles) per thread
    static constexpr int LDA = BM + 4;
    static constexpr int LDB = BN + 4;
    static constexpr int A_F4 = BM * BK / 4 / THREADS;  // float4 loads per thread per slab
    static constexpr int B_F4 = BN * BK / 4 / THREADS;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "thread tile must be float4-granular");
    static_assert(A_F4 >= 1 && B_F4 >= 1, "slab too small for the thread count");
};

template <int BM, int BN>
__global__ void __launch_bounds__(THREADS, 2) wino_gemm_ffma_kernel(const float *__restrict__ U,
                                                                 const float *__restrict__ V, float *__restrict__ M,
                                                                 int oc, int tp, int icp) {
    using C = FfmaCfg<BM, BN>;
    __shared__ __align__(16) float As[2][BK][C::LDA];
    __shared__ __align__(16) float Bs[2][BK][C::LDB];

    const int p = blockIdx.z;
    const int oc0 = blockIdx.y * BM;
    const int t0 = blockIdx.x * BN;
    const float *Up = U + (size_t)p * oc * icp;
    const float *Vp = V + (size_t)p * tp * icp;
    float *Mp = M + (size_t)p * oc * tp;

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;

    float4 a_stage[C::A_F4], b_stage[C::B_F4];

    auto load_slab = [&](int k0) {
#pragma unroll
        for (int i = 0; i < C::A_F4; ++i) {
            const int idx = tid + i * THREADS;
            const int row = idx / (BK / 4), kq = idx % (BK / 4);
            const int r = oc0 + row, k = k0 + kq * 4;
            a_stage[i] = (r < oc && k < icp) ? __ldg(reinterpret_cast<const float4 *>(Up + (size_t)r * icp + k))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < C::B_F4; ++i) {
            const int idx = tid + i * THREADS;
            const int row = idx / (BK / 4), kq = idx % (BK / 4);
            const int r = t0 + row, k = k0 + kq * 4;
            b_stage[i] = (r < tp && k < icp) ? __ldg(reinterpret_cast<const float4 *>(Vp + (size_t)r * icp + k))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto store_slab = [&](int buf) {
#pragma unroll
        for (int i = 0; i < C::A_F4; ++i) {
            const int idx = tid + i * THREADS;
            const int row = idx / (BK / 4), kq = idx % (BK / 4);
            As[buf][kq * 4 + 0][row] = a_stage[i].x;
            As[buf][kq * 4 + 1][row] = a_stage[i].y;
            As[buf][kq * 4 + 2][row] = a_stage[i].z;
            As[buf][kq * 4 + 3][row] = a_stage[i].w;
        }
#pragma unroll
        for (int i = 0; i < C::B_F4; ++i) {
            const int idx = tid + i * THREADS;
            const int row = idx / (BK / 4), kq = idx % (BK / 4);
            Bs[buf][kq * 4 + 0][row] = b_stage[i].x;
            Bs[buf][kq * 4 + 1][row] = b_stage[i].y;
            Bs[buf][kq * 4 + 2][row] = b_stage[i].z;
            Bs[buf][kq * 4 + 3][row] = b_stage[i].w;
        }
    };

    float acc[C::TM][C::TN];
#pragma unroll
    for (int i = 0; i < C::TM; ++i)
#pragma unroll
        for (int j = 0; j < C::TN; ++j) acc[i][j] = 0.0f;

    pdl_trigger();
    pdl_wait();

    load_slab(0);
    store_slab(0);
    __syncthreads();

    const int n_slabs = (icp + BK - 1) / BK;
    for (int s = 0; s < n_slabs; ++s) {
        const int buf = s & 1;
        if (s + 1 < n_slabs) load_slab((s + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[C::TM], b[C::TN];
            // rows are split in float4 groups strided by 64 (16 threads x 4) so a warp's 128-bit
            // reads of one k-row touch consecutive banks
#pragma unroll
            for (int g = 0; g < C::TM / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&As[buf][k][g * 64 + ty * 4]);
                a[g * 4 + 0] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < C::TN / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4 *>(&Bs[buf][k][g * 64 + tx * 4]);
                b[g * 4 + 0] = v.x; b[g * 4 + 1] = v.y; b[g * 4 + 2] = v.z; b[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < C::TM; ++i)
#pragma unroll
                for (int j = 0; j < C::TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < n_slabs) {
            store_slab(buf ^ 1);
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < C::TM; ++i) {
        const int r = oc0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= oc) continue;
#pragma unroll
        for (int g = 0; g < C::TN / 4; ++g) {
            const int c = t0 + g * 64 + tx * 4;
            if (c < tp)  // tp is a multiple of 8, so a float4 never straddles the end
                *reinterpret_cast<float4 *>(Mp + (size_t)r * tp + c) =
                    make_float4(acc[i][g * 4 + 0], acc[i][g * 4 + 1], acc[i][g * 4 + 2], acc[i][g * 4 + 3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Few tiles (small feature maps at batch 1: 28x28 -> 25 tiles, 14x14 -> 9, 7x7 -> 4).  The GEMM is a
// stream over U with a short N, so the blocked kernel above would multiply mostly padding.  Here a
// thread owns ONE output channel and ALL TN tiles of a position: its row of U goes straight from
// global memory to registers (each element is used by exactly this thread), V_p is staged transposed
// in shared memory a K-chunk at a time and read as broadcasts, and the TN accumulators take one FMA
// per input channel in ascending order -- the same chain as the blocked kernel and the reference.
// ---------------------------------------------------------------------------------------------
constexpr int SK_THREADS = 128;
constexpr int SK_KC = 256;  // input channels staged per chunk

template <int TN>
__global__ void __launch_bounds__(SK_THREADS) wino_gemm_ffma_skinny_kernel(const float *__restrict__ U,
                                                                           const float *__restrict__ V,
                                                                           float *__restrict__ M, int oc, int tp,
                                                                           int icp) {
    constexpr int TNP = (TN + 3) / 4 * 4;
    __shared__ __align__(16) float Vs[SK_KC * TNP];
    const int tid = threadIdx.x;
    const int p = blockIdx.y;
    const int row = blockIdx.x * SK_THREADS + tid;
    const int row_ld = row < oc ? row : oc - 1;
    const float *up = U + ((size_t)p * oc + row_ld) * icp;
    const float *Vp = V + (size_t)p * tp * icp;

    float acc[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[j] = 0.0f;

    pdl_trigger();
    pdl_wait();

    for (int k0 = 0; k0 < icp; k0 += SK_KC) {
        const int kc = min(SK_KC, icp - k0);  // multiple of 8
        __syncthreads();
        // stage V_p[t][k0..k0+kc) as Vs[k][t]; consecutive threads take consecutive tiles
        for (int idx = tid; idx < TNP * (kc / 4); idx += SK_THREADS) {
            const int t = idx % TNP, k4 = idx / TNP;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < tp) v = __ldg(reinterpret_cast<const float4 *>(Vp + (size_t)t * icp + k0 + k4 * 4));
            Vs[(k4 * 4 + 0) * TNP + t] = v.x;
            Vs[(k4 * 4 + 1) * TNP + t] = v.y;
            Vs[(k4 * 4 + 2) * TNP + t] = v.z;
            Vs[(k4 * 4 + 3) * TNP + t] = v.w;
        }
        __syncthreads();
        float4 u_next = __ldg(reinterpret_cast<const float4 *>(up + k0));
        for (int k = 0; k < kc; k += 4) {
            const float4 u = u_next;
            if (k + 4 < kc) u_next = __ldg(reinterpret_cast<const float4 *>(up + k0 + k + 4));
            const float uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
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

// Same computation with U streamed by TMA: a producer warp keeps a ring of 128(oc) x 32(ic) boxes of U in
// flight (128-byte swizzle), so HBM latency is hidden by the ring instead of by each thread's own
// loads; the 128 consumer threads read their row of the landed box (conflict-free through the swizzle),
// V_p is staged transposed a 256-channel chunk at a time.  The chain per output element is unchanged:
// one accumulator, one FMA per input channel, ascending.
constexpr int ST_STAGES = 5;
constexpr int ST_KC = 256;
constexpr int ST_THREADS = 160;  // 4 consumer warps + 1 producer warp
constexpr int ST_BOX = 128 * 32 * 4;

template <int TN>
__global__ void __launch_bounds__(ST_THREADS) wino_gemm_ffma_skinny_tma_kernel(const __grid_constant__ CUtensorMap tmU,
                                                                               const float *__restrict__ V,
                                                                               float *__restrict__ M, int *status,
                                                                               int oc, int tp, int icp) {
    using namespace tc;
    constexpr int TNP = (TN + 3) / 4 * 4;
    extern __shared__ uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[ST_STAGES], empty[ST_STAGES]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * ST_STAGES);
    const uint32_t ring = (smem_u32(smem_raw) + 128 + 1023) & ~1023u;
    const uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    float *Vs = reinterpret_cast<float *>(smem_raw + (ring - smem_u32(smem_raw)) + ST_STAGES * ST_BOX);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = blockIdx.y, oc0 = blockIdx.x * 128;
    const int num_kb = (icp + 31) / 32;
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
        if (lane == 0) {  // U is constant: no need to wait for the input transform
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % ST_STAGES;
                const uint32_t ph = (uint32_t)(kb / ST_STAGES) & 1u;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, status)) break;
                mbar_expect_tx(bar_full(s), ST_BOX);
                tma_load_3d(ring + s * ST_BOX, &tmU, bar_full(s), kb * 32, oc0, p);
            }
        }
    } else {
        pdl_wait();  // V comes from the input transform launched just before
        const int row = oc0 + tid;
        const float *Vp = V + (size_t)p * tp * icp;
        float acc[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[j] = 0.0f;
        // `ok` turns false when a bounded wait gives up; the warp then skips the math but still walks the
        // loop so that all four consumer warps meet at every chunk barrier
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
            if (kb % (ST_KC / 32) == 0) {
                const int k0 = kb * 32;
                asm volatile("bar.sync 1, 128;" ::: "memory");  // consumers only: everyone is done with the old chunk
                for (int idx = tid; idx < TNP * (ST_KC / 4); idx += 128) {
                    const int t = idx % TNP, k4 = idx / TNP;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (t < tp && k0 + k4 * 4 < icp) v = __ldg(reinterpret_cast<const float4 *>(Vp + (size_t)t * icp + k0 + k4 * 4));
                    Vs[(k4 * 4 + 0) * TNP + t] = v.x;
                    Vs[(k4 * 4 + 1) * TNP + t] = v.y;
                    Vs[(k4 * 4 + 2) * TNP + t] = v.z;
                    Vs[(k4 * 4 + 3) * TNP + t] = v.w;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            const int s = kb % ST_STAGES;
            const uint32_t ph = (uint32_t)(kb / ST_STAGES) & 1u;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_full(s), ph, abort_flag, status));
            if (!ok) continue;
            const uint8_t *a = ring_ptr + s * ST_BOX + tid * 128;  // this thread's oc row: 32 floats, swizzled
            const float *vk = Vs + (size_t)(kb % (ST_KC / 32)) * 32 * TNP;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 u = *reinterpret_cast<const float4 *>(a + ((c ^ (tid & 7)) << 4));
                const float uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const float4 *b4 = reinterpret_cast<const float4 *>(vk + (c * 4 + kk) * TNP);
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
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(s));  // this warp no longer reads the stage
        }
        if (ok && row < oc) {
            float *dst = M + ((size_t)p * oc + row) * tp;
#pragma unroll
            for (int j = 0; j < TN; ++j) dst[j] = acc[j];
        }
    }
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let boxes still in flight land before the CTA goes
    }
}

bool skinny_uses_tma() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_SKINNY");
        state = (e && e[0] == 'l') ? 0 : 1;  // FASTCONV_SKINNY=ldg keeps the per-thread global loads
    }
    return state == 1;
}

template <int TN>
int launch_skinny_tma(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    constexpr int TNP = (TN + 3) / 4 * 4;
    CUtensorMap tmU;
    FC_PROPAGATE(tc::make_map_3d(&tmU, d_U, g.icp, g.oc, 64, 128));
    const size_t smem = 128 + 1024 + (size_t)ST_STAGES * ST_BOX + (size_t)ST_KC * TNP * sizeof(float);
    FC_CHECK_CUDA(cudaFuncSetAttribute(wino_gemm_ffma_skinny_tma_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    dim3 grid((unsigned)ceil_div(g.oc, 128), 64), block(ST_THREADS);
    FC_CHECK_CUDA(launch_pdl(wino_gemm_ffma_skinny_tma_kernel<TN>, grid, block, smem, ctx->stream, tmU, d_V, d_M,
                             ctx->d_status, g.oc, g.tp, g.icp));
    return FC_OK;
}

template <int TN>
int launch_skinny(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    if (skinny_uses_tma() && ctx->d_status != nullptr) return launch_skinny_tma<TN>(ctx, d_U, d_V, d_M, g);
    dim3 grid((unsigned)ceil_div(g.oc, SK_THREADS), 64), block(SK_THREADS);
    FC_CHECK_CUDA(launch_pdl(wino_gemm_ffma_skinny_kernel<TN>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.tp, g.icp));
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
    // 64 is the float4-group stride of the thread mapping, so BM and BN are 64 or 128.
    const bool wide_n = cfg && cfg->bn ? cfg->bn == 128 : g.tp > 64;
    const bool wide_m = cfg && cfg->bm ? cfg->bm == 128 : g.oc > 64;
    const unsigned gx_n = (unsigned)ceil_div(g.tp, wide_n ? 128 : 64);
    const unsigned gy_m = (unsigned)ceil_div(g.oc, wide_m ? 128 : 64);
    dim3 grid(gx_n, gy_m, 64), block(THREADS);
    if (wide_m && wide_n)
        FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_kernel<128, 128>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.tp, g.icp)));
    else if (wide_m)
        FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_kernel<128, 64>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.tp, g.icp)));
    else if (wide_n)
        FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_kernel<64, 128>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.tp, g.icp)));
    else
        FC_CHECK_CUDA((launch_pdl(wino_gemm_ffma_kernel<64, 64>, grid, block, 0, ctx->stream, d_U, d_V, d_M, g.oc, g.tp, g.icp)));
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
