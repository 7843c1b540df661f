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
#include "fc_internal.h"

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
__global__ void __launch_bounds__(THREADS) wino_gemm_ffma_kernel(const float *__restrict__ U,
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

}  // namespace

int launch_wino_gemm_ffma(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g) {
    // 64 is the float4-group stride of the thread mapping, so BM and BN are 64 or 128.
    const bool wide_n = g.tp > 64;
    const bool wide_m = g.oc > 64;
    const unsigned gx_n = (unsigned)ceil_div(g.tp, wide_n ? 128 : 64);
    const unsigned gy_m = (unsigned)ceil_div(g.oc, wide_m ? 128 : 64);
    dim3 grid(gx_n, gy_m, 64), block(THREADS);
    if (wide_m && wide_n)
        wino_gemm_ffma_kernel<128, 128><<<grid, block, 0, ctx->stream>>>(d_U, d_V, d_M, g.oc, g.tp, g.icp);
    else if (wide_m)
        wino_gemm_ffma_kernel<128, 64><<<grid, block, 0, ctx->stream>>>(d_U, d_V, d_M, g.oc, g.tp, g.icp);
    else if (wide_n)
        wino_gemm_ffma_kernel<64, 128><<<grid, block, 0, ctx->stream>>>(d_U, d_V, d_M, g.oc, g.tp, g.icp);
    else
        wino_gemm_ffma_kernel<64, 64><<<grid, block, 0, ctx->stream>>>(d_U, d_V, d_M, g.oc, g.tp, g.icp);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
