// im2col path: gather dump + implicit-GEMM convolution on the FP32 pipes ("mirrored" mode).
//
// The reference materialises B[(ic*kh+u)*kw+v][i*ow+j] (ConvIm2colLayer::im2col,
// convLayer/im2colConv.cpp:285-309) and multiplies A[oc][K] * B with packed register kernels whose
// accumulation per output element is one fused multiply-add per k, k ascending
// (im2col/gemm_kernel.cpp:350-420; kc blocks continue through C, convLayer/im2colConv.cpp:465-557).
// Here the matrix is never built: the CTA's operand loader computes the same index map on the fly
// and zero-fills the padding, and each output element keeps one accumulator fed in ascending k.
#include "fc_internal.h"

namespace fc {

namespace {

// ---- gather dump (debug / parity): exactly the reference's index map ---------------------------
__global__ void im2col_gather_kernel(const float *__restrict__ in, float *__restrict__ B, int ic, int ih, int iw,
                                     int kh, int kw, int sh, int sw, int pad_l, int pad_t, int oh, int ow) {
    const size_t total = (size_t)ic * kh * kw * oh * ow;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(idx % ow);
        size_t r = idx / ow;
        const int i = (int)(r % oh);
        r /= oh;
        const int v = (int)(r % kw);
        r /= kw;
        const int u = (int)(r % kh);
        const int c = (int)(r / kh);
        const int row = u - pad_t + i * sh, col = v - pad_l + j * sw;
        B[idx] = (row < 0 || row >= ih || col < 0 || col >= iw) ? 0.0f : in[((size_t)c * ih + row) * iw + col];
    }
}

constexpr int BK = 16;
constexpr int THREADS = 256;

struct IgemmParams {
    int n, ic, ih, iw, oc, kh, kw, sh, sw, pad_l, pad_t, oh, ow;
    int K;        // ic*kh*kw
    int npix;     // n*oh*ow
};

template <int BM, int BN>
__global__ void __launch_bounds__(THREADS) igemm_ffma_kernel(const float *__restrict__ in,
                                                             const float *__restrict__ A, float *__restrict__ out,
                                                             IgemmParams P) {
    constexpr int TM = BM / 16, TN = BN / 16;
    constexpr int LDA = BM + 4, LDB = BN + 4;
    constexpr int A_PER = BM * BK / THREADS;  // scalar A loads per thread per slab
    constexpr int B_PER = BN * BK / THREADS;  // gathered B loads per thread per slab
    constexpr int B_KSTEP = THREADS / BN;     // k rows covered per pass of the loader
    __shared__ __align__(16) float As[2][BK][LDA];
    __shared__ __align__(16) float Bs[2][BK][LDB];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int oc0 = blockIdx.y * BM;
    const int pix0 = blockIdx.x * BN;

    // the pixel this thread gathers for is fixed for the whole K loop
    const int bn = tid % BN, bk0 = tid / BN;
    const int pix = pix0 + bn;
    const bool pix_ok = pix < P.npix;
    int img = 0, oi = 0, oj = 0;
    if (pix_ok) {
        img = pix / (P.oh * P.ow);
        const int rem = pix - img * P.oh * P.ow;
        oi = rem / P.ow;
        oj = rem - oi * P.ow;
    }
    const int base_row = oi * P.sh - P.pad_t, base_col = oj * P.sw - P.pad_l;
    const float *img_ptr = in + (size_t)img * P.ic * P.ih * P.iw;
    const int khw = P.kh * P.kw;

    float a_stage[A_PER], b_stage[B_PER];

    auto load_slab = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_PER; ++i) {
            const int idx = tid + i * THREADS;
            const int row = idx / BK, kk = idx % BK;
            const int r = oc0 + row, k = k0 + kk;
            a_stage[i] = (r < P.oc && k < P.K) ? __ldg(A + (size_t)r * P.K + k) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < B_PER; ++i) {
            const int k = k0 + bk0 + i * B_KSTEP;
            float val = 0.0f;
            if (pix_ok && k < P.K) {
                const int c = k / khw;
                const int r2 = k - c * khw;
                const int u = r2 / P.kw;
                const int v = r2 - u * P.kw;
                const int row = base_row + u, col = base_col + v;
                if (row >= 0 && row < P.ih && col >= 0 && col < P.iw)
                    val = __ldg(img_ptr + ((size_t)c * P.ih + row) * P.iw + col);
            }
            b_stage[i] = val;
        }
    };
    auto store_slab = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; ++i) {
            const int idx = tid + i * THREADS;
            As[buf][idx % BK][idx / BK] = a_stage[i];
        }
#pragma unroll
        for (int i = 0; i < B_PER; ++i) Bs[buf][bk0 + i * B_KSTEP][bn] = b_stage[i];
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    load_slab(0);
    store_slab(0);
    __syncthreads();

    const int n_slabs = (P.K + BK - 1) / BK;
    for (int s = 0; s < n_slabs; ++s) {
        const int buf = s & 1;
        if (s + 1 < n_slabs) load_slab((s + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
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
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < n_slabs) {
            store_slab(buf ^ 1);
            __syncthreads();
        }
    }

    const int ohw = P.oh * P.ow;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = oc0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= P.oc) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int px = pix0 + (j / 4) * 64 + tx * 4 + (j % 4);
            if (px >= P.npix) continue;
            const int im = px / ohw;
            out[((size_t)im * P.oc + r) * ohw + (px - im * ohw)] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Small problems (batch-1 ResNet layers: 49..3136 pixels, a few hundred channels).  The blocked kernel
// above would launch a handful of CTAs, each walking the whole reduction alone.  Here a thread owns one
// output pixel and TM output channels: consecutive threads read consecutive pixels of the input
// (coalesced, stride sw), the k -> (c,u,v) decode is uniform per step and kept in counters, the
// weights of the TM channels are staged in shared memory a chunk at a time and read as broadcasts.
// The chain per output element is the same: one accumulator, one FMA per k, ascending.
// ---------------------------------------------------------------------------------------------
constexpr int DR_THREADS = 128;
constexpr int DR_KC = 256;
constexpr int DR_BATCH = 8;  // input values fetched ahead of the FMAs that consume them

template <int TM, int PXB>
__global__ void __launch_bounds__(DR_THREADS) igemm_ffma_direct_kernel(const float *__restrict__ in,
                                                                       const float *__restrict__ A,
                                                                       float *__restrict__ out, IgemmParams P) {
    constexpr int GROUPS = DR_THREADS / PXB;  // channel groups per block
    constexpr int OCB = TM * GROUPS;          // output channels per block
    __shared__ __align__(16) float As[DR_KC][OCB];
    const int tid = threadIdx.x;
    const int px_l = tid % PXB, grp = tid / PXB;
    const int pix = blockIdx.x * PXB + px_l;
    const int ocb0 = blockIdx.y * OCB, oc0 = ocb0 + grp * TM;
    const int ohw = P.oh * P.ow;
    const bool pix_ok = pix < P.npix;
    int img = 0, oi = 0, oj = 0;
    if (pix_ok) {
        img = pix / ohw;
        const int rem = pix - img * ohw;
        oi = rem / P.ow;
        oj = rem - oi * P.ow;
    }
    const int base_row = oi * P.sh - P.pad_t, base_col = oj * P.sw - P.pad_l;
    const float *pix_ptr = in + (size_t)img * P.ic * P.ih * P.iw + (ptrdiff_t)base_row * P.iw + base_col;

    float acc[TM];
#pragma unroll
    for (int i = 0; i < TM; ++i) acc[i] = 0.0f;

    int c = 0, u = 0, v = 0;  // decode of the running k, the same in every thread
    for (int k0 = 0; k0 < P.K; k0 += DR_KC) {
        const int kc = min(DR_KC, P.K - k0);
        __syncthreads();
        for (int idx = tid; idx < DR_KC * OCB; idx += DR_THREADS) {
            const int j = idx / DR_KC, kk = idx - j * DR_KC;  // consecutive threads walk k: coalesced rows of A
            As[kk][j] = (ocb0 + j < P.oc && kk < kc) ? __ldg(A + (size_t)(ocb0 + j) * P.K + k0 + kk) : 0.0f;
        }
        __syncthreads();
        for (int kk = 0; kk < kc; kk += DR_BATCH) {
            float val[DR_BATCH];
#pragma unroll
            for (int j = 0; j < DR_BATCH; ++j) {  // all loads of the batch first, so they overlap
                val[j] = 0.0f;
                if (kk + j < kc) {
                    const int row = base_row + u, col = base_col + v;
                    if (pix_ok && (unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw)
                        val[j] = __ldg(pix_ptr + (c * P.ih + u) * P.iw + v);
                    if (++v == P.kw) {
                        v = 0;
                        if (++u == P.kh) {
                            u = 0;
                            ++c;
                        }
                    }
                }
            }
            // rows of As past kc are zero, so a short last batch adds exact zeros
#pragma unroll
            for (int j = 0; j < DR_BATCH; ++j)
#pragma unroll
                for (int i = 0; i < TM; ++i) acc[i] = __fmaf_rn(As[kk + j][grp * TM + i], val[j], acc[i]);
        }
    }
    if (pix_ok) {
        float *dst = out + ((size_t)img * P.oc + oc0) * ohw + (pix - img * ohw);
#pragma unroll
        for (int i = 0; i < TM; ++i)
            if (oc0 + i < P.oc) dst[(size_t)i * ohw] = acc[i];
    }
}

template <int TM, int PXB>
int launch_direct(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const IgemmParams &P) {
    constexpr int OCB = TM * (DR_THREADS / PXB);
    dim3 grid((unsigned)ceil_div(P.npix, PXB), (unsigned)ceil_div(P.oc, OCB)), block(DR_THREADS);
    igemm_ffma_direct_kernel<TM, PXB><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace

int launch_im2col_gather(fc_context *ctx, const float *d_in, float *d_B, const fc_conv_desc &d, int oh, int ow,
                         int image) {
    const size_t total = (size_t)d.ic * d.kh * d.kw * oh * ow;
    const unsigned blocks = (unsigned)(ceil_div(total, 256) > 148 * 32 ? 148 * 32 : ceil_div(total, 256));
    const float *src = d_in + (size_t)image * d.ic * d.ih * d.iw;
    im2col_gather_kernel<<<blocks, 256, 0, ctx->stream>>>(src, d_B, d.ic, d.ih, d.iw, d.kh, d.kw, d.sh, d.sw,
                                                          d.pad_left, d.pad_top, oh, ow);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

int launch_igemm_ffma(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const fc_conv_desc &d,
                      int oh, int ow, const KernelCfg *cfg) {
    IgemmParams P;
    P.n = d.batch; P.ic = d.ic; P.ih = d.ih; P.iw = d.iw; P.oc = d.oc; P.kh = d.kh; P.kw = d.kw;
    P.sh = d.sh; P.sw = d.sw; P.pad_l = d.pad_left; P.pad_t = d.pad_top; P.oh = oh; P.ow = ow;
    P.K = d.ic * d.kh * d.kw;
    P.npix = d.batch * oh * ow;
    const bool wide_m = cfg && cfg->bm ? cfg->bm == 128 : d.oc > 64;
    const bool wide_n = cfg && cfg->bn ? cfg->bn == 128 : P.npix > 64;
    // skinny = 1 forces the thread-per-pixel kernel, 2 the blocked one; otherwise the blocked kernel only when
    // its grid gives the machine about one and a half CTAs per SM
    const size_t blocked_ctas = ceil_div(P.npix, wide_n ? 128 : 64) * ceil_div(d.oc, wide_m ? 128 : 64);
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int pick = cfg ? cfg->skinny : 0;
    if (pick == 1 || (pick == 0 && 2 * blocked_ctas < 3 * (size_t)sms)) {
        // few output elements: fewer channels per thread, so more threads share the (latency-bound) chains
        const bool thin = (size_t)P.npix * d.oc < (size_t)sms * 2048;
        if (P.npix >= 96) return thin ? launch_direct<4, 128>(ctx, d_in, d_kernel, d_out, P)
                                      : launch_direct<8, 128>(ctx, d_in, d_kernel, d_out, P);
        if (P.npix >= 48) return thin ? launch_direct<4, 64>(ctx, d_in, d_kernel, d_out, P)
                                      : launch_direct<8, 64>(ctx, d_in, d_kernel, d_out, P);
        return thin ? launch_direct<4, 32>(ctx, d_in, d_kernel, d_out, P) : launch_direct<8, 32>(ctx, d_in, d_kernel, d_out, P);
    }
    dim3 grid((unsigned)ceil_div(P.npix, wide_n ? 128 : 64), (unsigned)ceil_div(d.oc, wide_m ? 128 : 64)), block(THREADS);
    if (wide_m && wide_n)
        igemm_ffma_kernel<128, 128><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P);
    else if (wide_m)
        igemm_ffma_kernel<128, 64><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P);
    else if (wide_n)
        igemm_ffma_kernel<64, 128><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P);
    else
        igemm_ffma_kernel<64, 64><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
