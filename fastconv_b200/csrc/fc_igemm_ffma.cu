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

// Packed fp32 arithmetic of sm_100: one instruction, two independent IEEE fused multiply-adds (the halves of 64-bit
// register pairs), each rounded exactly like a scalar fma.rn: same chains, half the issue slots.
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

constexpr int BK = 16;
constexpr int THREADS = 256;

struct IgemmParams {
    int n, ic, ih, iw, oc, kh, kw, sh, sw, pad_l, pad_t, oh, ow;
    int K;        // ic*kh*kw
    int npix;     // n*oh*ow
    // elements from one image to the next in the input and in the output: ic*ih*iw and oc*oh*ow, or those of the
    // whole tensors when the launch computes one group of a grouped convolution
    long long in_img_stride, out_img_stride;
};

template <int BM, int BN>
__global__ void __launch_bounds__(THREADS) igemm_ffma_kernel(const float *__restrict__ in,
                                                             const float *__restrict__ A, float *__restrict__ out,
                                                             IgemmParams P, Epilogue ep) {
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
    const float *img_ptr = in + (size_t)img * P.in_img_stride;
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

    uint64_t acc2[TM][TN / 2];  // pairs of neighbouring pixels, one packed FMA per pair
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc2[i][j] = 0ull;

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
            float lo, hi;
            unpack2(acc2[i][j / 2], lo, hi);
            out[(size_t)im * P.out_img_stride + (size_t)r * ohw + (px - im * ohw)] = ep(j % 2 ? hi : lo, r);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Small and medium problems (batch-1 ResNet layers: 49..3136 pixels, up to 4608-long reductions).  The
// 16 x 16-thread kernel above launches a handful of CTAs for them and decodes k -> (c,u,v) with two integer
// divisions per gathered element.  This kernel takes the decode from a per-layer table (one int2 per k:
// element offset inside the image and (u,v)), brings both operands to shared memory with asynchronous
// copies through a ring of 3 to 8 stages (weights as 16-byte pieces along k, gathered input as 4-byte pieces with
// zero fill for the padding), and comes in block shapes from 128x128 down to 8x32 so that even a 49-pixel
// layer spreads over the machine.  Lanes run along output channels, so a thread reads four k-steps of
// its weight rows in one conflict-free 128-bit read and its pixels as a broadcast.  The chain per output
// element is unchanged: one accumulator, one FMA per k, ascending.
// ---------------------------------------------------------------------------------------------
constexpr int TK_KC = 32, TK_KCP = 36;

__device__ __forceinline__ void cp_async_zfill_16(void *smem_dst, const void *gmem_src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_zfill_4(void *smem_dst, const void *gmem_src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}

// The second launch bound is there for the register allocator: without it ptxas squeezes the small shapes into 32
// registers and every shared-memory read is consumed right after it is issued, its latency exposed on a chain that
// is already sequential in k.
// TK_STAGES: depth of the ring.  Small blocks do little math per stage, so they need a deeper ring to keep the
// two dependent global accesses of the gather (decode table, then the element) off the critical path.
template <int BM, int BN, int TM, int TN, int TK_STAGES>
__global__ void __launch_bounds__((BM / TM) * (BN / TN), TK_STAGES * (BM * 36 + 32 * (BN + 4)) * 4 > 113 * 1024 ? 1 : 2)
    igemm_ffma_tile_kernel(const float *__restrict__ in, const float *__restrict__ A, float *__restrict__ out,
                           const int2 *__restrict__ ktab, IgemmParams P, int a_vec, Epilogue ep,
                           const float *__restrict__ bmat, int ld) {
    constexpr int OCL = BM / TM, NT = OCL * (BN / TN), BNP = BN + 4;
    constexpr int B_STEP = NT / BN, B_ITERS = TK_KC / B_STEP;
    static_assert(NT % BN == 0 && TK_KC % B_STEP == 0 && (TN == 1 || TN == 2 || TN == 4 || TN == 8), "block shape");
    // a thread of a large block gathers many elements per slab; holding their decode entries one slab ahead would
    // cost two registers each, and such a block has the math to cover the table read instead
    constexpr bool DEC_AHEAD = B_ITERS <= 8;
    extern __shared__ __align__(16) float tk_smem[];
    float(*As)[BM][TK_KCP] = reinterpret_cast<float(*)[BM][TK_KCP]>(tk_smem);
    float(*Bs)[TK_KC][BNP] = reinterpret_cast<float(*)[TK_KC][BNP]>(tk_smem + TK_STAGES * BM * TK_KCP);

    const int tid = threadIdx.x;
    const int oc0 = blockIdx.y * BM, pix0 = blockIdx.x * BN;
    const int ohw = P.oh * P.ow;

    // the pixel this thread gathers for is fixed for the whole reduction
    const int lp = tid % BN, lk0 = tid / BN;
    const int gpix = pix0 + lp;
    const bool gpix_ok = gpix < P.npix;
    int base_row = 0, base_col = 0;
    const float *pix_ptr = in;
    if (gpix_ok) {
        const int img = gpix / ohw, rem = gpix - img * ohw;
        const int oi = rem / P.ow, oj = rem - oi * P.ow;
        base_row = oi * P.sh - P.pad_t;
        base_col = oj * P.sw - P.pad_l;
        pix_ptr = in + (size_t)img * P.in_img_stride + (ptrdiff_t)base_row * P.iw + base_col;
    }

    // The decode entries of the NEXT slab are fetched while the copies of this one are issued, so the table read
    // (a global load) is never waited for on the way to the copy that depends on it.
    const int k_padded = ((P.K + TK_KC - 1) / TK_KC) * TK_KC;  // entries in the table
    int2 dec[DEC_AHEAD ? B_ITERS : 1];
    auto fetch_decode = [&](int k0) {
        if (!DEC_AHEAD || bmat != nullptr) return;  // (the gathered matrix was materialised: no decode needed)
#pragma unroll
        for (int r = 0; r < B_ITERS; ++r) {
            const int k = k0 + lk0 + r * B_STEP;
            dec[r] = k < k_padded ? __ldg(ktab + k) : make_int2(0, 0x4000 << 16);
        }
    };
    fetch_decode(0);

    auto load_stage = [&](int st, int k0) {  // called with k0 = 0, 32, 64, ... in this order
        if (a_vec) {  // rows of A are 16-byte aligned: K is a multiple of 4
            for (int idx = tid; idx < BM * (TK_KC / 4); idx += NT) {
                const int row = idx / (TK_KC / 4), c4 = (idx % (TK_KC / 4)) * 4;
                const bool ok = oc0 + row < P.oc && k0 + c4 < P.K;
                cp_async_zfill_16(&As[st][row][c4], A + (ok ? (size_t)(oc0 + row) * P.K + k0 + c4 : 0), ok);
            }
        } else {
            for (int idx = tid; idx < BM * TK_KC; idx += NT) {
                const int row = idx / TK_KC, kk = idx % TK_KC;
                const bool ok = oc0 + row < P.oc && k0 + kk < P.K;
                cp_async_zfill_4(&As[st][row][kk], A + (ok ? (size_t)(oc0 + row) * P.K + k0 + kk : 0), ok);
            }
        }
        if (bmat != nullptr) {  // rows of the materialised matrix: 16-byte pieces, no index arithmetic per element
            for (int idx = tid; idx < TK_KC * (BN / 4); idx += NT) {
                const int kk = idx / (BN / 4), c4 = (idx % (BN / 4)) * 4;
                const bool ok = k0 + kk < P.K;
                cp_async_zfill_16(&Bs[st][kk][c4], bmat + (ok ? (size_t)(k0 + kk) * ld + pix0 + c4 : 0), ok);
            }
            return;
        }
#pragma unroll
        for (int r = 0; r < B_ITERS; ++r) {
            const int kk = lk0 + r * B_STEP;
            // the table is padded to a multiple of 32 with out-of-image entries
            const int2 e = DEC_AHEAD ? dec[DEC_AHEAD ? r : 0] : __ldg(ktab + k0 + kk);
            const int row = base_row + (e.y >> 16), col = base_col + (e.y & 0xffff);
            const bool ok = gpix_ok && (unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw;
            cp_async_zfill_4(&Bs[st][kk][lp], ok ? pix_ptr + e.x : in, ok);
        }
        fetch_decode(k0 + TK_KC);
    };

    const int ox = tid % OCL, pxl = tid / OCL;
    // accumulators: pairs of neighbouring pixels in one 64-bit register when a thread owns at least two
    constexpr int TP = TN >= 2 ? TN / 2 : 1;
    uint64_t acc2[TM][TP];
    float acc1[TM];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        acc1[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < TP; ++j) acc2[i][j] = 0ull;
    }

    const int n_slabs = (P.K + TK_KC - 1) / TK_KC;
#pragma unroll
    for (int s = 0; s < TK_STAGES - 1; ++s) {
        if (s < n_slabs) load_stage(s, s * TK_KC);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int s = 0; s < n_slabs; ++s) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TK_STAGES - 2) : "memory");
        __syncthreads();  // slab s has landed for everyone, and everyone is done with the stage refilled next
        const int nxt = s + TK_STAGES - 1;
        if (nxt < n_slabs) load_stage(nxt % TK_STAGES, nxt * TK_KC);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = s % TK_STAGES;
#pragma unroll
        for (int k4 = 0; k4 < TK_KC / 4; ++k4) {
            // all operands of four k-steps first (TM 128-bit reads of the weights, four reads of the pixels), then
            // their FMAs: the reads of the next group overlap the chain of this one
            float4 a[TM];
            float b[4][TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = *reinterpret_cast<const float4 *>(&As[st][ox + OCL * i][k4 * 4]);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float *bp = &Bs[st][k4 * 4 + kk][pxl * TN];
                if constexpr (TN == 8) {
                    const float4 t = *reinterpret_cast<const float4 *>(bp), w = *reinterpret_cast<const float4 *>(bp + 4);
                    b[kk][0] = t.x; b[kk][1] = t.y; b[kk][2] = t.z; b[kk][3] = t.w;
                    b[kk][4] = w.x; b[kk][5] = w.y; b[kk][6] = w.z; b[kk][7] = w.w;
                } else if constexpr (TN == 4) {
                    const float4 t = *reinterpret_cast<const float4 *>(bp);
                    b[kk][0] = t.x; b[kk][1] = t.y; b[kk][2] = t.z; b[kk][3] = t.w;
                } else if constexpr (TN == 2) {
                    const float2 t = *reinterpret_cast<const float2 *>(bp);
                    b[kk][0] = t.x; b[kk][1] = t.y;
                } else {
                    b[kk][0] = *bp;
                }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint64_t bpair[TP];
                if constexpr (TN >= 2) {
#pragma unroll
                    for (int j = 0; j < TP; ++j) bpair[j] = pack2(b[kk][2 * j], b[kk][2 * j + 1]);
                }
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
                    if constexpr (TN >= 2) {
                        const uint64_t ap = pack2(av, av);
#pragma unroll
                        for (int j = 0; j < TP; ++j) acc2[i][j] = fma2(ap, bpair[j], acc2[i][j]);
                    } else {
                        acc1[i] = __fmaf_rn(av, b[kk][0], acc1[i]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    if constexpr (TN >= 4) {
        // four consecutive pixels from a multiple of four lie in one image and on a 16-byte boundary when the
        // plane size is a multiple of four: one 128-bit store per channel instead of four scattered words
        if (ohw % 4 == 0 && P.out_img_stride % 4 == 0) {
#pragma unroll
            for (int q = 0; q < TN / 4; ++q) {
                const int pix = pix0 + pxl * TN + q * 4;
                if (pix >= P.npix) continue;  // npix is a multiple of four here, so a started group is complete
                const int img = pix / ohw, rem = pix - img * ohw;
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const int r = oc0 + ox + OCL * i;
                    if (r >= P.oc) continue;
                    float4 v;
                    unpack2(acc2[i][q * 2], v.x, v.y);
                    unpack2(acc2[i][q * 2 + 1], v.z, v.w);
                    v.x = ep(v.x, r); v.y = ep(v.y, r); v.z = ep(v.z, r); v.w = ep(v.w, r);
                    *reinterpret_cast<float4 *>(out + (size_t)img * P.out_img_stride + (size_t)r * ohw + rem) = v;
                }
            }
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int pix = pix0 + pxl * TN + j;
        if (pix >= P.npix) continue;
        const int img = pix / ohw, rem = pix - img * ohw;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = oc0 + ox + OCL * i;
            float v = acc1[i];
            if constexpr (TN >= 2) {
                float lo, hi;
                unpack2(acc2[i][j / 2], lo, hi);
                v = j % 2 ? hi : lo;
            }
            if (r < P.oc) out[(size_t)img * P.out_img_stride + (size_t)r * ohw + rem] = ep(v, r);
        }
    }
}

// Few output pixels and a long reduction (the 7x7 and 14x14 ResNet layers): every block row would gather the same
// K x pixels matrix again, at some sixteen instructions per element against one FMA per element and channel.  Here
// the matrix is written once -- B[k][pixel], rows padded with zeros to `ld` floats -- and the blocks stream it with
// 16-byte copies.  It is at most a few MB and stays in L2.
__global__ void __launch_bounds__(256) im2col_matrix_kernel(const float *__restrict__ in, const int2 *__restrict__ ktab,
                                                            float *__restrict__ B, IgemmParams P, int ld) {
    const int ohw = P.oh * P.ow;
    const size_t total = (size_t)P.K * ld;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int pix = (int)(idx % ld), k = (int)(idx / ld);
        float v = 0.0f;
        if (pix < P.npix) {
            const int img = pix / ohw, rem = pix - img * ohw;
            const int oi = rem / P.ow, oj = rem - oi * P.ow;
            const int2 e = __ldg(ktab + k);
            const int row = oi * P.sh - P.pad_t + (e.y >> 16), col = oj * P.sw - P.pad_l + (e.y & 0xffff);
            if ((unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw)
                v = __ldg(in + (size_t)img * P.in_img_stride + (ptrdiff_t)(oi * P.sh - P.pad_t) * P.iw + (oj * P.sw - P.pad_l) + e.x);
        }
        B[idx] = v;
    }
}

template <int BM, int BN, int TM, int TN, int TK_STAGES>
int launch_tile(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const int2 *d_ktab,
                const IgemmParams &P, const Epilogue &ep, const float *d_bmat = nullptr, int ld = 0) {
    constexpr int NT = (BM / TM) * (BN / TN);
    const size_t smem = (size_t)TK_STAGES * (BM * TK_KCP + TK_KC * (BN + 4)) * sizeof(float);
    FC_CHECK_CUDA(cudaFuncSetAttribute(igemm_ffma_tile_kernel<BM, BN, TM, TN, TK_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    dim3 grid((unsigned)ceil_div(P.npix, BN), (unsigned)ceil_div(P.oc, BM)), block(NT);
    igemm_ffma_tile_kernel<BM, BN, TM, TN, TK_STAGES><<<grid, block, smem, ctx->stream>>>(d_in, d_kernel, d_out, d_ktab, P,
                                                                              P.K % 4 == 0 ? 1 : 0, ep, d_bmat, ld);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// ---------------------------------------------------------------------------------------------
// Depthwise convolution (group == input channels): every output channel reads ONE input channel, so the
// reduction is kh*kw long and the layer is pure streaming.  One thread per output element, the same chain as
// everywhere else: one accumulator, one FMA per (u,v), ascending.  `mult` output channels share an input channel.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) depthwise_kernel(const float *__restrict__ in, const float *__restrict__ w,
                                                        float *__restrict__ out, IgemmParams P, int mult, Epilogue ep) {
    const int ohw = P.oh * P.ow;
    const size_t total = (size_t)P.n * P.oc * ohw;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int rem = (int)(idx % ohw);
        const size_t r = idx / ohw;
        const int k = (int)(r % P.oc), img = (int)(r / P.oc);
        const int oi = rem / P.ow, oj = rem - oi * P.ow;
        const int row0 = oi * P.sh - P.pad_t, col0 = oj * P.sw - P.pad_l;
        const float *src = in + ((size_t)img * P.ic + k / mult) * P.ih * P.iw;
        const float *wk = w + (size_t)k * P.kh * P.kw;
        float acc = 0.0f;
        for (int u = 0; u < P.kh; ++u) {
            const int row = row0 + u;
            for (int v = 0; v < P.kw; ++v) {
                const int col = col0 + v;
                const float b = ((unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw)
                                    ? __ldg(src + (size_t)row * P.iw + col) : 0.0f;
                acc = __fmaf_rn(__ldg(wk + u * P.kw + v), b, acc);
            }
        }
        out[idx] = ep(acc, k);
    }
}

// ---------------------------------------------------------------------------------------------
// M, N and K all at most 32: the reference leaves its blocked SGEMM and runs the scalar triple loop
// ConvIm2colLayer::GEMM (convLayer/im2colConv.cpp:400-432, chosen at im2colConv.h:30-31), whose statement
// `C += temp * B` is a separate multiplication and addition, k ascending.  One thread per output element keeps
// that chain: a rounded product, then a rounded sum.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) igemm_tiny_unfused_kernel(const float *__restrict__ in, const float *__restrict__ A,
                                                                 float *__restrict__ out, IgemmParams P, Epilogue ep) {
    const int ohw = P.oh * P.ow;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P.n * P.oc * ohw) return;
    const int rem = idx % ohw, r = idx / ohw, k = r % P.oc, img = r / P.oc;
    const int oi = rem / P.ow, oj = rem - oi * P.ow;
    const float *src = in + (size_t)img * P.in_img_stride;
    const float *a = A + (size_t)k * P.K;
    float acc = 0.0f;
    int kk = 0;
    for (int c = 0; c < P.ic; ++c)
        for (int u = 0; u < P.kh; ++u)
            for (int v = 0; v < P.kw; ++v, ++kk) {
                const int row = oi * P.sh - P.pad_t + u, col = oj * P.sw - P.pad_l + v;
                const float b = ((unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw)
                                    ? __ldg(src + ((size_t)c * P.ih + row) * P.iw + col) : 0.0f;
                acc = __fadd_rn(acc, __fmul_rn(__ldg(a + kk), b));
            }
    out[(size_t)img * P.out_img_stride + (size_t)k * ohw + rem] = ep(acc, k);
}

}  // namespace

// the reference's own switch to its scalar GEMM (convLayer/im2colConv.h:30-31), per image as the reference has no batch
bool igemm_is_tiny(const fc_conv_desc &d, int oh, int ow) {
    return d.oc <= 32 && oh * ow <= 32 && d.ic * d.kh * d.kw <= 32;
}

int launch_depthwise(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const fc_conv_desc &d,
                     int oh, int ow, const Epilogue &ep) {
    IgemmParams P;
    P.n = d.batch; P.ic = d.ic; P.ih = d.ih; P.iw = d.iw; P.oc = d.oc; P.kh = d.kh; P.kw = d.kw;
    P.sh = d.sh; P.sw = d.sw; P.pad_l = d.pad_left; P.pad_t = d.pad_top; P.oh = oh; P.ow = ow;
    P.K = d.kh * d.kw;
    P.npix = d.batch * oh * ow;
    P.in_img_stride = (long long)d.ic * d.ih * d.iw;
    P.out_img_stride = (long long)d.oc * oh * ow;
    const size_t total = (size_t)d.batch * d.oc * oh * ow;
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const unsigned blocks = (unsigned)(ceil_div(total, 256) > (size_t)sms * 16 ? (size_t)sms * 16 : ceil_div(total, 256));
    depthwise_kernel<<<blocks, 256, 0, ctx->stream>>>(d_in, d_kernel, d_out, P, d.oc / d.ic, ep);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

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

// A layer streams a materialised gathered matrix when it has few output pixels and a long reduction (see
// im2col_matrix_kernel); its rows are padded to a multiple of 64 floats, the widest pixel block.
bool igemm_wants_matrix(const fc_conv_desc &d, int oh, int ow) {
    return d.group == 1 && (long long)d.batch * oh * ow <= 256 && (long long)d.ic * d.kh * d.kw >= 512;
}
size_t igemm_matrix_ld(const fc_conv_desc &d, int oh, int ow) { return (size_t)round_up(d.batch * oh * ow, 64); }

size_t igemm_ktab_entries(const fc_conv_desc &d) { return (size_t)round_up(d.ic * d.kh * d.kw, TK_KC); }

void igemm_fill_ktab(const fc_conv_desc &d, int *host_pairs) {
    const int K = d.ic * d.kh * d.kw, Kp = round_up(K, TK_KC);
    for (int k = 0; k < Kp; ++k) {
        if (k < K) {
            const int c = k / (d.kh * d.kw), r = k - c * d.kh * d.kw, u = r / d.kw, v = r - u * d.kw;
            host_pairs[2 * k] = (c * d.ih + u) * d.iw + v;
            host_pairs[2 * k + 1] = (u << 16) | v;
        } else {  // past the reduction: a row far below the image, so the copy zero-fills
            host_pairs[2 * k] = 0;
            host_pairs[2 * k + 1] = 0x4000 << 16;
        }
    }
}

int launch_igemm_ffma(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const fc_conv_desc &d,
                      int oh, int ow, const KernelCfg *cfg, const int *d_ktab, const Epilogue &ep, size_t in_img_stride,
                      size_t out_img_stride, float *d_bmat) {
    IgemmParams P;
    P.n = d.batch; P.ic = d.ic; P.ih = d.ih; P.iw = d.iw; P.oc = d.oc; P.kh = d.kh; P.kw = d.kw;
    P.sh = d.sh; P.sw = d.sw; P.pad_l = d.pad_left; P.pad_t = d.pad_top; P.oh = oh; P.ow = ow;
    P.K = d.ic * d.kh * d.kw;
    P.npix = d.batch * oh * ow;
    P.in_img_stride = in_img_stride ? (long long)in_img_stride : (long long)d.ic * d.ih * d.iw;
    P.out_img_stride = out_img_stride ? (long long)out_img_stride : (long long)d.oc * oh * ow;
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    if (igemm_is_tiny(d, oh, ow)) {  // the one shape class whose reference arithmetic is not a fused multiply-add
        const int total = d.batch * d.oc * oh * ow;
        FC_CHECK_CUDA(launch_pdl(igemm_tiny_unfused_kernel, dim3((unsigned)ceil_div(total, 256)), dim3(256), 0, ctx->stream,
                                 d_in, d_kernel, d_out, P, ep));
        return FC_OK;
    }
    const int pick = cfg ? cfg->skinny : 0;
    const bool wide_m = cfg && cfg->bm ? cfg->bm == 128 : d.oc > 64;
    const bool wide_n = cfg && cfg->bn ? cfg->bn == 128 : P.npix > 64;
    // skinny = 2 asks for the 16x16-thread kernel; otherwise the table-driven kernel, in the block shape bm x bn when
    // skinny = 1 names one, else in the heuristic's
    if (d_ktab && pick != 2) {
        const int2 *tab = reinterpret_cast<const int2 *>(d_ktab);
        const int shapes[5][2] = {{64, 64}, {32, 64}, {32, 32}, {16, 32}, {8, 32}};
        // 8x8 and 8x4 outputs per thread, two CTAs per SM: a third to a half fewer shared-memory reads per FMA
        // than 64x64, once the grid fills every CTA slot of the machine and the channel blocks are not mostly padding
        const int large[3][2] = {{128, 128}, {128, 64}, {64, 128}};
        int bm = 0, bn = 0;
        if (pick == 1 && cfg->bm && cfg->bn) {
            bm = cfg->bm; bn = cfg->bn;
        } else {
            // the largest block that still puts a CTA on about two thirds of the SMs, else the one with most CTAs:
            // Tuning() consistently preferred ~100-130 CTAs of a larger block (fewer gather instructions per FMA,
            // fewer re-reads of the weights) over 200-400 CTAs of the smallest one
            size_t best = 0;
            for (const auto &sh : large) {
                const size_t rows = ceil_div(d.oc, sh[0]), ctas = ceil_div(P.npix, sh[1]) * rows;
                if (ctas >= 2 * (size_t)sms && 4 * (size_t)d.oc >= 3 * rows * sh[0]) { bm = sh[0]; bn = sh[1]; break; }
            }
            if (bm == 0) for (const auto &sh : shapes) {
                const size_t ctas = ceil_div(P.npix, sh[1]) * ceil_div(d.oc, sh[0]);
                if (20 * ctas >= 13 * (size_t)sms) { bm = sh[0]; bn = sh[1]; break; }
                if (ctas > best) { best = ctas; bm = sh[0]; bn = sh[1]; }
            }
        }
        const float *bmat = nullptr;
        int ld = 0;
        if (d_bmat != nullptr && igemm_wants_matrix(d, oh, ow)) {  // write the gathered matrix once, then stream it
            ld = (int)igemm_matrix_ld(d, oh, ow);
            const size_t total = (size_t)P.K * ld;
            const unsigned blocks = (unsigned)(ceil_div(total, 256) > (size_t)sms * 8 ? (size_t)sms * 8 : ceil_div(total, 256));
            im2col_matrix_kernel<<<blocks, 256, 0, ctx->stream>>>(d_in, tab, d_bmat, P, ld);
            FC_CHECK_CUDA(cudaGetLastError());
            bmat = d_bmat;
        }
        if (bm == 128 && bn == 128) return launch_tile<128, 128, 8, 8, 3>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 128 && bn == 64) return launch_tile<128, 64, 8, 4, 3>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 64 && bn == 128) return launch_tile<64, 128, 4, 8, 3>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 64 && bn == 64) return launch_tile<64, 64, 4, 4, 3>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 32 && bn == 64) return launch_tile<32, 64, 2, 4, 4>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 32 && bn == 32) return launch_tile<32, 32, 2, 2, 6>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 16 && bn == 32) return launch_tile<16, 32, 1, 2, 8>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        if (bm == 8 && bn == 32) return launch_tile<8, 32, 1, 1, 8>(ctx, d_in, d_kernel, d_out, tab, P, ep, bmat, ld);
        set_error("no table-driven implicit GEMM with a %d x %d block", bm, bn);
        return FC_ERR_INVALID_ARG;
    }
    // no table (the stage entry point outside a planned layer): the 16x16-thread kernel for every size
    dim3 grid((unsigned)ceil_div(P.npix, wide_n ? 128 : 64), (unsigned)ceil_div(d.oc, wide_m ? 128 : 64)), block(THREADS);
    if (wide_m && wide_n)
        igemm_ffma_kernel<128, 128><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P, ep);
    else if (wide_m)
        igemm_ffma_kernel<128, 64><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P, ep);
    else if (wide_n)
        igemm_ffma_kernel<64, 128><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P, ep);
    else
        igemm_ffma_kernel<64, 64><<<grid, block, 0, ctx->stream>>>(d_in, d_kernel, d_out, P, ep);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
