// Winograd F(6x6,3x3) transform kernels: filter (one-time), input, output.
//
// The arithmetic mirrors FastConv's NEON transforms operation by operation so
// that, together with the sequential-FMA TensorGEMM, the whole layer is
// bit-identical to the reference: every multiply and add below is an explicit
// round-to-nearest intrinsic (the compiler may not contract them into FMAs),
// and __fmaf_rn appears exactly where the reference issues vfmaq_f32.
//
// Layouts (ic contiguous, padded with zeros to icp = roundup(ic, 8)):
//   U: packed 128 x 32 boxes (upack_index)   V[p][tp][icp]   M[p][oc][tp]     p = col*8 + row
#include <cuda_fp16.h>

#include <cstdlib>

#include "fc_internal.h"

namespace fc {

__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }

// G applied along one axis: winograd_f6k3_kernel_transform_v1, winoF63ZC/winoF63ZC.cpp:14-79.
__device__ __forceinline__ void filter_transform_1d(float g0, float g1, float g2, float w[8]) {
    float w2 = add(g0, g2);
    float w4 = add(g0, mul(4.0f, g2));
    float w6 = add(g2, mul(4.0f, g0));
    const float two_g1 = mul(g1, 2.0f);
    float w1 = add(w2, g1);
    w2 = sub(w2, g1);
    float w3 = add(w4, two_g1);
    w4 = sub(w4, two_g1);
    float w5 = add(w6, two_g1);
    w6 = sub(w6, two_g1);
    const float c29 = (float)(-2.0 / 9), c90 = (float)(1.0 / 90), c180 = (float)(1.0 / 180);
    w[0] = g0;
    w[1] = mul(w1, c29);
    w[2] = mul(w2, c29);
    w[3] = mul(w3, c90);
    w[4] = mul(w4, c90);
    w[5] = mul(w5, c180);
    w[6] = mul(w6, c180);
    w[7] = g2;
}

// B^T applied along one axis, in place: input_transform_v1, winoF63ZC/winoF63ZC.cpp:112-169.
__device__ __forceinline__ void input_transform_1d(float &r0, float &r1, float &r2, float &r3, float &r4, float &r5,
                                                   float &r6, float &r7) {
    const float n0 = add(sub(r0, r6), mul(sub(r4, r2), 5.25f));
    const float n7 = add(sub(r7, r1), mul(sub(r3, r5), 5.25f));
    const float t1 = sub(add(r2, r6), mul(r4, 4.25f));
    const float t2 = sub(add(r1, r5), mul(r3, 4.25f));
    const float s1 = mul(r4, 1.25f);
    const float s2 = mul(r3, 2.5f);
    float p1 = sub(add(r6, mul(r2, 0.25f)), s1);
    float p2 = add(sub(mul(r1, 0.5f), s2), mul(r5, 2.0f));
    const float n3 = add(p1, p2);
    const float n4 = sub(p1, p2);
    p1 = add(r6, mul(sub(r2, s1), 4.0f));
    p2 = add(sub(mul(r1, 2.0f), s2), mul(r5, 0.5f));
    const float n5 = add(p1, p2);
    const float n6 = sub(p1, p2);
    r1 = add(t1, t2);
    r2 = sub(t1, t2);
    r0 = n0; r3 = n3; r4 = n4; r5 = n5; r6 = n6; r7 = n7;
}

// A^T applied along one axis: winograd_f6k3_output_transform_inplace_v1,
// winoF63ZC/winoF63ZC.cpp:171-228 (vfmaq_f32(a,b,c) = a + b*c, fused).
__device__ __forceinline__ void output_transform_1d(float m0, float m1, float m2, float m3, float m4, float m5,
                                                    float m6, float m7, float s[6]) {
    const float a12 = add(m1, m2), s12 = sub(m1, m2);
    const float a34 = add(m3, m4), s34 = sub(m3, m4);
    const float a56 = add(m5, m6), s56 = sub(m5, m6);
    float o0 = add(m0, a12);
    float o5 = add(m7, s12);
    float o1 = __fmaf_rn(16.0f, s56, s12);
    float o4 = __fmaf_rn(16.0f, a34, a12);
    float o2 = __fmaf_rn(8.0f, a56, a12);
    float o3 = __fmaf_rn(8.0f, s34, s12);
    o0 = __fmaf_rn(32.0f, a56, o0);
    o0 = add(o0, a34);
    o5 = __fmaf_rn(32.0f, s34, o5);
    o5 = add(o5, s56);
    o1 = __fmaf_rn(s34, 2.0f, o1);
    o4 = __fmaf_rn(a56, 2.0f, o4);
    o2 = __fmaf_rn(a34, 4.0f, o2);
    o3 = __fmaf_rn(s56, 4.0f, o3);
    s[0] = o0; s[1] = o1; s[2] = o2; s[3] = o3; s[4] = o4; s[5] = o5;
}

// ---------------------------------------------------------------------------------------------
// Filter transform: U = G g G^T, G over the filter rows first, then over the columns
// (offline_kernel_transform_v1, winoF63ZC/winoF63ZC.cpp:286-297).  One thread per (oc, ic) of the padded
// box grid; threads of a warp walk ic, so each of the 64 stores per thread is one 128-byte row of a
// packed 128 x 32 box (see upack_index).  Padding rows and columns are written as zeros.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) filter_transform_kernel(const float *__restrict__ kernel,
                                                               float *__restrict__ U, int oc, int ic, int n_ocb,
                                                               int n_kb) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int k = blockIdx.y;
    if (c >= n_kb * U_BOX_COLS) return;
    const size_t plane = (size_t)n_ocb * n_kb * U_BOX_ELEMS;  // floats per position
    float *dst = U + upack_index(0, k, c, n_ocb, n_kb);
    if (c >= ic || k >= oc) {  // zero padding of the box grid
#pragma unroll
        for (int p = 0; p < 64; ++p) dst[p * plane] = 0.0f;
        return;
    }
    const float *g = kernel + ((size_t)k * ic + c) * 9;
    float gv[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) gv[i] = g[i];
    float gg[8][3];
#pragma unroll
    for (int v = 0; v < 3; ++v) {
        float w[8];
        filter_transform_1d(gv[v], gv[3 + v], gv[6 + v], w);
#pragma unroll
        for (int r = 0; r < 8; ++r) gg[r][v] = w[r];
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float w[8];
        filter_transform_1d(gg[r][0], gg[r][1], gg[r][2], w);
#pragma unroll
        for (int col = 0; col < 8; ++col) dst[(size_t)(col * 8 + r) * plane] = w[col];
    }
}

int launch_filter_transform(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic) {
    const int n_ocb = (oc + U_BOX_ROWS - 1) / U_BOX_ROWS, n_kb = (ic + U_BOX_COLS - 1) / U_BOX_COLS;
    dim3 block(128), grid((unsigned)ceil_div(n_kb * U_BOX_COLS, 128), (unsigned)(n_ocb * U_BOX_ROWS));
    filter_transform_kernel<<<grid, block, 0, ctx->stream>>>(d_kernel, d_U, oc, ic, n_ocb, n_kb);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// Same transform written in the layout of the FP32 (FFMA) TensorGEMM: U[p][ic][ocp] with the OUTPUT channel
// contiguous (ocp = oc rounded up to 4), so that a k-row of a GEMM tile is one contiguous run and goes to
// shared memory with plain 16-byte async copies, no transposition.  Threads of a warp walk oc.
__global__ void __launch_bounds__(128) filter_transform_rowmajor_kernel(const float *__restrict__ kernel,
                                                                        float *__restrict__ U, int oc, int ic, int icp,
                                                                        int ocp) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    const int c = blockIdx.y;
    if (k >= ocp) return;
    const size_t plane = (size_t)icp * ocp;
    float *dst = U + (size_t)c * ocp + k;
    if (c >= ic || k >= oc) {
#pragma unroll
        for (int p = 0; p < 64; ++p) dst[p * plane] = 0.0f;
        return;
    }
    const float *g = kernel + ((size_t)k * ic + c) * 9;
    float gv[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) gv[i] = g[i];
    float gg[8][3];
#pragma unroll
    for (int v = 0; v < 3; ++v) {
        float w[8];
        filter_transform_1d(gv[v], gv[3 + v], gv[6 + v], w);
#pragma unroll
        for (int r = 0; r < 8; ++r) gg[r][v] = w[r];
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float w[8];
        filter_transform_1d(gg[r][0], gg[r][1], gg[r][2], w);
#pragma unroll
        for (int col = 0; col < 8; ++col) dst[(size_t)(col * 8 + r) * plane] = w[col];
    }
}

int launch_filter_transform_rowmajor(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic) {
    const int icp = round_up(ic, 8), ocp = round_up(oc, 4);
    dim3 block(128), grid((unsigned)ceil_div(ocp, 128), (unsigned)icp);
    filter_transform_rowmajor_kernel<<<grid, block, 0, ctx->stream>>>(d_kernel, d_U, oc, ic, icp, ocp);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// ---------------------------------------------------------------------------------------------
// Input transform: V = B^T d B per 8x8 tile at (6*ty - pad, 6*tx - pad), zero outside the image
// (winoF63ZC/winoF63ZC.cpp:541-612); B^T over the tile rows first, then the columns (:614-630).
//
// The layers this serves at batch 1 are tiny, so the kernel is built for latency: a block owns ONE tile
// and 32 channels and spreads each (tile, channel) item over 8 threads.
//   phase 1  256 threads fetch the 32 windows: 8 consecutive floats of an image row per lane group,
//            zero outside the image / past the last tile / past the last channel (so the padding of V
//            falls out of the arithmetic);
//   pass 1   thread (x, channel) transforms column x of its window in place in shared memory;
//   pass 2   thread (y, channel) transforms row y and stores the 8 positions p = x*8 + y, each warp
//            store being one 128-byte line of V[p][tile][c..c+31].
// Shared memory is indexed [y*8+x][channel] with the channel fastest, so every access is conflict-free.
// ---------------------------------------------------------------------------------------------
constexpr int IT_CH = 32;
constexpr int IT_LD = IT_CH + 1;

__global__ void __launch_bounds__(256) input_transform_kernel(const float *__restrict__ in, float *__restrict__ V,
                                                              int n_tiles, int ic, int icp, int tp, int ih, int iw,
                                                              int pad, int th, int tw) {
    __shared__ float win[64 * IT_LD];
    const int tid = threadIdx.x;
    const int c0 = blockIdx.y * IT_CH, tile = blockIdx.x;
    pdl_trigger();
    pdl_wait();  // the input may be the previous layer's output; V may still be read by an earlier GEMM
    {
        const int x = tid & 7, cl = tid >> 3;
        const int c = c0 + cl;
        const int per_img = th * tw;
        const int img = tile / per_img, tt = tile - img * per_img;
        const int row0 = (tt / tw) * 6 - pad, col = (tt % tw) * 6 - pad + x;
        const bool ok = c < ic && tile < n_tiles && col >= 0 && col < iw;
        const float *src = in + ((size_t)img * ic + c) * ih * iw + col;
        float v[8];
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            const int yy = row0 + y;
            v[y] = (ok && yy >= 0 && yy < ih) ? __ldg(src + (ptrdiff_t)yy * iw) : 0.0f;
        }
#pragma unroll
        for (int y = 0; y < 8; ++y) win[(y * 8 + x) * IT_LD + cl] = v[y];
    }
    __syncthreads();
    const int lane = tid & 31, w = tid >> 5;  // w = column (pass 1) or row (pass 2) of the window
    {
        float *q = win + w * IT_LD + lane;  // column w: elements (y*8 + w)
        float r0 = q[0 * 8 * IT_LD], r1 = q[1 * 8 * IT_LD], r2 = q[2 * 8 * IT_LD], r3 = q[3 * 8 * IT_LD];
        float r4 = q[4 * 8 * IT_LD], r5 = q[5 * 8 * IT_LD], r6 = q[6 * 8 * IT_LD], r7 = q[7 * 8 * IT_LD];
        input_transform_1d(r0, r1, r2, r3, r4, r5, r6, r7);
        q[0 * 8 * IT_LD] = r0; q[1 * 8 * IT_LD] = r1; q[2 * 8 * IT_LD] = r2; q[3 * 8 * IT_LD] = r3;
        q[4 * 8 * IT_LD] = r4; q[5 * 8 * IT_LD] = r5; q[6 * 8 * IT_LD] = r6; q[7 * 8 * IT_LD] = r7;
    }
    __syncthreads();
    const int c = c0 + lane;
    if (c >= icp) return;
    const float *q = win + w * 8 * IT_LD + lane;  // row w: elements (w*8 + x)
    float r0 = q[0 * IT_LD], r1 = q[1 * IT_LD], r2 = q[2 * IT_LD], r3 = q[3 * IT_LD];
    float r4 = q[4 * IT_LD], r5 = q[5 * IT_LD], r6 = q[6 * IT_LD], r7 = q[7 * IT_LD];
    input_transform_1d(r0, r1, r2, r3, r4, r5, r6, r7);
    const size_t plane = (size_t)tp * icp;
    float *dst = V + (size_t)w * plane + (size_t)tile * icp + c;  // p = x*8 + w
    dst[0 * 8 * plane] = r0; dst[1 * 8 * plane] = r1; dst[2 * 8 * plane] = r2; dst[3 * 8 * plane] = r3;
    dst[4 * 8 * plane] = r4; dst[5 * 8 * plane] = r5; dst[6 * 8 * plane] = r6; dst[7 * 8 * plane] = r7;
}

int launch_input_transform(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g) {
    dim3 block(256), grid((unsigned)g.tp, (unsigned)ceil_div(g.icp, IT_CH));
    FC_CHECK_CUDA(launch_pdl(input_transform_kernel, grid, block, 0, ctx->stream, d_in, d_V, g.tiles, g.ic, g.icp, g.tp,
                             g.ih, g.iw, g.pad, g.th, g.tw));
    return FC_OK;
}

// The same transform written in the layout of the FP32 (FFMA) TensorGEMM: V[p][ic][tp] with the TILE axis
// contiguous.  Lanes run along consecutive tiles (TPW = 32, 16 or 8 of them, the rest of the warp taking
// further channels), so the window loads sweep contiguous image rows and every store is one run of
// V[p][c][tile..].  Same three phases as above, eight threads per (tile, channel) item.
template <int TPW>
__global__ void __launch_bounds__(256) input_transform_rowmajor_kernel(const float *__restrict__ in,
                                                                       float *__restrict__ V, int n_tiles, int ic,
                                                                       int icp, int tp, int ih, int iw, int pad,
                                                                       int th, int tw) {
    constexpr int CPB = 32 / TPW;  // channels per block
    __shared__ float win[64 * IT_LD];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int tl = lane % TPW, cl = lane / TPW;
    const int tile = blockIdx.x * TPW + tl, c = blockIdx.y * CPB + cl;
    pdl_trigger();
    pdl_wait();
    {   // phase 1: thread (lane, w) fetches row w of its item's window
        const int per_img = th * tw;
        const int img = tile / per_img, tt = tile - img * per_img;
        const int yy = (tt / tw) * 6 - pad + w, col0 = (tt % tw) * 6 - pad;
        const bool ok = c < ic && tile < n_tiles && yy >= 0 && yy < ih;
        const float *src = in + (((size_t)img * ic + c) * ih + yy) * iw + col0;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const int xx = col0 + x;
            win[(w * 8 + x) * IT_LD + lane] = (ok && xx >= 0 && xx < iw) ? __ldg(src + x) : 0.0f;
        }
    }
    __syncthreads();
    {
        float *q = win + w * IT_LD + lane;  // column w
        float r0 = q[0 * 8 * IT_LD], r1 = q[1 * 8 * IT_LD], r2 = q[2 * 8 * IT_LD], r3 = q[3 * 8 * IT_LD];
        float r4 = q[4 * 8 * IT_LD], r5 = q[5 * 8 * IT_LD], r6 = q[6 * 8 * IT_LD], r7 = q[7 * 8 * IT_LD];
        input_transform_1d(r0, r1, r2, r3, r4, r5, r6, r7);
        q[0 * 8 * IT_LD] = r0; q[1 * 8 * IT_LD] = r1; q[2 * 8 * IT_LD] = r2; q[3 * 8 * IT_LD] = r3;
        q[4 * 8 * IT_LD] = r4; q[5 * 8 * IT_LD] = r5; q[6 * 8 * IT_LD] = r6; q[7 * 8 * IT_LD] = r7;
    }
    __syncthreads();
    if (c >= icp || tile >= tp) return;
    const float *q = win + w * 8 * IT_LD + lane;  // row w
    float r0 = q[0 * IT_LD], r1 = q[1 * IT_LD], r2 = q[2 * IT_LD], r3 = q[3 * IT_LD];
    float r4 = q[4 * IT_LD], r5 = q[5 * IT_LD], r6 = q[6 * IT_LD], r7 = q[7 * IT_LD];
    input_transform_1d(r0, r1, r2, r3, r4, r5, r6, r7);
    const size_t plane = (size_t)icp * tp;
    float *dst = V + (size_t)w * plane + (size_t)c * tp + tile;  // p = x*8 + w
    dst[0 * 8 * plane] = r0; dst[1 * 8 * plane] = r1; dst[2 * 8 * plane] = r2; dst[3 * 8 * plane] = r3;
    dst[4 * 8 * plane] = r4; dst[5 * 8 * plane] = r5; dst[6 * 8 * plane] = r6; dst[7 * 8 * plane] = r7;
}

// Many tiles (large feature maps or batches): throughput matters more than latency, and the three-phase kernel above
// is bound by instruction issue (0.72 of the issue slots used, DRAM at 29 %), not by memory.  Here one thread owns a
// whole (channel, tile) item: 64 loads in flight, both passes in registers, 64 stores; no shared memory, no barrier,
// about half the instructions per item.  Lanes run along consecutive tiles, warps along channels.
constexpr int ITW_WARPS = 4;

template <bool ALONG_TILES>
__global__ void __launch_bounds__(32 * ITW_WARPS) input_transform_rowmajor_wide_kernel(
    const float *__restrict__ in, float *__restrict__ V, int n_tiles, int ic, int icp, int tp, int ih, int iw, int pad,
    int th, int tw, bool allow_pairs) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the warps of a block: ITW_WARPS channels of the same 32 tiles, or one channel of 32 * ITW_WARPS consecutive tiles
    const int tile = ALONG_TILES ? blockIdx.x * 32 * ITW_WARPS + threadIdx.x : blockIdx.x * 32 + lane;
    const int c = ALONG_TILES ? blockIdx.y : blockIdx.y * ITW_WARPS + warp;
    pdl_trigger();
    pdl_wait();  // the input may be the previous layer's output; V may still be read by an earlier GEMM
    if (c >= icp || tile >= tp) return;
    float r[8][8];  // [y][x]
    unsigned rows = 0, cols = 0;  // bit y / bit x set: inside the image
    const float *src = in;
    if (c < ic && tile < n_tiles) {
        const int per_img = th * tw;
        const int img = tile / per_img, tt = tile - img * per_img;
        const int y0 = (tt / tw) * 6 - pad, x0 = (tt % tw) * 6 - pad;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            rows |= (unsigned)(y0 + i >= 0 && y0 + i < ih) << i;
            cols |= (unsigned)(x0 + i >= 0 && x0 + i < iw) << i;
        }
        src = in + (((ptrdiff_t)img * ic + c) * ih + y0) * iw + x0;
    }
    // An even row length and an 8-byte aligned image let the window rows travel as aligned pairs: the window starts
    // at x0 = 6*tx - pad, whose parity is the padding's, so the pair grid starts `shift` = pad & 1 elements to its left
    // and 4 (or, shifted, 5) pairs cover it; with an even row length a pair lies wholly inside or wholly outside the
    // image.  37 % fewer load instructions than element by element, which is what this kernel is short of.
    const bool pairs = allow_pairs && (iw & 1) == 0 && (reinterpret_cast<uintptr_t>(in) & 7) == 0;
    if (pairs) {
        const int shift = pad & 1;
        // pair j holds window elements 2j - shift and 2j + 1 - shift; the one of them that always belongs to the window
        // (element 2j, or 7 for the fifth pair) says whether the pair lies inside the image
        unsigned pair_ok = 0;
#pragma unroll
        for (int j = 0; j < 5; ++j) pair_ok |= ((cols >> (j < 4 ? 2 * j : 7)) & 1u) << j;
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            const float2 *rp = reinterpret_cast<const float2 *>(src + (ptrdiff_t)y * iw - shift);
            float f[10];
#pragma unroll
            for (int j = 0; j < 5; ++j) {
                float2 q = make_float2(0.f, 0.f);
                if ((j < 4 || shift) && ((rows >> y) & (pair_ok >> j) & 1u)) q = __ldg(rp + j);
                f[2 * j] = q.x;
                f[2 * j + 1] = q.y;
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) r[y][x] = shift ? f[x + 1] : f[x];
        }
    } else if (rows == 0xffu && cols == 0xffu) {
#pragma unroll
        for (int y = 0; y < 8; ++y)
#pragma unroll
            for (int x = 0; x < 8; ++x) r[y][x] = __ldg(src + (ptrdiff_t)y * iw + x);
    } else {
#pragma unroll
        for (int y = 0; y < 8; ++y)
#pragma unroll
            for (int x = 0; x < 8; ++x)
                r[y][x] = ((rows >> y) & (cols >> x) & 1u) ? __ldg(src + (ptrdiff_t)y * iw + x) : 0.0f;
    }
#pragma unroll
    for (int x = 0; x < 8; ++x)  // along y, for every column
        input_transform_1d(r[0][x], r[1][x], r[2][x], r[3][x], r[4][x], r[5][x], r[6][x], r[7][x]);
#pragma unroll
    for (int y = 0; y < 8; ++y)  // along x, for every row
        input_transform_1d(r[y][0], r[y][1], r[y][2], r[y][3], r[y][4], r[y][5], r[y][6], r[y][7]);
    const size_t plane = (size_t)icp * tp;
    float *dst = V + (size_t)c * tp + tile;
#pragma unroll
    for (int x = 0; x < 8; ++x)
#pragma unroll
        for (int y = 0; y < 8; ++y) dst[(size_t)(x * 8 + y) * plane] = r[y][x];  // p = x*8 + y
}

// Which layers take the throughput-oriented input transform: one thread per item needs items enough to fill the
// machine.  From 64 tiles and 64 K (channel, tile) items on -- 8 images, whole VGG-16 stack: 1.607 ms against 1.619 ms
// with the kernel kept to 1024 tiles and more; one image: 0.381 against 0.382 ms the other way round, which is why the
// item count is part of the rule.  $FASTCONV_IT_WIDE_MIN=<tiles> replaces the rule by a plain threshold.
static bool it_wide(const WinoGeom &g) {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("FASTCONV_IT_WIDE_MIN");
        v = e && atoi(e) > 0 ? atoi(e) : 0;
    }
    if (v > 0) return g.tiles >= v;
    return g.tiles >= 64 && (long long)g.tiles * g.icp >= 64 * 1024;
}

int launch_input_transform_rowmajor(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g) {
    dim3 block(256);
    if (it_wide(g)) {
        static const bool pairs_on = !(getenv("FASTCONV_IT_PAIRS") && atoi(getenv("FASTCONV_IT_PAIRS")) == 0);
        // a block of four warps along the tile axis writes runs of 512 bytes per (position, channel) instead of 128:
        // measured 1-4 % faster at 64 images
        dim3 wblock(32 * ITW_WARPS);
        if (g.tiles >= 32 * ITW_WARPS) {
            dim3 grid((unsigned)ceil_div(g.tp, 32 * ITW_WARPS), (unsigned)g.icp);
            FC_CHECK_CUDA(launch_pdl(input_transform_rowmajor_wide_kernel<true>, grid, wblock, 0, ctx->stream, d_in, d_V, g.tiles,
                                     g.ic, g.icp, g.tp, g.ih, g.iw, g.pad, g.th, g.tw, pairs_on));
        } else {
            dim3 grid((unsigned)ceil_div(g.tp, 32), (unsigned)ceil_div(g.icp, ITW_WARPS));
            FC_CHECK_CUDA(launch_pdl(input_transform_rowmajor_wide_kernel<false>, grid, wblock, 0, ctx->stream, d_in, d_V, g.tiles,
                                     g.ic, g.icp, g.tp, g.ih, g.iw, g.pad, g.th, g.tw, pairs_on));
        }
        return FC_OK;
    }
    if (g.tiles > 16) {
        dim3 grid((unsigned)ceil_div(g.tp, 32), (unsigned)g.icp);
        FC_CHECK_CUDA(launch_pdl(input_transform_rowmajor_kernel<32>, grid, block, 0, ctx->stream, d_in, d_V, g.tiles,
                                 g.ic, g.icp, g.tp, g.ih, g.iw, g.pad, g.th, g.tw));
    } else if (g.tiles > 8) {
        dim3 grid((unsigned)ceil_div(g.tp, 16), (unsigned)ceil_div(g.icp, 2));
        FC_CHECK_CUDA(launch_pdl(input_transform_rowmajor_kernel<16>, grid, block, 0, ctx->stream, d_in, d_V, g.tiles,
                                 g.ic, g.icp, g.tp, g.ih, g.iw, g.pad, g.th, g.tw));
    } else {
        dim3 grid((unsigned)ceil_div(g.tp, 8), (unsigned)ceil_div(g.icp, 4));
        FC_CHECK_CUDA(launch_pdl(input_transform_rowmajor_kernel<8>, grid, block, 0, ctx->stream, d_in, d_V, g.tiles,
                                 g.ic, g.icp, g.tp, g.ih, g.iw, g.pad, g.th, g.tw));
    }
    return FC_OK;
}

// ---------------------------------------------------------------------------------------------
// Output transform: Y = A^T M A, A^T over the tile columns first (for every row), then over the
// rows (winoF63ZC/winoF63ZC.cpp:905-912), clipped store at the right/bottom edges (:928-969).
//
// Also built for latency: a block owns TPW consecutive tiles of OCB = 32/TPW output channels and
// spreads every (oc, tile) item over 8 threads.
//   pass 1   warp r (0..7) loads row r of M's 8x8 (8 loads per thread, the lanes of a channel run
//            along the contiguous tile axis of M[p][oc][tile]) and reduces it to 6 values;
//   pass 2   warp j (0..5) reduces column j over the 8 rows and stages the 6 outputs;
//   store    the staged 6 x (6*TPW) block of every channel is written along the output rows: tiles
//            that are neighbours in x are neighbours in memory.
// TPW is 32, 16 or 8 so that small feature maps (9 or 4 tiles) do not idle most lanes.
// ---------------------------------------------------------------------------------------------
template <int TPW, typename Store>
__device__ __forceinline__ void output_transform_block(const float *__restrict__ M, int n_tiles, int oc, int tp, int oh,
                                                       int ow, int th, int tw, Store store) {
    constexpr int OCB = 32 / TPW;
    constexpr int ROW = TPW * 6 + 1;
    __shared__ float hbuf[8][6][33];          // [row][j][lane]
    __shared__ float stage[OCB][6][ROW];      // [oc][i][tile*6 + j]
    __shared__ int tile_org[TPW];             // element offset of each tile's top-left output, -1 past the end
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int tl = lane % TPW, ol = lane / TPW;
    const int t_base = blockIdx.x * TPW, k_base = blockIdx.y * OCB;
    const int t = t_base + tl, k = k_base + ol;
    const bool active = t < n_tiles && k < oc;
    const size_t plane = (size_t)oc * tp;
    if (threadIdx.x < TPW) {
        const int tile = t_base + threadIdx.x;
        int org = -1;
        if (tile < n_tiles) {
            const int per_img = th * tw;
            const int img = tile / per_img, tt = tile - img * per_img;
            org = ((tt / tw) * 6) << 16 | ((tt % tw) * 6);  // y0 : x0 (both below 32768)
            tile_org[threadIdx.x] = org;
        } else {
            tile_org[threadIdx.x] = -1;
        }
    }
    pdl_trigger();
    pdl_wait();  // M comes from the GEMM launched just before
    {   // pass 1: row w of the 8x8, positions p = col*8 + w
        float m[8];
        const float *src = M + (size_t)w * plane + (size_t)k * tp + t;
#pragma unroll
        for (int col = 0; col < 8; ++col) m[col] = active ? __ldg(src + (size_t)col * 8 * plane) : 0.0f;
        float h[6];
        output_transform_1d(m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], h);
#pragma unroll
        for (int j = 0; j < 6; ++j) hbuf[w][j][lane] = h[j];
    }
    __syncthreads();
    if (w < 6) {  // pass 2: column w over the 8 rows
        float s[6];
        output_transform_1d(hbuf[0][w][lane], hbuf[1][w][lane], hbuf[2][w][lane], hbuf[3][w][lane], hbuf[4][w][lane],
                            hbuf[5][w][lane], hbuf[6][w][lane], hbuf[7][w][lane], s);
#pragma unroll
        for (int i = 0; i < 6; ++i) stage[ol][i][tl * 6 + w] = s[i];
    }
    __syncthreads();
    const int per_img = th * tw;
    // 6 rows x OCB channels x (6*TPW) floats, one element per thread and step, consecutive threads on
    // consecutive floats of an output row; the tile origins were decoded once into tile_org
    constexpr int PER_ROW = TPW * 6;
    const size_t out_page = (size_t)oh * ow;
    for (int idx = threadIdx.x; idx < OCB * 6 * PER_ROW; idx += 256) {
        const int e = idx % PER_ROW, i = (idx / PER_ROW) % 6, o = idx / (PER_ROW * 6);
        const int te = e / 6, j = e - te * 6;
        const int org = tile_org[te], kk = k_base + o;
        if (org < 0 || kk >= oc) continue;
        const int y = (org >> 16) + i, x = (org & 0xffff) + j;
        const int img = (t_base + te) / per_img;
        if (y < oh && x < ow) store(((size_t)img * oc + kk) * out_page + (size_t)y * ow + x, kk, stage[o][i][e]);
    }
}

template <int TPW>
__global__ void __launch_bounds__(256) output_transform_kernel(const float *__restrict__ M, float *__restrict__ out,
                                                               int n_tiles, int oc, int tp, int oh, int ow, int th,
                                                               int tw, Epilogue ep) {
    output_transform_block<TPW>(M, n_tiles, oc, tp, oh, ow, th, tw,
                                [out, ep](size_t at, int ch, float v) { out[at] = ep(v, ch); });
}

// The same transform for a layer whose output channels are split over several GPUs: every result is stored
// into the output buffer of each GPU (its own and, through peer-mapped pointers over NVLink, the others'), so
// the all-gather of the channel slabs happens in the stores of the transform itself.  dst.base[r] already
// points at this rank's first channel inside rank r's buffer.
template <int TPW>
__global__ void __launch_bounds__(256) output_transform_scatter_kernel(const float *__restrict__ M, PeerOuts dst,
                                                                       int n_tiles, int oc, int tp, int oh, int ow,
                                                                       int th, int tw, Epilogue ep) {
    output_transform_block<TPW>(M, n_tiles, oc, tp, oh, ow, th, tw, [&dst, ep](size_t at, int ch, float v) {
        v = ep(v, ch);
#pragma unroll
        for (int r = 0; r < FC_MAX_PEERS; ++r)
            if (r < dst.count) dst.base[r][at] = v;
    });
}

// Scatter with the step kept on the device and the publication folded into the kernel.  Every block stores its
// results into the buffers of the parity of this forward; when a block is done, one of its threads orders the block's
// stores before a device-wide ticket; the block that draws the last ticket issues ONE system-wide fence and writes the
// step number into flag[rank] of every rank.  Nothing is passed by the host per forward, so a CUDA graph can replay
// the launch, and no separate publishing kernel follows.
template <int TPW>
__global__ void __launch_bounds__(256) output_transform_scatter_publish_kernel(const float *__restrict__ M,
                                                                               ScatterPublish dst, int n_tiles, int oc,
                                                                               int tp, int oh, int ow, int th, int tw,
                                                                               Epilogue ep) {
    __shared__ int s_step;
    // read after the predecessor in the stream has completed (the block helper waits for it before it touches M;
    // the counter was last written by this layer's previous forward, which is older still)
    pdl_wait();
    if (threadIdx.x == 0) s_step = *reinterpret_cast<volatile int *>(dst.step) + 1;
    __syncthreads();
    const int step = s_step, parity = step & 1;
    output_transform_block<TPW>(M, n_tiles, oc, tp, oh, ow, th, tw, [&dst, ep, parity](size_t at, int ch, float v) {
        v = ep(v, ch);
#pragma unroll
        for (int r = 0; r < FC_MAX_PEERS; ++r)
            if (r < dst.count) dst.base[parity][r][at] = v;
    });
    __syncthreads();  // every thread of the block has issued its stores
    if (threadIdx.x == 0) {
        __threadfence();  // ... and they are ordered before the ticket
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(dst.ticket, 1u) == total - 1) {
            *dst.ticket = 0;         // for the next launch
            __threadfence_system();  // every block's stores, observed through its ticket, before the flags
            for (int r = 0; r < dst.count; ++r) *reinterpret_cast<volatile int *>(dst.flags[r] + dst.rank) = step;
            *reinterpret_cast<volatile int *>(dst.step) = step;
            __threadfence_system();
        }
    }
}

// Many tiles (large feature maps or batches): throughput matters more than latency.  One thread per
// (oc, tile) item keeps all 64 loads of M in flight at once and does both passes in registers; a warp
// covers 32 consecutive tiles of one output channel and stages its 6 x 192 results so that the stores
// run along the output rows.  No block-wide synchronisation.
constexpr int OTW_WARPS = 4;

template <bool ALONG_TILES, bool UPFRONT>
__global__ void __launch_bounds__(32 * OTW_WARPS, UPFRONT ? 4 : 1) output_transform_wide_kernel(const float *__restrict__ M,
                                                                              float *__restrict__ out, int n_tiles,
                                                                              int oc, int tp, int oh, int ow, int th,
                                                                              int tw, Epilogue ep) {
    constexpr int ROW = 32 * 6 + 2;
    __shared__ float stage[OTW_WARPS][6][ROW];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the warps of a block: OTW_WARPS channels of the same 32 tiles, or one channel of 32 * OTW_WARPS consecutive tiles
    const int t_base = ALONG_TILES ? (blockIdx.x * OTW_WARPS + warp) * 32 : blockIdx.x * 32;
    const int t = t_base + lane, k = ALONG_TILES ? blockIdx.y : blockIdx.y * OTW_WARPS + warp;
    const size_t plane = (size_t)oc * tp;
    pdl_trigger();
    pdl_wait();  // M comes from the GEMM launched just before
    if (k >= oc) return;  // whole warp
    if (t < n_tiles) {
        const float *src = M + (size_t)k * tp + t;
        float h[8][6];
        if constexpr (UPFRONT) {
            // all 64 values of the item requested before the first is used: the kernel lives on loads in flight
            float m[8][8];
#pragma unroll
            for (int row = 0; row < 8; ++row)
#pragma unroll
                for (int col = 0; col < 8; ++col) m[row][col] = __ldg(src + (size_t)(col * 8 + row) * plane);
#pragma unroll
            for (int row = 0; row < 8; ++row)
                output_transform_1d(m[row][0], m[row][1], m[row][2], m[row][3], m[row][4], m[row][5], m[row][6], m[row][7], h[row]);
        } else {
#pragma unroll
            for (int row = 0; row < 8; ++row) {
                float m[8];
#pragma unroll
                for (int col = 0; col < 8; ++col) m[col] = __ldg(src + (size_t)(col * 8 + row) * plane);
                output_transform_1d(m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], h[row]);
            }
        }
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            float s[6];
            output_transform_1d(h[0][j], h[1][j], h[2][j], h[3][j], h[4][j], h[5][j], h[6][j], h[7][j], s);
#pragma unroll
            for (int i = 0; i < 6; ++i) stage[warp][i][lane * 6 + j] = s[i];
        }
    }
    // every lane decodes the origin of ITS tile once; the store loop below fetches the origin of the tile an element
    // belongs to by shuffle instead of dividing again
    int my_org = -1;  // y0 << 16 | x0 of the tile's first output, -1 past the end
    size_t my_base = 0;
    if (t < n_tiles) {
        const int per_img = th * tw;
        const int img = t / per_img, tt = t - img * per_img;
        my_org = ((tt / tw) * 6) << 16 | ((tt % tw) * 6);
        my_base = ((size_t)img * oc + k) * oh * ow;
    }
    __syncwarp();
    // lane writes elements e = lane, lane+32, ... of every staged row: e -> (tile e/6, column e%6)
#pragma unroll
    for (int it = 0; it < 6; ++it) {
        const int e = lane + it * 32;
        const int te = e / 6, j = e - te * 6;
        const int org = __shfl_sync(0xffffffffu, my_org, te);
        const size_t base = __shfl_sync(0xffffffffu, my_base, te);
        if (org < 0) continue;
        const int y0 = org >> 16, x = (org & 0xffff) + j;
        if (x >= ow) continue;
        float *dst = out + base + (size_t)y0 * ow + x;
#pragma unroll
        for (int i = 0; i < 6; ++i)
            if (y0 + i < oh) dst[(size_t)i * ow] = ep(stage[warp][i][e], k);
    }
}

// ---------------------------------------------------------------------------------------------
// Layers with at most 4 input channels (the first layer of an image network): the TensorGEMM costs 64 x ic fused
// multiply-adds per (output channel, tile) item, far less than writing the item's 64 values of M and reading them
// back.  So the output transform computes them itself, straight from U[p][ic][ocp] and V[p][ic][tp], with the
// same chain as the TensorGEMM (one accumulator from +0, one fused multiply-add per input channel in ascending order:
// bit-identical values of M), and M never exists in memory.
//
// A block owns 32 consecutive tiles x FUSED_OCC output channels.  Its slice of the filter sits in shared memory as one
// float4 (channels 0..3, zero past ic) per (position, output channel), its slab of V as [position, channel][tile]; a
// thread owns one tile and two output channels at a time, so that every value of V read feeds two chains.  The rest is
// output_transform_wide_kernel.
// ---------------------------------------------------------------------------------------------
constexpr int FUSED_OCC = 16, FUSED_WARPS = 4;

template <int IC, bool EPI>
__global__ void __launch_bounds__(32 * FUSED_WARPS, 3) output_transform_fused_gemm_kernel(
    const float *__restrict__ U, const float *__restrict__ V, float *__restrict__ out, int n_tiles, int oc, int ocp,
    int icp, int tp, int oh, int ow, int th, int tw, Epilogue ep) {
    constexpr int ROW = 32 * 6 + 2, THREADS = 32 * FUSED_WARPS;
    extern __shared__ __align__(16) float fused_smem[];
    float4(*s_u)[FUSED_OCC] = reinterpret_cast<float4(*)[FUSED_OCC]>(fused_smem);
    float(*s_v)[32] = reinterpret_cast<float(*)[32]>(fused_smem + 64 * FUSED_OCC * 4);  // [p * IC + c][tile of the block]
    float(*stage)[6][ROW] = reinterpret_cast<float(*)[6][ROW]>(fused_smem + 64 * FUSED_OCC * 4 + 64 * IC * 32);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 32 + lane, k_base = blockIdx.y * FUSED_OCC;
    // Both operand slices travel through registers with every load in flight at once: the filter's first (it does not
    // depend on the preceding kernel), then, after the wait for the input transform, the slab of V; only then are they
    // parked in shared memory -- one round trip to memory per block.
    constexpr int P_STEP = THREADS / FUSED_OCC;  // positions covered by one sweep of the block over the filter
    constexpr int ROWS = 64 / FUSED_WARPS * IC;  // rows of V per warp: warp w brings positions [16w, 16w + 16)
    const int kl = threadIdx.x % FUSED_OCC, p0 = threadIdx.x / FUSED_OCC;
    float u[64 / P_STEP][4], v[ROWS];
    {
        const int k = k_base + kl;
        const float *ub = U + (size_t)p0 * icp * ocp + k;
#pragma unroll
        for (int i = 0; i < 64 / P_STEP; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                u[i][c] = c < IC && k < oc ? __ldg(ub + ((size_t)(i * P_STEP) * icp + c) * ocp) : 0.f;
    }
    pdl_trigger();
    pdl_wait();
    {
        const float *vb = V + (size_t)(warp * (64 / FUSED_WARPS)) * icp * tp + t;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) v[i] = t < n_tiles ? __ldg(vb + ((size_t)(i / IC) * icp + i % IC) * tp) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 64 / P_STEP; ++i)
        s_u[p0 + i * P_STEP][kl] = make_float4(u[i][0], u[i][1], u[i][2], u[i][3]);
#pragma unroll
    for (int i = 0; i < ROWS; ++i) s_v[warp * ROWS + i][lane] = v[i];
    __syncthreads();

    // Where this lane stores: element e = lane + 32*it of every staged row belongs to tile e/6, column e%6.  None of it
    // depends on the output channel, so it is worked out once: offset inside a channel's page, image, valid rows.
    const size_t out_page = (size_t)oh * ow;
    int st_off[6], st_img[6], st_rows[6];
    {
        int my_org = -1, my_img = 0;  // y0 << 16 | x0 of the tile's first output, -1 past the end
        if (t < n_tiles) {
            const int per_img = th * tw;
            const int img = t / per_img, tt = t - img * per_img;
            my_org = ((tt / tw) * 6) << 16 | ((tt % tw) * 6);
            my_img = img;
        }
#pragma unroll
        for (int it = 0; it < 6; ++it) {
            const int e = lane + it * 32;
            const int te = e / 6, j = e - te * 6;
            const int org = __shfl_sync(0xffffffffu, my_org, te);
            st_img[it] = __shfl_sync(0xffffffffu, my_img, te);
            const int y0 = org >> 16, x = (org & 0xffff) + j;
            st_off[it] = y0 * ow + x;
            st_rows[it] = org < 0 || x >= ow ? 0 : min(6, oh - y0);
        }
    }
    constexpr int PER_WARP = FUSED_OCC / FUSED_WARPS;
#pragma unroll 1
    for (int pair = 0; pair < PER_WARP / 2; ++pair) {
        const int kl0 = warp * PER_WARP + pair * 2, k0 = k_base + kl0;
        if (k0 >= oc) break;  // whole warp
        float h0[8][6], h1[8][6];
#pragma unroll
        for (int row = 0; row < 8; ++row) {
            float m0[8], m1[8];
#pragma unroll
            for (int col = 0; col < 8; ++col) {
                const int p = col * 8 + row;
                const float4 u0 = s_u[p][kl0], u1 = s_u[p][kl0 + 1];
                const float a0[4] = {u0.x, u0.y, u0.z, u0.w}, a1[4] = {u1.x, u1.y, u1.z, u1.w};
                float x0 = 0.f, x1 = 0.f;
#pragma unroll
                for (int c = 0; c < IC; ++c) {
                    const float v = s_v[p * IC + c][lane];
                    x0 = __fmaf_rn(a0[c], v, x0);
                    x1 = __fmaf_rn(a1[c], v, x1);
                }
                m0[col] = x0;
                m1[col] = x1;
            }
            output_transform_1d(m0[0], m0[1], m0[2], m0[3], m0[4], m0[5], m0[6], m0[7], h0[row]);
            output_transform_1d(m1[0], m1[1], m1[2], m1[3], m1[4], m1[5], m1[6], m1[7], h1[row]);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int k = k0 + half;
            if (k >= oc) break;  // whole warp
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                float s[6];
                if (half == 0)
                    output_transform_1d(h0[0][j], h0[1][j], h0[2][j], h0[3][j], h0[4][j], h0[5][j], h0[6][j], h0[7][j], s);
                else
                    output_transform_1d(h1[0][j], h1[1][j], h1[2][j], h1[3][j], h1[4][j], h1[5][j], h1[6][j], h1[7][j], s);
#pragma unroll
                for (int i = 0; i < 6; ++i) stage[warp][i][lane * 6 + j] = s[i];
            }
            __syncwarp();
            float b = 0.f;
            if (EPI && ep.bias != nullptr) b = __ldg(ep.bias + k);
#pragma unroll
            for (int it = 0; it < 6; ++it) {
                float *dst = out + ((size_t)st_img[it] * oc + k) * out_page + st_off[it];
#pragma unroll
                for (int i = 0; i < 6; ++i) {
                    if (i >= st_rows[it]) break;
                    float v = stage[warp][i][lane + it * 32];
                    if (EPI) {
                        if (ep.bias != nullptr) v = __fadd_rn(v, b);
                        if (ep.relu) v = fmaxf(v, 0.0f);
                    }
                    dst[(size_t)i * ow] = v;
                }
            }
            __syncwarp();  // the staged rows are free again
        }
    }
}

// ---------------------------------------------------------------------------------------------
// fp16 copy of the packed filter (FC_MATH_TF32_U16).  Per position p the largest magnitude picks a power of two 2^e
// with max|U_p| / 2^e in [2^13, 2^14): every value is divided by it (exact) and rounded to fp16, which keeps TF32's 11
// significant bits for everything within 2^-27 of the largest value; the scale goes into scales[p] and is multiplied
// back onto the accumulator.  The boxes keep their order and shape (128 channels x 32 input channels, now 8 KB).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) filter_u16_max_kernel(const float *__restrict__ U, unsigned *__restrict__ maxbits,
                                                             size_t per_pos) {
    const int p = blockIdx.y;
    const float *src = U + (size_t)p * per_pos;
    float m = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_pos; i += (size_t)gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(src[i]));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(maxbits + p, __float_as_uint(m));  // non-negative floats order like their bits
}

__global__ void __launch_bounds__(256) filter_u16_convert_kernel(const float *__restrict__ U, __half *__restrict__ H,
                                                                 float *__restrict__ scales,
                                                                 const unsigned *__restrict__ maxbits, size_t per_pos) {
    const int p = blockIdx.y;
    const float mx = __uint_as_float(maxbits[p]);
    int e = 0;
    if (mx > 0.0f) {
        frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1)
        e -= 14;         // mx / 2^e in [2^13, 2^14)
    }
    const float inv = ldexpf(1.0f, -e);
    if (blockIdx.x == 0 && threadIdx.x == 0) scales[p] = ldexpf(1.0f, e);
    const float *src = U + (size_t)p * per_pos;
    __half *dst = H + (size_t)p * per_pos;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_pos; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __float2half_rn(src[i] * inv);
}

// the fp16 boxes, then 64 scales, then 64 words the maxima are gathered in
size_t filter_u16_floats(const WinoGeom &g) { return (size_t)64 * g.n_ocb * g.n_kb * U_BOX_ELEMS / 2 + 128; }

int launch_filter_to_u16(fc_context *ctx, const float *d_U32, float *d_U16, const WinoGeom &g) {
    const size_t per_pos = (size_t)g.n_ocb * g.n_kb * U_BOX_ELEMS;
    float *scales = const_cast<float *>(filter_u16_scales(d_U16, g));
    unsigned *maxbits = reinterpret_cast<unsigned *>(scales + 64);
    FC_CHECK_CUDA(cudaMemsetAsync(maxbits, 0, 64 * sizeof(unsigned), ctx->stream));
    const unsigned blocks = (unsigned)(ceil_div(per_pos, 256) > 64 ? 64 : ceil_div(per_pos, 256));
    filter_u16_max_kernel<<<dim3(blocks, 64), 256, 0, ctx->stream>>>(d_U32, maxbits, per_pos);
    filter_u16_convert_kernel<<<dim3(blocks, 64), 256, 0, ctx->stream>>>(d_U32, reinterpret_cast<__half *>(d_U16), scales,
                                                                        maxbits, per_pos);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// tile count from which the throughput-oriented output transform is taken ($FASTCONV_OT_WIDE_MIN overrides it)
static int wide_min_tiles() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("FASTCONV_OT_WIDE_MIN");
        v = e && atoi(e) > 0 ? atoi(e) : 64;  // measured on 8 images: 200 tiles 25 -> 16 us, 72 tiles 14 -> 12 us
    }
    return v;
}

int launch_output_transform(fc_context *ctx, const float *d_M, float *d_out, const WinoGeom &g, const Epilogue &ep) {
    dim3 block(256);
    if (g.tiles >= wide_min_tiles()) {
        dim3 wblock(32 * OTW_WARPS);
        static const bool upfront_off = getenv("FASTCONV_OT_UPFRONT") && atoi(getenv("FASTCONV_OT_UPFRONT")) == 0;
        const bool upfront = !upfront_off && (size_t)g.tiles * g.oc >= 512 * 1024;
        if (g.tiles >= 32 * OTW_WARPS) {  // four warps along the tile axis: reads of 512 bytes per position (1 % faster)
            dim3 grid((unsigned)ceil_div(g.tiles, 32 * OTW_WARPS), (unsigned)g.oc);
            FC_CHECK_CUDA(launch_pdl(upfront ? output_transform_wide_kernel<true, true> : output_transform_wide_kernel<true, false>,
                                     grid, wblock, 0, ctx->stream, d_M, d_out, g.tiles, g.oc, g.tp, g.oh, g.ow, g.th, g.tw, ep));
        } else {
            dim3 grid((unsigned)ceil_div(g.tiles, 32), (unsigned)ceil_div(g.oc, OTW_WARPS));
            FC_CHECK_CUDA(launch_pdl(output_transform_wide_kernel<false, false>, grid, wblock, 0, ctx->stream, d_M, d_out, g.tiles,
                                     g.oc, g.tp, g.oh, g.ow, g.th, g.tw, ep));
        }
        return FC_OK;
    }
    if (g.tiles > 16) {
        dim3 grid((unsigned)ceil_div(g.tiles, 32), (unsigned)g.oc);
        FC_CHECK_CUDA(launch_pdl(output_transform_kernel<32>, grid, block, 0, ctx->stream, d_M, d_out, g.tiles, g.oc, g.tp,
                                 g.oh, g.ow, g.th, g.tw, ep));
    } else if (g.tiles > 8) {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 2));
        FC_CHECK_CUDA(launch_pdl(output_transform_kernel<16>, grid, block, 0, ctx->stream, d_M, d_out, g.tiles, g.oc, g.tp,
                                 g.oh, g.ow, g.th, g.tw, ep));
    } else {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 4));
        FC_CHECK_CUDA(launch_pdl(output_transform_kernel<8>, grid, block, 0, ctx->stream, d_M, d_out, g.tiles, g.oc, g.tp,
                                 g.oh, g.ow, g.th, g.tw, ep));
    }
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

bool output_transform_can_fuse_gemm(const WinoGeom &g) { return g.ic <= 4 && g.tiles >= 32; }

int launch_output_transform_fused_gemm(fc_context *ctx, const float *d_U, const float *d_V, float *d_out,
                                       const WinoGeom &g, const Epilogue &ep) {
    FC_REQUIRE(output_transform_can_fuse_gemm(g), FC_ERR_UNSUPPORTED, "fused TensorGEMM: %d input channels, %d tiles",
               g.ic, g.tiles);
    dim3 block(32 * FUSED_WARPS), grid((unsigned)ceil_div(g.tiles, 32), (unsigned)ceil_div(g.oc, FUSED_OCC));
    const size_t smem = sizeof(float) * (64 * FUSED_OCC * 4 + 64 * (size_t)g.ic * 32 + FUSED_WARPS * 6 * (32 * 6 + 2));
    auto go = [&](auto kern) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        return launch_pdl(kern, grid, block, smem, ctx->stream, d_U, d_V, d_out, g.tiles, g.oc, g.ocp, g.icp, g.tp, g.oh,
                          g.ow, g.th, g.tw, ep);
    };
    const bool epi = ep.bias != nullptr || ep.relu;
    switch (g.ic) {
        case 1: FC_CHECK_CUDA(epi ? go(output_transform_fused_gemm_kernel<1, true>) : go(output_transform_fused_gemm_kernel<1, false>)); break;
        case 2: FC_CHECK_CUDA(epi ? go(output_transform_fused_gemm_kernel<2, true>) : go(output_transform_fused_gemm_kernel<2, false>)); break;
        case 3: FC_CHECK_CUDA(epi ? go(output_transform_fused_gemm_kernel<3, true>) : go(output_transform_fused_gemm_kernel<3, false>)); break;
        default: FC_CHECK_CUDA(epi ? go(output_transform_fused_gemm_kernel<4, true>) : go(output_transform_fused_gemm_kernel<4, false>)); break;
    }
    return FC_OK;
}

int launch_output_transform_scatter(fc_context *ctx, const float *d_M, const PeerOuts &dst, const WinoGeom &g,
                                    const Epilogue &ep) {
    dim3 block(256);
    if (g.tiles > 16) {
        dim3 grid((unsigned)ceil_div(g.tiles, 32), (unsigned)g.oc);
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_kernel<32>, grid, block, 0, ctx->stream, d_M, dst, g.tiles, g.oc,
                                 g.tp, g.oh, g.ow, g.th, g.tw, ep));
    } else if (g.tiles > 8) {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 2));
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_kernel<16>, grid, block, 0, ctx->stream, d_M, dst, g.tiles, g.oc,
                                 g.tp, g.oh, g.ow, g.th, g.tw, ep));
    } else {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 4));
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_kernel<8>, grid, block, 0, ctx->stream, d_M, dst, g.tiles, g.oc,
                                 g.tp, g.oh, g.ow, g.th, g.tw, ep));
    }
    return FC_OK;
}

int launch_output_transform_scatter_publish(fc_context *ctx, const float *d_M, const ScatterPublish &dst,
                                            const WinoGeom &g, const Epilogue &ep) {
    dim3 block(256);
    if (g.tiles > 16) {
        dim3 grid((unsigned)ceil_div(g.tiles, 32), (unsigned)g.oc);
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_publish_kernel<32>, grid, block, 0, ctx->stream, d_M, dst, g.tiles,
                                 g.oc, g.tp, g.oh, g.ow, g.th, g.tw, ep));
    } else if (g.tiles > 8) {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 2));
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_publish_kernel<16>, grid, block, 0, ctx->stream, d_M, dst, g.tiles,
                                 g.oc, g.tp, g.oh, g.ow, g.th, g.tw, ep));
    } else {
        dim3 grid(1, (unsigned)ceil_div(g.oc, 4));
        FC_CHECK_CUDA(launch_pdl(output_transform_scatter_publish_kernel<8>, grid, block, 0, ctx->stream, d_M, dst, g.tiles,
                                 g.oc, g.tp, g.oh, g.ow, g.th, g.tw, ep));
    }
    return FC_OK;
}

}  // namespace fc
