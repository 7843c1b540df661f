// Winograd F(6x6,3x3) transform kernels: filter (one-time), input, output.
//
// The arithmetic mirrors FastConv's NEON transforms operation by operation so
// that, together with the sequential-FMA TensorGEMM, the whole layer is
// bit-identical to the reference: every multiply and add below is an explicit
// round-to-nearest intrinsic (the compiler may not contract them into FMAs),
// and __fmaf_rn appears exactly where the reference issues vfmaq_f32.
//
// Layouts (ic contiguous, padded with zeros to icp = roundup(ic, 8)):
//   U[p][oc][icp]   V[p][tp][icp]   M[p][oc][tp]     p = col*8 + row
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
// (offline_kernel_transform_v1, winoF63ZC/winoF63ZC.cpp:286-297).  One thread per (oc, ic);
// threads of a warp walk ic so the 64 stores per thread are coalesced.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) filter_transform_kernel(const float *__restrict__ kernel,
                                                               float *__restrict__ U, int oc, int ic, int icp) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int k = blockIdx.y;
    if (c >= icp) return;
    const size_t plane = (size_t)oc * icp;
    float *dst = U + (size_t)k * icp + c;
    if (c >= ic) {  // zero padding of the reduction axis
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

int launch_filter_transform(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic, int icp) {
    dim3 block(128), grid((unsigned)ceil_div(icp, 128), (unsigned)oc);
    filter_transform_kernel<<<grid, block, 0, ctx->stream>>>(d_kernel, d_U, oc, ic, icp);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// ---------------------------------------------------------------------------------------------
// Input transform: V = B^T d B per 8x8 tile at (6*ty - pad, 6*tx - pad), zero outside the image
// (winoF63ZC/winoF63ZC.cpp:541-612); B^T over the tile rows first, then the columns (:614-630).
//
// A block owns 8 consecutive tiles x 32 consecutive channels.  Phase 1 stages the 8x8 windows into
// shared memory with loads that run along the image rows (8 consecutive floats per lane group, four
// channels per warp instruction) -- zero-filled outside the image, past the last tile and past the
// last channel, so the padding of V falls out of the arithmetic.  Phase 2 gives every thread one
// (tile, channel): it reads its window with the channel as the fastest index (conflict-free), runs
// the two passes in registers and stores the 64 positions, each warp store being one 128-byte line
// of V[p][tile][c..c+31].
// ---------------------------------------------------------------------------------------------
constexpr int IT_TILES = 8;
constexpr int IT_CH = 32;
constexpr int IT_LD = IT_CH + 1;  // padded channel stride in shared memory

__global__ void __launch_bounds__(IT_CH * IT_TILES) input_transform_kernel(const float *__restrict__ in,
                                                                          float *__restrict__ V, int n_tiles, int ic,
                                                                          int icp, int tp, int ih, int iw, int pad,
                                                                          int th, int tw) {
    extern __shared__ float win[];  // [tile][y*8+x][channel (padded)]
    const int tid = threadIdx.x;
    const int c0 = blockIdx.x * IT_CH, t0 = blockIdx.y * IT_TILES;
    const int per_img = th * tw;

    {   // phase 1: lane group of 8 walks x, 32 groups walk the channels
        const int x = tid & 7, cl = tid >> 3;
        const int c = c0 + cl;
        const bool c_ok = c < ic;
#pragma unroll 1
        for (int t = 0; t < IT_TILES; ++t) {
            const int tile = t0 + t;
            const bool t_ok = c_ok && tile < n_tiles;
            const int img = tile / per_img, tt = tile - img * per_img;
            const int row0 = (tt / tw) * 6 - pad, col = (tt % tw) * 6 - pad + x;
            const float *src = in + ((size_t)img * ic + c) * ih * iw + col;
            const bool x_ok = t_ok && col >= 0 && col < iw;
            float v[8];
#pragma unroll
            for (int y = 0; y < 8; ++y) {
                const int yy = row0 + y;
                v[y] = (x_ok && yy >= 0 && yy < ih) ? __ldg(src + (size_t)yy * iw) : 0.0f;
            }
#pragma unroll
            for (int y = 0; y < 8; ++y) win[(t * 64 + y * 8 + x) * IT_LD + cl] = v[y];
        }
    }
    __syncthreads();

    const int lane = tid & 31, t = tid >> 5;
    const int c = c0 + lane, tile = t0 + t;
    if (c >= icp || tile >= tp) return;
    const float *w = win + (size_t)t * 64 * IT_LD + lane;
    float d[8][8];
#pragma unroll
    for (int y = 0; y < 8; ++y)
#pragma unroll
        for (int x = 0; x < 8; ++x) d[y][x] = w[(y * 8 + x) * IT_LD];
#pragma unroll
    for (int x = 0; x < 8; ++x)
        input_transform_1d(d[0][x], d[1][x], d[2][x], d[3][x], d[4][x], d[5][x], d[6][x], d[7][x]);
    const size_t plane = (size_t)tp * icp;
    float *dst = V + (size_t)tile * icp + c;
#pragma unroll
    for (int y = 0; y < 8; ++y) {
        input_transform_1d(d[y][0], d[y][1], d[y][2], d[y][3], d[y][4], d[y][5], d[y][6], d[y][7]);
#pragma unroll
        for (int x = 0; x < 8; ++x) dst[(size_t)(x * 8 + y) * plane] = d[y][x];
    }
}

int launch_input_transform(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g) {
    static bool attr_set = false;
    const size_t smem = (size_t)IT_TILES * 64 * IT_LD * sizeof(float);
    if (!attr_set) {
        FC_CHECK_CUDA(cudaFuncSetAttribute(input_transform_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    dim3 block(IT_CH * IT_TILES), grid((unsigned)ceil_div(g.icp, IT_CH), (unsigned)ceil_div(g.tp, IT_TILES));
    input_transform_kernel<<<grid, block, smem, ctx->stream>>>(d_in, d_V, g.tiles, g.ic, g.icp, g.tp, g.ih, g.iw, g.pad,
                                                               g.th, g.tw);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

// ---------------------------------------------------------------------------------------------
// Output transform: Y = A^T M A, A^T over the tile columns first (for every row), then over the
// rows (winoF63ZC/winoF63ZC.cpp:905-912), clipped store at the right/bottom edges (:928-969).
//
// One thread per (oc, tile).  A warp covers TPW consecutive tiles of 32/TPW output channels (TPW =
// 32, 16 or 8, chosen from the tile count so that small feature maps do not idle most lanes); the
// 64 loads per thread from M[p][oc][tile] are contiguous across the lanes of a channel.  The 6x6
// results go through shared memory so that the stores run along the output rows: tiles that are
// neighbours in x are neighbours in memory, so a warp writes runs of 6*TPW consecutive floats.
// ---------------------------------------------------------------------------------------------
constexpr int OT_WARPS = 4;

template <int TPW>
__global__ void __launch_bounds__(32 * OT_WARPS) output_transform_kernel(const float *__restrict__ M,
                                                                        float *__restrict__ out, int n_tiles, int oc,
                                                                        int tp, int oh, int ow, int th, int tw) {
    constexpr int OCW = 32 / TPW;            // output channels per warp
    constexpr int ROW = TPW * 6 + 2;         // floats per staged output row (+2: fewer bank conflicts)
    __shared__ float stage[OT_WARPS][OCW][6][ROW];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tl = lane % TPW, ol = lane / TPW;
    const int t_base = blockIdx.x * TPW;
    const int k_base = (blockIdx.y * OT_WARPS + warp) * OCW;
    const int t = t_base + tl, k = k_base + ol;
    const size_t plane = (size_t)oc * tp;
    const bool active = t < n_tiles && k < oc;
    if (active) {
        const float *src = M + (size_t)k * tp + t;
        float h[8][6];
#pragma unroll
        for (int row = 0; row < 8; ++row) {
            float m[8];
#pragma unroll
            for (int col = 0; col < 8; ++col) m[col] = __ldg(src + (size_t)(col * 8 + row) * plane);
            output_transform_1d(m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], h[row]);
        }
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            float s[6];
            output_transform_1d(h[0][j], h[1][j], h[2][j], h[3][j], h[4][j], h[5][j], h[6][j], h[7][j], s);
#pragma unroll
            for (int i = 0; i < 6; ++i) stage[warp][ol][i][tl * 6 + j] = s[i];
        }
    }
    __syncwarp();
    const int per_img = th * tw;
    // each lane now writes elements e = lane, lane+32, ... of every staged row: e -> (tile e/6, column e%6)
#pragma unroll 1
    for (int o = 0; o < OCW; ++o) {
        const int kk = k_base + o;
        if (kk >= oc) break;
        for (int e = lane; e < TPW * 6; e += 32) {
            const int te = e / 6, j = e - te * 6;
            const int tile = t_base + te;
            if (tile >= n_tiles) continue;
            const int img = tile / per_img, tt = tile - img * per_img;
            const int y0 = (tt / tw) * 6, x = (tt % tw) * 6 + j;
            if (x >= ow) continue;
            float *dst = out + ((size_t)img * oc + kk) * oh * ow + (size_t)y0 * ow + x;
#pragma unroll
            for (int i = 0; i < 6; ++i)
                if (y0 + i < oh) dst[(size_t)i * ow] = stage[warp][o][i][e];
        }
    }
}

int launch_output_transform(fc_context *ctx, const float *d_M, float *d_out, const WinoGeom &g) {
    dim3 block(32 * OT_WARPS);
    if (g.tiles > 16) {
        dim3 grid((unsigned)ceil_div(g.tiles, 32), (unsigned)ceil_div(g.oc, OT_WARPS));
        output_transform_kernel<32><<<grid, block, 0, ctx->stream>>>(d_M, d_out, g.tiles, g.oc, g.tp, g.oh, g.ow, g.th, g.tw);
    } else if (g.tiles > 8) {
        dim3 grid(1, (unsigned)ceil_div(g.oc, OT_WARPS * 2));
        output_transform_kernel<16><<<grid, block, 0, ctx->stream>>>(d_M, d_out, g.tiles, g.oc, g.tp, g.oh, g.ow, g.th, g.tw);
    } else {
        dim3 grid(1, (unsigned)ceil_div(g.oc, OT_WARPS * 4));
        output_transform_kernel<8><<<grid, block, 0, ctx->stream>>>(d_M, d_out, g.tiles, g.oc, g.tp, g.oh, g.ow, g.th, g.tw);
    }
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
