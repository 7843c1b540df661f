/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of FastConv's convolution hot path.
 *
 * This file is the checker the CUDA path is compared against.  Only tests/,
 * __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may load
 * it; the product library never links, calls or falls back to it.
 *
 * Parity pin: every function below is validated bit-for-bit against the
 * reference's own sources compiled on this host (oracle/_ref, see
 * oracle/Makefile) by tests/test_oracle_golden.py, and against the
 * golden vectors under tests/golden/ that were generated from that build.
 * The reference itself ships no tests, fixtures or known-answer vectors.
 *
 * All arithmetic is IEEE binary32, compiled with -ffp-contract=off so that a
 * multiply followed by an add stays two roundings, exactly like the separate
 * NEON vector operations of the reference; fmaf() marks the places where the
 * reference issues a fused multiply-add (vfmaq_f32).
 *
 * Citations are paths inside the reference tree.
 *
 * Winograd-domain layouts used here (chosen for the GPU, not the reference's
 * register-blocked panels; the values are the same):
 *   position p = col*8 + row of the 8x8 transformed tile, which equals the
 *   reference's depth*4 + lane with depth = 2*col + row/4, lane = row%4
 *   (store order winoF63ZC/winoF63ZC.cpp:632-647 and :293-313).
 *   U[p][oc][ic], V[p][tile][ic], M[p][oc][tile]; tile = n*tileH*tileW + ty*tileW + tx.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* 1-D transforms                                                             */
/* ------------------------------------------------------------------------- */

/* G (8x3) applied along one axis: winograd_f6k3_kernel_transform_v1,
 * winoF63ZC/winoF63ZC.cpp:14-79.  The scale constants are doubles narrowed to
 * float (vdupq_n_f32(-2.0/9) etc., :68-77). */
static void filter_transform_1d(const float g0, const float g1, const float g2, float w[8]) {
    const float f4 = 4.0f, f2 = 2.0f;
    float w2 = g0 + g2;
    float w4 = g0 + f4 * g2;
    float w6 = g2 + f4 * g0;
    const float two_g1 = g1 * f2;
    float w1 = w2 + g1;
    w2 = w2 - g1;
    float w3 = w4 + two_g1;
    w4 = w4 - two_g1;
    float w5 = w6 + two_g1;
    w6 = w6 - two_g1;
    const float c29 = (float)(-2.0 / 9);
    const float c90 = (float)(1.0 / 90);
    const float c180 = (float)(1.0 / 180);
    w[0] = g0;
    w[1] = w1 * c29;
    w[2] = w2 * c29;
    w[3] = w3 * c90;
    w[4] = w4 * c90;
    w[5] = w5 * c180;
    w[6] = w6 * c180;
    w[7] = g2;
}

/* B^T (8x8) applied along one axis: input_transform_v1,
 * winoF63ZC/winoF63ZC.cpp:112-169 (expression order and parenthesisation kept). */
static void input_transform_1d(float r[8]) {
    const float f5_25 = 5.25f, f4_25 = 4.25f, f4 = 4.0f, f2_5 = 2.5f, f2 = 2.0f, f1_25 = 1.25f, f0_5 = 0.5f,
                f0_25 = 0.25f;
    float r0 = r[0], r1 = r[1], r2 = r[2], r3 = r[3], r4 = r[4], r5 = r[5], r6 = r[6], r7 = r[7];
    float t1, t2, s1, s2, p1, p2;
    r0 = r0 - r6 + (r4 - r2) * f5_25;
    r7 = r7 - r1 + (r3 - r5) * f5_25;
    t1 = r2 + r6 - r4 * f4_25;
    t2 = r1 + r5 - r3 * f4_25;
    s1 = r4 * f1_25;
    s2 = r3 * f2_5;
    p1 = r6 + r2 * f0_25 - s1;
    p2 = r1 * f0_5 - s2 + r5 * f2;
    r3 = p1 + p2;
    r4 = p1 - p2;
    p1 = r6 + (r2 - s1) * f4;
    p2 = r1 * f2 - s2 + r5 * f0_5;
    r5 = p1 + p2;
    r6 = p1 - p2;
    r1 = t1 + t2;
    r2 = t1 - t2;
    r[0] = r0; r[1] = r1; r[2] = r2; r[3] = r3; r[4] = r4; r[5] = r5; r[6] = r6; r[7] = r7;
}

/* A^T (6x8) applied along one axis: winograd_f6k3_output_transform_inplace_v1,
 * winoF63ZC/winoF63ZC.cpp:171-228.  vfmaq_f32(a, b, c) = a + b*c fused. */
static void output_transform_1d(const float m[8], float s[6]) {
    const float a12 = m[1] + m[2], s12 = m[1] - m[2];
    const float a34 = m[3] + m[4], s34 = m[3] - m[4];
    const float a56 = m[5] + m[6], s56 = m[5] - m[6];
    float m0 = m[0] + a12;
    float m5 = m[7] + s12;
    float m1 = fmaf(16.0f, s56, s12);
    float m4 = fmaf(16.0f, a34, a12);
    float m2 = fmaf(8.0f, a56, a12);
    float m3 = fmaf(8.0f, s34, s12);
    m0 = fmaf(32.0f, a56, m0);
    m0 += a34;
    m5 = fmaf(32.0f, s34, m5);
    m5 += s56;
    m1 = fmaf(s34, 2.0f, m1);
    m4 = fmaf(a56, 2.0f, m4);
    m2 = fmaf(a34, 4.0f, m2);
    m3 = fmaf(s56, 4.0f, m3);
    s[0] = m0; s[1] = m1; s[2] = m2; s[3] = m3; s[4] = m4; s[5] = m5;
}

/* ------------------------------------------------------------------------- */
/* Winograd F(6x6,3x3) stages                                                 */
/* ------------------------------------------------------------------------- */

static int tiles_1d(int out) { return (out + 5) / 6; }

/* U = G g G^T.  Pass order as offline_kernel_transform_v1
 * (winoF63ZC/winoF63ZC.cpp:286-297): G over the filter rows first, then over
 * the filter columns.  kernel is [oc][ic][3][3]; U is [64][oc][ic_stride]. */
void oracle_wino_filter_transform(float *U, const float *kernel, int oc, int ic, int ic_stride) {
#pragma omp parallel for collapse(2)
    for (int k = 0; k < oc; ++k) {
        for (int c = 0; c < ic; ++c) {
            const float *g = kernel + ((size_t)k * ic + c) * 9;
            float gg[8][3]; /* (G g)[row][v] */
            for (int v = 0; v < 3; ++v) {
                float w[8];
                filter_transform_1d(g[0 * 3 + v], g[1 * 3 + v], g[2 * 3 + v], w);
                for (int r = 0; r < 8; ++r) gg[r][v] = w[r];
            }
            for (int r = 0; r < 8; ++r) {
                float w[8];
                filter_transform_1d(gg[r][0], gg[r][1], gg[r][2], w);
                for (int col = 0; col < 8; ++col)
                    U[((size_t)(col * 8 + r) * oc + k) * ic_stride + c] = w[col];
            }
        }
    }
}

/* V = B^T d B on 8x8 input tiles at (6*ty - pad, 6*tx - pad), zero outside the
 * image (winoF63ZC/winoF63ZC.cpp:541-612).  Pass order (:614-630): B^T over the
 * tile rows first, then over the tile columns.  in is [n][ic][ih][iw]; V is
 * [64][tile_stride][ic_stride]. */
void oracle_wino_input_transform(float *V, const float *in, int n, int ic, int ih, int iw, int pad, int tile_stride,
                                 int ic_stride) {
    const int oh = ih + 2 * pad - 2, ow = iw + 2 * pad - 2;
    const int th = tiles_1d(oh), tw = tiles_1d(ow);
#pragma omp parallel for collapse(2)
    for (int t = 0; t < n * th * tw; ++t) {
        for (int c = 0; c < ic; ++c) {
            const int img = t / (th * tw), tt = t % (th * tw);
            const int row0 = (tt / tw) * 6 - pad, col0 = (tt % tw) * 6 - pad;
            const float *src = in + ((size_t)img * ic + c) * ih * iw;
            float d[8][8];
            for (int y = 0; y < 8; ++y)
                for (int x = 0; x < 8; ++x) {
                    const int yy = row0 + y, xx = col0 + x;
                    d[y][x] = (yy >= 0 && yy < ih && xx >= 0 && xx < iw) ? src[(size_t)yy * iw + xx] : 0.0f;
                }
            for (int x = 0; x < 8; ++x) { /* rows */
                float r[8];
                for (int y = 0; y < 8; ++y) r[y] = d[y][x];
                input_transform_1d(r);
                for (int y = 0; y < 8; ++y) d[y][x] = r[y];
            }
            for (int y = 0; y < 8; ++y) { /* columns */
                float r[8];
                for (int x = 0; x < 8; ++x) r[x] = d[y][x];
                input_transform_1d(r);
                for (int x = 0; x < 8; ++x)
                    V[((size_t)(x * 8 + y) * tile_stride + t) * ic_stride + c] = r[x];
            }
        }
    }
}

/* M[p][oc][tile] = sum over ic ascending of U*V, one fused multiply-add per
 * step starting from 0 (TensorGEMMInnerKernel4x4x5_v1,
 * winoF63ZC/TensorGEMMZC.cpp:585-697; gemmBuf is zeroed before the call,
 * convLayer/winoF63ConvZC.cpp:230-232, and ic-blocks continue the same chain
 * through memory). */
void oracle_wino_gemm(float *M, const float *U, const float *V, int oc, int ic, int tiles, int ic_stride,
                      int tile_stride_v, int tile_stride_m) {
#pragma omp parallel for collapse(2)
    for (int p = 0; p < 64; ++p) {
        for (int k = 0; k < oc; ++k) {
            const float *u = U + ((size_t)p * oc + k) * ic_stride;
            for (int t = 0; t < tiles; ++t) {
                const float *v = V + ((size_t)p * tile_stride_v + t) * ic_stride;
                float acc = 0.0f;
                for (int c = 0; c < ic; ++c) acc = fmaf(u[c], v[c], acc);
                M[((size_t)p * oc + k) * tile_stride_m + t] = acc;
            }
        }
    }
}

/* Y = A^T M A, clipped at the right/bottom edges (winoF63ZC/winoF63ZC.cpp:869-973).
 * Pass order (:905-912): A^T over the tile columns first (for each row), then
 * over the rows.  out is [n][oc][oh][ow]. */
void oracle_wino_output_transform(float *out, const float *M, int n, int oc, int oh, int ow, int tile_stride_m) {
    const int th = tiles_1d(oh), tw = tiles_1d(ow);
#pragma omp parallel for collapse(2)
    for (int k = 0; k < oc; ++k) {
        for (int t = 0; t < n * th * tw; ++t) {
            const int img = t / (th * tw), tt = t % (th * tw);
            float m[8][8], h[8][6], y[6][6];
            for (int col = 0; col < 8; ++col)
                for (int row = 0; row < 8; ++row)
                    m[row][col] = M[((size_t)(col * 8 + row) * oc + k) * tile_stride_m + t];
            for (int row = 0; row < 8; ++row) output_transform_1d(m[row], h[row]);
            for (int j = 0; j < 6; ++j) {
                float colv[8], s[6];
                for (int row = 0; row < 8; ++row) colv[row] = h[row][j];
                output_transform_1d(colv, s);
                for (int i = 0; i < 6; ++i) y[i][j] = s[i];
            }
            const int y0 = (tt / tw) * 6, x0 = (tt % tw) * 6;
            float *dst = out + ((size_t)img * oc + k) * oh * ow;
            for (int i = 0; i < 6 && y0 + i < oh; ++i)
                for (int j = 0; j < 6 && x0 + j < ow; ++j) dst[(size_t)(y0 + i) * ow + x0 + j] = y[i][j];
        }
    }
}

/* Whole layer: the four stages above.  3x3, stride 1, symmetric padding -- the
 * only shape the reference's Winograd driver handles (it derives the output
 * size as ih + 2*pad - 2, winoF63ZC/winoF63ZC.cpp:334-338). */
int oracle_wino_forward(float *out, const float *in, const float *kernel, int n, int ic, int oc, int ih, int iw,
                        int pad) {
    const int oh = ih + 2 * pad - 2, ow = iw + 2 * pad - 2;
    if (oh < 1 || ow < 1 || n < 1 || ic < 1 || oc < 1) return -1;
    const int tiles = n * tiles_1d(oh) * tiles_1d(ow);
    float *U = (float *)malloc((size_t)64 * oc * ic * sizeof(float));
    float *V = (float *)malloc((size_t)64 * tiles * ic * sizeof(float));
    float *M = (float *)malloc((size_t)64 * oc * tiles * sizeof(float));
    if (!U || !V || !M) {
        free(U); free(V); free(M);
        return -2;
    }
    oracle_wino_filter_transform(U, kernel, oc, ic, ic);
    oracle_wino_input_transform(V, in, n, ic, ih, iw, pad, tiles, ic);
    oracle_wino_gemm(M, U, V, oc, ic, tiles, ic, tiles, tiles);
    oracle_wino_output_transform(out, M, n, oc, oh, ow, tiles);
    free(U); free(V); free(M);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* im2col + SGEMM path                                                        */
/* ------------------------------------------------------------------------- */

/* Gathered matrix B[(ic*kh + u)*kw + v][i*ow + j] = in[ic][i*sh + u - pad_t][j*sw + v - pad_l]
 * or 0 outside the image: ConvIm2colLayer::im2col, convLayer/im2colConv.cpp:285-309.
 * One image; returns the output size through oh/ow. */
void oracle_im2col(float *B, const float *in, int ic, int ih, int iw, int kh, int kw, int sh, int sw, int pad_l,
                   int pad_r, int pad_t, int pad_b, int *oh_out, int *ow_out) {
    const int ow = (iw + pad_l + pad_r - kw) / sw + 1;
    const int oh = (ih + pad_t + pad_b - kh) / sh + 1;
    if (oh_out) *oh_out = oh;
    if (ow_out) *ow_out = ow;
    size_t idx = 0;
    for (int c = 0; c < ic; ++c)
        for (int u = 0; u < kh; ++u)
            for (int v = 0; v < kw; ++v)
                for (int i = 0; i < oh; ++i)
                    for (int j = 0; j < ow; ++j) {
                        const int row = u - pad_t + i * sh, col = v - pad_l + j * sw;
                        B[idx++] = (row < 0 || row >= ih || col < 0 || col >= iw)
                                       ? 0.0f
                                       : in[((size_t)c * ih + row) * iw + col];
                    }
}

/* C[oc][pixel] = sum over k = (ic,u,v) ascending of A[oc][k] * B[k][pixel], one
 * fused multiply-add per k starting from C = 0.  This is the accumulation
 * order of the reference's register kernels (im2col/gemm_kernel.cpp:350-420,
 * `fmla` per k with C loaded first; kc blocks continue the chain through C,
 * convLayer/im2colConv.cpp:465-557).  When M = oc, N = oh*ow and K are all at
 * most 32 the reference runs its scalar GEMM instead (convLayer/im2colConv.h:30-31,
 * im2colConv.cpp:400-432): `C += temp * B`, a separate multiplication and
 * addition per k.  The reference never zeroes C (conv_layer.h:79); the
 * restatement starts from zero.  Bit-equal to the reference's sgemm() run
 * through oracle/_ref (tests/test_oracle_golden.py).
 * in is [n][ic][ih][iw], kernel [oc][ic][kh][kw], out [n][oc][oh][ow]. */
int oracle_im2col_gemm_forward(float *out, const float *in, const float *kernel, int n, int ic, int oc, int ih,
                               int iw, int kh, int kw, int sh, int sw, int pad_l, int pad_r, int pad_t, int pad_b) {
    const int ow = (iw + pad_l + pad_r - kw) / sw + 1;
    const int oh = (ih + pad_t + pad_b - kh) / sh + 1;
    if (oh < 1 || ow < 1) return -1;
    const int scalar_gemm = oc <= 32 && oh * ow <= 32 && ic * kh * kw <= 32;
#pragma omp parallel for collapse(2)
    for (int img = 0; img < n; ++img) {
        for (int k = 0; k < oc; ++k) {
            const float *a = kernel + (size_t)k * ic * kh * kw;
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    float acc = 0.0f;
                    for (int c = 0; c < ic; ++c) {
                        const float *src = in + ((size_t)img * ic + c) * ih * iw;
                        for (int u = 0; u < kh; ++u)
                            for (int v = 0; v < kw; ++v) {
                                const int row = u - pad_t + i * sh, col = v - pad_l + j * sw;
                                const float b = (row < 0 || row >= ih || col < 0 || col >= iw)
                                                    ? 0.0f
                                                    : src[(size_t)row * iw + col];
                                const float av = a[(c * kh + u) * kw + v];
                                acc = scalar_gemm ? acc + av * b : fmaf(av, b, acc);
                            }
                    }
                    out[(((size_t)img * oc + k) * oh + i) * ow + j] = acc;
                }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Direct convolutions                                                        */
/* ------------------------------------------------------------------------- */

/* The reference's own self-check convolution: per input channel a 9-term (or
 * kh*kw-term) partial sum `total`, then `sum += total`, all in binary32 with
 * separate multiply and add (convLayer/naiveConv.h:24-64,
 * convLayer/naiveConv_wudu.h:24-84). */
int oracle_naive_conv(float *out, const float *in, const float *kernel, int n, int ic, int oc, int ih, int iw,
                      int kh, int kw, int sh, int sw, int pad_l, int pad_r, int pad_t, int pad_b) {
    const int ow = (iw + pad_l + pad_r - kw) / sw + 1;
    const int oh = (ih + pad_t + pad_b - kh) / sh + 1;
    if (oh < 1 || ow < 1) return -1;
#pragma omp parallel for collapse(2)
    for (int img = 0; img < n; ++img) {
        for (int k = 0; k < oc; ++k) {
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    float sum = 0.0f;
                    for (int c = 0; c < ic; ++c) {
                        const float *src = in + ((size_t)img * ic + c) * ih * iw;
                        const float *g = kernel + ((size_t)k * ic + c) * kh * kw;
                        float total = 0.0f;
                        for (int u = 0; u < kh; ++u)
                            for (int v = 0; v < kw; ++v) {
                                const int row = u - pad_t + i * sh, col = v - pad_l + j * sw;
                                const float b = (row < 0 || row >= ih || col < 0 || col >= iw)
                                                    ? 0.0f
                                                    : src[(size_t)row * iw + col];
                                total += b * g[u * kw + v];
                            }
                        sum += total;
                    }
                    out[(((size_t)img * oc + k) * oh + i) * ow + j] = sum;
                }
        }
    }
    return 0;
}

/* Ground truth: the same convolution accumulated in binary64 (not a reference
 * function; used to report every path's distance from the exact result). */
int oracle_direct_conv_f64(double *out, const float *in, const float *kernel, int n, int ic, int oc, int ih, int iw,
                           int kh, int kw, int sh, int sw, int pad_l, int pad_r, int pad_t, int pad_b) {
    const int ow = (iw + pad_l + pad_r - kw) / sw + 1;
    const int oh = (ih + pad_t + pad_b - kh) / sh + 1;
    if (oh < 1 || ow < 1) return -1;
#pragma omp parallel for collapse(2)
    for (int img = 0; img < n; ++img) {
        for (int k = 0; k < oc; ++k) {
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    double acc = 0.0;
                    for (int c = 0; c < ic; ++c) {
                        const float *src = in + ((size_t)img * ic + c) * ih * iw;
                        const float *g = kernel + ((size_t)k * ic + c) * kh * kw;
                        for (int u = 0; u < kh; ++u) {
                            const int row = u - pad_t + i * sh;
                            if (row < 0 || row >= ih) continue;
                            for (int v = 0; v < kw; ++v) {
                                const int col = v - pad_l + j * sw;
                                if (col < 0 || col >= iw) continue;
                                acc += (double)src[(size_t)row * iw + col] * (double)g[u * kw + v];
                            }
                        }
                    }
                    out[(((size_t)img * oc + k) * oh + i) * ow + j] = acc;
                }
        }
    }
    return 0;
}

/* Mean absolute error over the elements whose error exceeds 1e-5, the figure
 * the reference prints as "The difference is" (utility/helper.cpp:74-89). */
float oracle_diff(const float *a, const float *b, int len) {
    int num = 0;
    double dif = 0.0;
    for (int i = 0; i < len; ++i) {
        const float err = fabsf(a[i] - b[i]);
        if (err > 1e-5f) {
            dif += err;
            ++num;
        }
    }
    return num == 0 ? 0.0f : (float)(dif / num);
}
