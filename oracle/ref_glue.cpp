/*
 * TEST INFRASTRUCTURE ONLY -- C entry points around the UNMODIFIED FastConv
 * reference sources, compiled where they lie (see oracle/Makefile) into
 * oracle/_ref/libfastconv_ref.so.  Only tests/, __graft_entry__.smoke() and
 * bench.py's CPU-baseline / reference arm may load that library; the product
 * library never links or calls it.
 *
 * What each entry point drives (paths are relative to the reference tree):
 *   ref_wino_f63_forward   -> winoF63_v1_multi            winoF63ZC/winoF63ZC.cpp:988
 *                             (buffer sizing as ConvWinoF63ZCLayer::Init,
 *                              convLayer/winoF63ConvZC.cpp:176-213)
 *   ref_naive_conv3x3      -> ConvNaiveLayer::Forward     convLayer/naiveConv.h:24-64
 *   ref_im2col / _v1       -> ConvIm2colLayer::im2col()   convLayer/im2colConv.cpp:285-309
 *                             ConvIm2colLayer::im2col_v1()                      :311-382
 *   ref_im2col_sgemm       -> ConvIm2colLayer::Init(), im2col_v1(), sgemm()
 *                             convLayer/im2colConv.cpp:224-235, 311-382, 384-398: GEMM_v2 (:434-565) with the
 *                             8x8 register kernel for one thread, GEMM_multithread (:568-703) for more, the
 *                             scalar GEMM (:400-432) when M, N, K <= 32
 *   ref_diff               -> diff()                      utility/helper.cpp:74-89
 *
 * The Winograd driver is called with tileRegBlock = 5, ocRegBlock = 4 and
 * num_threads > 1 semantics (winoF63_v1_multi): that combination binds only the
 * intrinsic micro-kernels TensorGEMMInnerKernel4x{1..4}x5_v1
 * (winoF63ZC/winoF63ZC.cpp:1043-1053); the tileRegBlock = 4 and single-thread
 * drivers bind aarch64 assembly kernels that cannot run on this host.
 */
#include <stdlib.h>
#include <string.h>
#include <omp.h>

/* Timer keeps its millisecond accumulator private; the stage split is read from it below */
#define private public
#include "utility/helper.h"
#undef private
#include "conv_layer.h"
#include "convLayer/naiveConv.h"
#include "convLayer/im2colConv.h"
#include "winoF63ZC/winoF63ZC.h"
#include "utility/common.h"
#include "utility/helper.h"

namespace {

/* reaches the protected gather buffer of the reference im2col layer */
class Im2colProbe : public ConvIm2colLayer {
public:
    using ConvIm2colLayer::ConvIm2colLayer;
    float *gathered() { return transform_input_data; }
};

}  // namespace

extern "C" {

int ref_host_is_shim(void) { return 1; }

/*
 * One Winograd F(6x6,3x3) forward of the reference, online filter transform
 * (scheduling 0).  stage_ms (may be NULL) receives InputTran, KernelTran,
 * TensorGEMM, OutputTran accumulated milliseconds of this call.
 */
int ref_wino_f63_forward(float *out, const float *in, const float *kernel, int ic, int oc, int ih, int iw,
                         int pad, int threads, int tile_block, int oc_block, int ic_block, double *stage_ms) {
    const int tile_reg = 5, oc_reg = 4;
    if (tile_block % tile_reg != 0 || oc_block % oc_reg != 0 || threads < 1) return -1;
    const int oh = ih + 2 * pad - 2, ow = iw + 2 * pad - 2;
    if (oh < 1 || ow < 1) return -1;
    const int tile_n = ((oh + 5) / 6) * ((ow + 5) / 6);
    omp_set_num_threads(threads);

    const size_t in_buf_n = (size_t)64 * ic_block * align_ceil(tile_n, tile_reg) + 64;
    const size_t gemm_buf_n = (size_t)64 * oc * align_ceil(tile_n, tile_reg) + 64;
    const size_t k_buf_n = (size_t)64 * ic_block * align_ceil(oc, oc_block) + 128;
    float *in_buf = (float *)_mm_malloc(in_buf_n * sizeof(float));
    float *gemm_buf = (float *)_mm_malloc(gemm_buf_n * sizeof(float));
    float *k_buf = (float *)_mm_malloc(k_buf_n * sizeof(float));
    /* the reference reads one float past each 3x3 filter (vld1q at +6) */
    float *k_copy = (float *)malloc(((size_t)oc * ic * 9 + 16) * sizeof(float));
    float *in_copy = (float *)malloc((size_t)ic * ih * iw * sizeof(float));
    if (!in_buf || !gemm_buf || !k_buf || !k_copy || !in_copy) return -2;
    memset(gemm_buf, 0, gemm_buf_n * sizeof(float));
    memset(in_buf, 0, in_buf_n * sizeof(float));
    memset(k_buf, 0, k_buf_n * sizeof(float));
    memset(k_copy, 0, ((size_t)oc * ic * 9 + 16) * sizeof(float));
    memcpy(k_copy, kernel, (size_t)oc * ic * 9 * sizeof(float));
    memcpy(in_copy, in, (size_t)ic * ih * iw * sizeof(float));

    Timer t_in, t_k, t_gemm, t_out;
    winoF63_v1_multi(out, in_copy, k_copy, ic, oc, ih, iw, pad, pad, 1, 1, tile_block, gemm_buf, oc_block, k_buf,
                     ic_block, in_buf, tile_reg, oc_reg, /*scheduling=*/0, threads, t_in, t_k, t_gemm, t_out);
    if (stage_ms) {
        stage_ms[0] = t_in.accumulate;
        stage_ms[1] = t_k.accumulate;
        stage_ms[2] = t_gemm.accumulate;
        stage_ms[3] = t_out.accumulate;
    }
    _mm_free(in_buf);
    _mm_free(gemm_buf);
    _mm_free(k_buf);
    free(k_copy);
    free(in_copy);
    return 0;
}

/* 3x3 stride-1 direct convolution exactly as the reference's self-check computes it */
int ref_naive_conv3x3(float *out, const float *in, const float *kernel, int ic, int oc, int ih, int iw, int pad) {
    ConvNaiveLayer layer((float *)in, (float *)kernel, NULL, NULL, ic, ih, iw, oc, 3, 3, 1, 1, pad, pad, pad, pad);
    layer.Forward();
    memcpy(out, layer.output_data, (size_t)oc * layer.get_output_height() * layer.get_output_width() * sizeof(float));
    return 0;
}

/* gathered matrix [ic*kh*kw][oh*ow]; which = 0 -> im2col(), 1 -> im2col_v1() */
int ref_im2col(float *gathered, const float *in, int ic, int ih, int iw, int kh, int kw, int sh, int sw, int pad_l,
               int pad_r, int pad_t, int pad_b, int which) {
    const size_t oc = 1;
    float *dummy_kernel = (float *)calloc((size_t)ic * kh * kw + 16, sizeof(float));
    if (!dummy_kernel) return -2;
    {
        Im2colProbe layer((float *)in, dummy_kernel, NULL, NULL, ic, ih, iw, oc, kh, kw, sh, sw, pad_l, pad_r, pad_t,
                          pad_b);
        if (which == 0)
            layer.im2col();
        else
            layer.im2col_v1();
        const size_t n = (size_t)ic * kh * kw * layer.get_output_height() * layer.get_output_width();
        memcpy(gathered, layer.gathered(), n * sizeof(float));
    }
    free(dummy_kernel);
    return 0;
}

/*
 * One forward of the reference's im2col layer: gather, then sgemm().  The reference never zeroes its
 * output and every register kernel computes C += A*B (im2col/gemm_kernel.cpp:350-400), so C is cleared
 * here first -- the one liberty taken.  Constructor defaults otherwise (mc 8, nc 256, kc 384, 8x8 kernel,
 * C in place; convLayer/im2colConv.h:16-18).  The register kernels run through their intrinsic branches:
 * the library is built from a copy of im2col/gemm_kernel.cpp and im2col/gemm_pack.cpp in which the one
 * line `#define __ARM_ASM` is blanked (oracle/Makefile), nothing else changed.
 */
int ref_im2col_sgemm(float *out, const float *in, const float *kernel, int ic, int oc, int ih, int iw, int kh, int kw,
                     int sh, int sw, int pad_l, int pad_r, int pad_t, int pad_b, int threads) {
    if (threads < 1) return -1;
    omp_set_num_threads(threads);
    Im2colProbe layer((float *)in, (float *)kernel, NULL, NULL, ic, ih, iw, oc, kh, kw, sh, sw, pad_l, pad_r, pad_t,
                      pad_b, 1, false, threads, 1);
    const size_t n = (size_t)oc * layer.get_output_height() * layer.get_output_width();
    layer.Init();
    memset(layer.output_data, 0, (n + 128) * sizeof(float));
    layer.im2col_v1();
    layer.sgemm();
    memcpy(out, layer.output_data, n * sizeof(float));
    return 0;
}

float ref_diff(const float *a, const float *b, int len) { return diff((float *)a, (float *)b, len); }

}  // extern "C"
