#include "im2colConv.h"

ConvIm2colLayer::ConvIm2colLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic, size_t ih,
                                 size_t iw, size_t oc, size_t kh, size_t kw, size_t sh, size_t sw, size_t pad_left,
                                 size_t pad_right, size_t pad_top, size_t pad_bottom, size_t g, bool bias, size_t nt,
                                 size_t iter, int, int, int, int, int, int, int, int, int, int, int)
    : ConvLayer(input, kernel, biasw, output_ref, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top,
                pad_bottom, g, bias, nt, iter),
      transform_input_data(NULL) {
    M = (int)output_channels;
    N = (int)(output_height * output_width);
    K = (int)(input_channels * kernel_height * kernel_width);
}

ConvIm2colLayer::~ConvIm2colLayer() { free(transform_input_data); }

int ConvIm2colLayer::Init() {
    printf("Algorithm: im2col\n");
    plan(FC_ALGO_IM2COL);
    return 1;  // as convLayer/im2colConv.cpp:234
}

int ConvIm2colLayer::Tuning() {
    plan(FC_ALGO_IM2COL);
    if (fc_conv_tune(conv, iterations > 0 ? (int)iterations : 1, 1) != FC_OK) {
        fprintf(stderr, "fastconv: %s\n", fc_last_error());
        exit(EXIT_FAILURE);
    }
    return 1;
}

int ConvIm2colLayer::Forward() {
    run_iterations();
    printf("Im2colTran time: %lfms\n", (double)stage_ms[0]);
    printf("Gemm time: %lfms\n", (double)stage_ms[2]);
    printf("Total time: %lfms\n", (double)stage_ms[4]);
    if (output_ref != NULL) diff(output_ref, output_data, (int)output_elems());
    return 1;
}

void ConvIm2colLayer::im2col() {
    plan(FC_ALGO_IM2COL);
    const size_t elems = (size_t)K * N;
    transform_input_data = (float *)realloc(transform_input_data, elems * sizeof(float));
    float *d_in = NULL, *d_out = NULL;
    void *d_b = NULL;
    fc_conv_device_buffers(conv, &d_in, &d_out);
    fc_conv_desc d = descriptor();
    if (fc_arena_alloc(ctx, elems * sizeof(float), &d_b) != FC_OK ||
        fc_memcpy_h2d(ctx, d_in, input_data, input_elems() * sizeof(float)) != FC_OK ||
        fc_im2col_gather(ctx, d_in, (float *)d_b, &d, 0) != FC_OK ||
        fc_memcpy_d2h(ctx, transform_input_data, d_b, elems * sizeof(float)) != FC_OK) {
        fprintf(stderr, "fastconv: %s\n", fc_last_error());
        exit(EXIT_FAILURE);
    }
    fc_arena_free(ctx, d_b);
}
