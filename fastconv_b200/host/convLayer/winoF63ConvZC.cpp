#include "winoF63ConvZC.h"

ConvWinoF63ZCLayer::ConvWinoF63ZCLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic,
                                       size_t ih, size_t iw, size_t oc, size_t kh, size_t kw, size_t sh, size_t sw,
                                       size_t pad_left, size_t pad_right, size_t pad_top, size_t pad_bottom, size_t g,
                                       bool bias, size_t nt, size_t iter)
    : ConvLayer(input, kernel, biasw, output_ref, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top,
                pad_bottom, g, bias, nt, iter) {}

ConvWinoF63ZCLayer::~ConvWinoF63ZCLayer() {}

// The reference searches ARM cache-blocking sizes (ocBlock x tileBlock x icBlock x loop order,
// convLayer/winoF63ConvZC.cpp:25-174).  Here the search space is the library's kernel configurations,
// compared on measured device time.
int ConvWinoF63ZCLayer::Tuning() {
    plan(FC_ALGO_WINOGRAD);
    if (fc_conv_tune(conv, iterations > 0 ? (int)iterations : 1, 1) != FC_OK) {
        fprintf(stderr, "fastconv: %s\n", fc_last_error());
        exit(EXIT_FAILURE);
    }
    return -1;
}

int ConvWinoF63ZCLayer::Init() {
    printf("Algorithm: winograd F63\n");
    plan(FC_ALGO_WINOGRAD);
    print_testing_line();
    return -1;  // as convLayer/winoF63ConvZC.cpp:212
}

int ConvWinoF63ZCLayer::Forward() {
    run_iterations();
    printf("InputTran time: %lfms\n", (double)stage_ms[0]);
    printf("KernelTran time: %lfms\n", (double)stage_ms[1]);
    printf("TensorGEMM time: %lfms\n", (double)stage_ms[2]);
    printf("OutputTran time: %lfms\n", (double)stage_ms[3]);
    printf("Total time: %lfms\n", (double)stage_ms[4]);
    if (output_ref != NULL) diff(output_ref, output_data, (int)output_elems());
    return 1;
}
