// Direct convolution layer for `-a direct`.  The reference parses the name but its case in main() is empty
// (ConvTest.cpp:369-371), so there is no class to mirror; this one follows the shape of the im2col layer
// (convLayer/im2colConv.h:9-53): same constructor arguments as ConvLayer, Init() and Forward() return 1.
// On the GPU it is the direct tensor-core kernel for ungrouped layers of stride 1 or 2 in the TF32 mode (shifted TMA boxes
// of an NHWC copy of the input, no Winograd transform); any other layer or mode runs as the implicit GEMM.
#ifndef DIRECTCONV_H
#define DIRECTCONV_H

#include "../conv_layer.h"

class ConvDirectLayer : public ConvLayer {
public:
    ConvDirectLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic, size_t ih, size_t iw,
                    size_t oc, size_t kh = 3, size_t kw = 3, size_t sh = 1, size_t sw = 1, size_t pad_left = 1,
                    size_t pad_right = 1, size_t pad_top = 1, size_t pad_bottom = 1, size_t g = 1, bool bias = 0,
                    size_t nt = 1, size_t iter = 10)
        : ConvLayer(input, kernel, biasw, output_ref, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top,
                    pad_bottom, g, bias, nt, iter) {}

    int Init() {
        printf("Algorithm: direct\n");
        plan(FC_ALGO_DIRECT);
        return 1;
    }

    int Tuning() {
        plan(FC_ALGO_DIRECT);
        if (fc_conv_tune(conv, iterations > 0 ? (int)iterations : 1, 1) != FC_OK) {
            fprintf(stderr, "fastconv: %s\n", fc_last_error());
            exit(EXIT_FAILURE);
        }
        return 1;
    }

    int Forward() {
        run_iterations();
        printf("Gemm time: %lfms\n", (double)stage_ms[2]);
        printf("Total time: %lfms\n", (double)stage_ms[4]);
        if (output_ref != NULL) diff(output_ref, output_data, (int)output_elems());
        return 1;
    }
};

#endif
