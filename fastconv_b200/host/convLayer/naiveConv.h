// ConvNaiveLayer -- the harness's self-check: a plain direct convolution on the HOST that ConvTest
// compares the GPU result with, as the reference does (convLayer/naiveConv.h:24-64 for 3x3 stride 1,
// convLayer/naiveConv_wudu.h:24-84 for any kernel size / stride).  It is a checker for the command-line
// tool only; no layer class and no library entry point ever computes through it.
#pragma once

#include "../conv_layer.h"

class ConvNaiveLayer : public ConvLayer {
public:
    ConvNaiveLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic, size_t ih, size_t iw,
                   size_t oc, size_t kh = 3, size_t kw = 3, size_t sh = 1, size_t sw = 1, size_t pad_left = 1,
                   size_t pad_right = 1, size_t pad_top = 1, size_t pad_bottom = 1, size_t g = 1, bool bias = 0,
                   size_t nt = 1, size_t iter = 10)
        : ConvLayer(input, kernel, biasw, output_ref, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top,
                    pad_bottom, g, bias, nt, iter) {}

    int Init() { return -1; }
    int Tuning() { return -1; }

    // per input channel a kh*kw partial sum `total`, then `sum += total` (the reference's order)
    int Forward() {
        const size_t in_page = input_height * input_width, out_page = output_height * output_width;
        const size_t k_page = kernel_height * kernel_width;
#pragma omp parallel for collapse(2)
        for (size_t n = 0; n < batch; ++n)
            for (size_t oc = 0; oc < output_channels; ++oc)
                for (size_t px = 0; px < out_page; ++px) {
                    const long y0 = (long)(px / output_width * stride_height) - (long)padding_top;
                    const long x0 = (long)(px % output_width * stride_width) - (long)padding_left;
                    float sum = 0;
                    for (size_t ic = 0; ic < input_channels; ++ic) {
                        const float *ip = input_data + (n * input_channels + ic) * in_page;
                        const float *kp = kernel_data + (oc * input_channels + ic) * k_page;
                        float total = 0;
                        for (size_t i = 0; i < kernel_height; ++i)
                            for (size_t j = 0; j < kernel_width; ++j) {
                                const long y = y0 + (long)i, x = x0 + (long)j;
                                if (y < 0 || y >= (long)input_height || x < 0 || x >= (long)input_width) continue;
                                total += ip[y * (long)input_width + x] * kp[i * kernel_width + j];
                            }
                        sum += total;
                    }
                    output_data[(n * output_channels + oc) * out_page + px] = sum;
                }
        return 1;
    }
};
