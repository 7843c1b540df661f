// ConvLayer -- the operator base class of the ConvTest harness, with the reference's constructor
// signature, members and virtuals (conv_layer.h:24-149).  What differs is below the interface:
// Init() plans the layer on a GPU through the C ABI of libfastconv_b200 and Forward() runs there.
//
// Ownership follows the reference (conv_layer.h:70-93): the constructor deep-copies input, kernel and
// bias; the layer owns output_data (HOST memory, filled by a device->host copy); output_ref is borrowed.
// Additions are optional and set after construction: set_batch(), set_math_mode(), set_context().
#pragma once

#include <assert.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fastconv_b200.h"
#include "utility/common.h"
#include "utility/helper.h"

// The process-wide GPU context the layers plan on unless one is given (device 0, arena sized on first use).
inline fc_context *&fastconv_default_context() {
    static fc_context *ctx = NULL;
    return ctx;
}

inline fc_context *fastconv_acquire_context(size_t arena_bytes) {
    fc_context *&ctx = fastconv_default_context();
    if (ctx == NULL && fc_context_create(0, arena_bytes, &ctx) != FC_OK) {
        fprintf(stderr, "fastconv: %s\n", fc_last_error());
        exit(EXIT_FAILURE);  // the reference exits when its buffers cannot be allocated
    }
    return ctx;
}

class ConvLayer {
public:
    ConvLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic, size_t ih, size_t iw, size_t oc,
              size_t kh = 3, size_t kw = 3, size_t sh = 1, size_t sw = 1, size_t pad_left = 1, size_t pad_right = 1,
              size_t pad_top = 1, size_t pad_bottom = 1, size_t g = 1, bool bias = 0, size_t nt = 1, size_t iter = 10)
        : output_data(NULL), input_channels(ic), input_width(iw), input_height(ih), output_channels(oc),
          kernel_width(kw), kernel_height(kh), stride_width(sw), stride_height(sh), padding_left(pad_left),
          padding_right(pad_right), padding_top(pad_top), padding_bottom(pad_bottom), group(g), bias_term(bias),
          num_threads(nt), iterations(iter), input_data(NULL), kernel_data(NULL), bias_data(NULL),
          output_ref(output_ref), batch(1), math_mode(FC_MATH_FP32_MIRRORED), ctx(NULL), conv(NULL),
          src_input(input) {
        assert(!(group == 0 || stride_width == 0 || stride_height == 0));
        output_width = (input_width + padding_left + padding_right - kernel_width) / stride_width + 1;
        output_height = (input_height + padding_top + padding_bottom - kernel_height) / stride_height + 1;
        const size_t k_elems = input_channels * output_channels * kw * kh;
        kernel_data = (float *)malloc((k_elems + 16) * sizeof(float));
        memcpy(kernel_data, kernel, k_elems * sizeof(float));
        if (bias_term && biasw) {
            bias_data = (float *)malloc(output_channels * sizeof(float));
            memcpy(bias_data, biasw, output_channels * sizeof(float));
        }
        copy_input(input);
        output_data = (float *)malloc(output_elems() * sizeof(float));
    }

    virtual ~ConvLayer() {
        if (conv) fc_conv_destroy(conv);
        free(input_data);
        free(kernel_data);
        free(bias_data);
        free(output_data);
        input_data = kernel_data = bias_data = output_data = NULL;
    }

    int get_output_height() { return (int)output_height; }
    int get_output_width() { return (int)output_width; }

    virtual int Init() { return -1; }
    virtual int Forward() { return -1; }
    virtual int Tuning() { return -1; }

    // ---- additions (the reference has no batch dimension and one arithmetic) -------------------
    // `input` given to the constructor must then hold n images; call before Init().
    void set_batch(size_t n) {
        batch = n;
        copy_input(src_input);
        output_data = (float *)realloc(output_data, output_elems() * sizeof(float));
    }
    void set_math_mode(int mode) { math_mode = mode; }
    void set_context(fc_context *c) { ctx = c; }
    const float *stage_milliseconds() const { return stage_ms; }
    // one machine-readable line for the layer (see print_json_line in ConvTest.cpp)
    void print_json(const fc_conv_desc &d);

    float *output_data;

protected:
    size_t input_elems() const { return batch * input_channels * input_height * input_width; }
    size_t output_elems() const { return batch * output_channels * output_height * output_width; }

    void copy_input(float *input) {
        input_data = (float *)realloc(input_data, input_elems() * sizeof(float));
        memcpy(input_data, input, input_elems() * sizeof(float));
    }

    fc_conv_desc descriptor() const {
        fc_conv_desc d;
        d.batch = (int)batch; d.ic = (int)input_channels; d.ih = (int)input_height; d.iw = (int)input_width;
        d.oc = (int)output_channels; d.kh = (int)kernel_height; d.kw = (int)kernel_width;
        d.sh = (int)stride_height; d.sw = (int)stride_width;
        d.pad_left = (int)padding_left; d.pad_right = (int)padding_right;
        d.pad_top = (int)padding_top; d.pad_bottom = (int)padding_bottom;
        d.group = (int)group;
        return d;
    }

    // Plans the layer on the GPU (uploads the kernel, sizes workspaces, one-time weight transform).
    // A failure prints the library's message and exits, like the reference's NULL-buffer checks.
    void plan(int algorithm) {
        if (conv) return;
        if (!ctx) {
            const size_t act = (input_elems() + output_elems()) * sizeof(float);
            const size_t wts = input_channels * output_channels * kernel_height * kernel_width * sizeof(float);
            const size_t tiles = batch * ((output_height + 5) / 6) * ((output_width + 5) / 6) + 8;
            const size_t wino = 64 * sizeof(float) * ((output_channels + 8) * (input_channels + 8) +
                                                      tiles * (input_channels + 8) + tiles * (output_channels + 8));
            ctx = fastconv_acquire_context(2 * (act + 8 * wts + wino) + (256u << 20));
        }
        fc_conv_desc d = descriptor();
        if (fc_conv_create(ctx, &d, algorithm, math_mode, kernel_data, &conv) != FC_OK) {
            fprintf(stderr, "fastconv: %s\n", fc_last_error());
            exit(EXIT_FAILURE);
        }
    }

    // One Forward from/to host memory, then `iterations` device-resident forwards timed per stage
    // with CUDA events (the reference's -i loop).
    void run_iterations() {
        if (fc_conv_forward_host(conv, input_data, output_data) != FC_OK) {
            fprintf(stderr, "fastconv: %s\n", fc_last_error());
            exit(EXIT_FAILURE);
        }
        float *d_in = NULL, *d_out = NULL;
        fc_conv_device_buffers(conv, &d_in, &d_out);
        const int iters = iterations > 0 ? (int)iterations : 1;
        if (fc_conv_profile(conv, d_in, d_out, iters, stage_ms) != FC_OK) {
            fprintf(stderr, "fastconv: %s\n", fc_last_error());
            exit(EXIT_FAILURE);
        }
        // the reference prints one "round time:" line per iteration of its -i loop (convLayer/winoF63ConvZC.cpp:245)
        float *rounds = (float *)malloc(iters * sizeof(float));
        int count = 0;
        if (rounds && fc_conv_round_times(conv, rounds, iters, &count) == FC_OK)
            for (int i = 0; i < count && i < iters; ++i) printf("round time: %lfms\n", (double)rounds[i]);
        free(rounds);
    }

    // The reference's line (convLayer/winoF63ConvZC.cpp:191-192) with this library's blocking in the three block
    // fields: tile block, channel block (0 = chosen per launch by the library) and the k-step of the kernels' operand
    // ring (16 floats in the fp32 mode, 32 in the tensor-core modes); then the tile count and the batch.
    void print_testing_line() {
        int bm = 0, bn = 0;
        if (conv) fc_conv_get_kernel_config(conv, &bm, &bn, NULL, NULL);
        const int tiles = (int)(batch * ((output_height + 5) / 6) * ((output_width + 5) / 6));
        printf("Testing ic=%d oc=%d width=%d tileBlock=%d ocBlock=%d icBlock=%d threads=%d tiles=%d batch=%d\n",
               (int)input_channels, (int)output_channels, (int)input_width, bn, bm,
               math_mode == FC_MATH_FP32_MIRRORED ? 16 : 32, (int)num_threads, tiles, (int)batch);
    }

    size_t input_channels, input_width, input_height;
    size_t output_channels, output_width, output_height;
    size_t kernel_width, kernel_height;
    size_t stride_width, stride_height;
    size_t padding_left, padding_right, padding_top, padding_bottom;
    size_t group;
    bool bias_term;
    size_t num_threads;  // accepted for compatibility; the GPU path does not use host threads
    size_t iterations;

    float *input_data;
    float *kernel_data;
    float *bias_data;
    float *output_ref;

    size_t batch;
    int math_mode;
    fc_context *ctx;
    fc_conv *conv;
    float stage_ms[5];

private:
    float *src_input;
};
