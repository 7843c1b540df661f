// Host utilities of the ConvTest harness: stopwatch, error metric, option enums.
//
// Same names and meaning as the reference's utility/helper.h (Timer :66-80, diff :40-41, the nnp_*
// option types :82-126) so that ConvTest and the layer classes read the same.  Timer measures host
// wall-clock; per-stage GPU times come from CUDA events inside the library (fc_conv_profile).
#pragma once

#include <stddef.h>
#include <stdio.h>
#include <time.h>

#include "fastconv_b200.h"

#define LOGI(...) fprintf(stdout, __VA_ARGS__)
#define LOGD(...) fprintf(stdout, __VA_ARGS__)
#define LOGE(...) fprintf(stderr, __VA_ARGS__)

class Timer {
public:
    Timer() : accumulate(0.0) {}
    virtual ~Timer() {}
    void startBench() { clock_gettime(CLOCK_MONOTONIC, &start); }
    void accumBench() { accumulate += lap(); }
    void add(double ms) { accumulate += ms; }  // device milliseconds measured by the library
    void printBench(const char *comment, int fold) { LOGD("%s %lfms\n", comment, accumulate / fold); }
    void endBench(const char *comment) { LOGD("%s %lfms\n", comment, lap()); }
    void endBench(const char *comment, double fold) { printf("%s time: %lfms\n", comment, lap() / fold); }
    double endBench(double fold) { return lap() / fold; }

private:
    double lap() {
        clock_gettime(CLOCK_MONOTONIC, &stop);
        return (stop.tv_sec - start.tv_sec) * 1000.0 + (stop.tv_nsec - start.tv_nsec) / 1000000.0;
    }
    timespec start, stop;
    double accumulate;
};

// mean |a-b| over the elements with |a-b| > 1e-5; prints "The difference is" (utility/helper.cpp:74-89)
inline float diff(float *arr1, float *arr2, int len) {
    const float d = fc_diff(arr1, arr2, len);
    LOGD("The difference is %.5f\n", d);
    return d;
}

struct nnp_size {
    size_t width;
    size_t height;
};

struct nnp_padding {
    size_t top;
    size_t right;
    size_t bottom;
    size_t left;
};

enum nnp_convolution_algorithm {
    nnp_convolution_algorithm_auto = FC_ALGO_AUTO,
    nnp_convolution_algorithm_direct = FC_ALGO_DIRECT,
    nnp_convolution_algorithm_im2col = FC_ALGO_IM2COL,
    nnp_convolution_algorithm_winograd = FC_ALGO_WINOGRAD
};

enum nnp_convolution_transform_strategy {
    nnp_convolution_transform_strategy_online = 0,
    nnp_convolution_transform_strategy_offline = 1
};

enum nnp_convolution_tuning_strategy {
    nnp_convolution_tuning_strategy_no_tuning = 0,
    nnp_convolution_tuning_strategy_grid_search = 1
};
