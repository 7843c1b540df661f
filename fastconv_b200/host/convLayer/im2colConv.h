// im2col + SGEMM layer: class name, constructor (including the ARM blocking arguments) and methods of
// the reference (convLayer/im2colConv.h:9-53).  The blocking arguments are accepted and ignored: the
// GPU kernel gathers the im2col matrix inside its operand producer and has its own tiling.
#ifndef IM2COLCONV_H
#define IM2COLCONV_H

#include "../conv_layer.h"

class ConvIm2colLayer : public ConvLayer {
public:
    ConvIm2colLayer(float *input, float *kernel, float *biasw, float *output_ref, size_t ic, size_t ih, size_t iw,
                    size_t oc, size_t kh = 3, size_t kw = 3, size_t sh = 1, size_t sw = 1, size_t pad_left = 1,
                    size_t pad_right = 1, size_t pad_top = 1, size_t pad_bottom = 1, size_t g = 1, bool bias = 0,
                    size_t nt = 1, size_t iter = 10, int mc = 8, int nc = 256, int kc = 384, int gemm_version = 1,
                    int row_batch = 8, int col_batch = 8, int pack_c_version = 0, int mt_pack_b_version = 2,
                    int prefetch_a = 256, int prefetch_b = 256, int prefetch_c = 0);
    ~ConvIm2colLayer();

    int Init();
    int Tuning();
    int Forward();

    // Materialises the gathered matrix [ic*kh*kw][oh*ow] of image 0 into transform_input_data (host), for
    // inspection: the index map of ConvIm2colLayer::im2col, convLayer/im2colConv.cpp:285-309.
    void im2col();
    const float *gathered() const { return transform_input_data; }

protected:
    int M, N, K;
    float *transform_input_data;
};

#endif
