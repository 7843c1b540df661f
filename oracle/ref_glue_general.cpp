/*
 * TEST INFRASTRUCTURE ONLY -- second translation unit of the checker library.
 * The reference ships two different classes both named ConvNaiveLayer
 * (convLayer/naiveConv.h: 3x3 stride-1 only; convLayer/naiveConv_wudu.h: any
 * kernel size / stride / padding).  This unit is compiled with
 * -DConvNaiveLayer=ConvNaiveGeneralLayer so both can live in one library.
 *
 *   ref_naive_conv_general -> ConvNaiveLayer::Forward   convLayer/naiveConv_wudu.h:24-84
 *
 * That Forward adds bias_data[oc*OH*OW + i] to every output element whenever the
 * pointer is non-NULL (naiveConv_wudu.h:78), and the base class always
 * allocates it (conv_layer.h:72) -- so an explicit all-zero bias plane is
 * passed to keep the sum free of uninitialised memory.
 */
#include <stdlib.h>
#include <string.h>

#include "convLayer/naiveConv_wudu.h"

extern "C" int ref_naive_conv_general(float *out, const float *in, const float *kernel, int ic, int oc, int ih,
                                      int iw, int kh, int kw, int sh, int sw, int pad_l, int pad_r, int pad_t,
                                      int pad_b) {
    const size_t ow = (iw + pad_l + pad_r - kw) / sw + 1;
    const size_t oh = (ih + pad_t + pad_b - kh) / sh + 1;
    float *zero_bias = (float *)calloc((size_t)oc * oh * ow, sizeof(float));
    if (!zero_bias) return -2;
    {
        ConvNaiveLayer layer((float *)in, (float *)kernel, zero_bias, NULL, ic, ih, iw, oc, kh, kw, sh, sw, pad_l,
                             pad_r, pad_t, pad_b);
        layer.Forward();
        memcpy(out, layer.output_data, (size_t)oc * oh * ow * sizeof(float));
    }
    free(zero_bias);
    return 0;
}
