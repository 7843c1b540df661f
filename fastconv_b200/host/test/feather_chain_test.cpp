// Exercises the FeatherCNN-style host interface over the GPU library: CommonMemPool / PrivateMemPool (utility/mempool.h),
// Blob (utility/blob.h), RuntimeParameter (rt_param.h), Layer (layer.h) and the convolution node built on them
// (feather_conv.h).  conv3x3 + bias + ReLU -> conv1x1 + bias + ReLU on device blobs, checked against a plain host
// loop.  Prints "feather chain ok" and exits 0 on success.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "feather_conv.h"
#include "tensor.h"

static float frand(unsigned &s) {
    s = s * 1664525u + 1013904223u;
    return ((s >> 8) & 0xffff) / 32768.0f - 1.0f;
}

static void host_conv_bias_relu(const std::vector<float> &in, const std::vector<float> &w, const std::vector<float> &b,
                                std::vector<float> &out, int n, int ic, int ih, int iw, int oc, int k, int pad) {
    const int oh = ih + 2 * pad - k + 1, ow = iw + 2 * pad - k + 1;
    out.assign((size_t)n * oc * oh * ow, 0.f);
    for (int img = 0; img < n; ++img)
        for (int o = 0; o < oc; ++o)
            for (int y = 0; y < oh; ++y)
                for (int x = 0; x < ow; ++x) {
                    double acc = 0.0;
                    for (int c = 0; c < ic; ++c)
                        for (int u = 0; u < k; ++u)
                            for (int v = 0; v < k; ++v) {
                                const int yy = y + u - pad, xx = x + v - pad;
                                if (yy < 0 || yy >= ih || xx < 0 || xx >= iw) continue;
                                acc += (double)in[(((size_t)img * ic + c) * ih + yy) * iw + xx] *
                                       w[(((size_t)o * ic + c) * k + u) * k + v];
                            }
                    const float v = (float)acc + b[o];
                    out[(((size_t)img * oc + o) * oh + y) * ow + x] = v > 0.f ? v : 0.f;
                }
}

#define REQUIRE(cond)                                                          \
    do {                                                                       \
        if (!(cond)) {                                                         \
            fprintf(stderr, "FAILED %s (line %d): %s\n", #cond, __LINE__, fc_last_error()); \
            return 1;                                                          \
        }                                                                      \
    } while (0)

int main() {
    fc_context *ctx = NULL;
    REQUIRE(fc_context_create(0, (size_t)256 << 20, &ctx) == FC_OK);
    {
        CommonMemPool<float> common(ctx);
        PrivateMemPool<float> pool(ctx);
        RuntimeParameter<float> rt(ctx, &common, 1);
        Tensor<float> unused;  // the reference's tensor.h is an empty class; so is this one
        (void)unused;

        // the pools by themselves
        REQUIRE(common.Request(1000, 3) && common.Request(4000, 3) && common.Alloc());
        float *scratch = NULL;
        REQUIRE(common.GetPtr(&scratch, 3) && scratch != NULL);
        float *priv = NULL;
        size_t sz = 0;
        REQUIRE(pool.Alloc(&priv, 777) && pool.GetSize(priv, &sz) && sz == 777);
        REQUIRE(pool.Free(&priv) && priv == NULL);
        REQUIRE(common.Free(3));

        const int n = 2, ic = 8, hw = 14, oc1 = 16, oc2 = 8;
        unsigned seed = 12345u;
        std::vector<float> x((size_t)n * ic * hw * hw), w1((size_t)oc1 * ic * 9), b1(oc1), w2((size_t)oc2 * oc1), b2(oc2);
        for (size_t i = 0; i < x.size(); ++i) x[i] = frand(seed);
        for (size_t i = 0; i < w1.size(); ++i) w1[i] = 0.2f * frand(seed);
        for (size_t i = 0; i < w2.size(); ++i) w2[i] = 0.3f * frand(seed);
        for (size_t i = 0; i < b1.size(); ++i) b1[i] = 0.1f * frand(seed);
        for (size_t i = 0; i < b2.size(); ++i) b2[i] = 0.1f * frand(seed);

        feather::Blob<float> data(&pool, n, ic, hw, hw, "data");
        data.Alloc();
        REQUIRE(data.data() != NULL && data.CopyData(ctx, x.data()));

        feather::ConvolutionLayer conv1("conv1", &rt, w1.data(), b1.data(), oc1, 3, 3, 1, 1);
        feather::ReluLayer relu1("relu1", &rt);
        feather::ConvolutionLayer conv2("conv2", &rt, w2.data(), b2.data(), oc2, 1, 1, 1, 0);
        feather::ReluLayer relu2("relu2", &rt);
        REQUIRE(relu1.Forward() == -1);  // not fused yet: there is no stand-alone ReLU
        REQUIRE(conv1.SetupBottomBlob(&data, "data") == 0 && conv1.SetupBottomBlob(&data, "data") == -1);
        REQUIRE(conv1.TryFuse(&relu1) == 1 && conv2.TryFuse(&relu2) == 1);
        REQUIRE(conv1.GenerateTopBlobs() == 0 && conv1.Init() == 0);
        REQUIRE(conv2.SetupBottomBlob(conv1.top_blob(0), conv1.top(0)) == 0);
        REQUIRE(conv2.GenerateTopBlobs() == 0 && conv2.Init() == 0);
        const feather::Blob<float> *out = conv2.top_blob("conv2");
        REQUIRE(out != NULL && out->num() == (size_t)n && out->channels() == (size_t)oc2 && out->height() == (size_t)hw);

        // two passes, device to device, nothing crosses to the host in between
        for (int pass = 0; pass < 2; ++pass) {
            REQUIRE(conv1.Forward() == 0 && relu1.Forward() == 0 && conv2.Forward() == 0 && relu2.Forward() == 0);
        }
        REQUIRE(fc_context_synchronize(ctx) == FC_OK);
        std::vector<float> got(out->data_size()), mid, want;
        REQUIRE(out->ReadData(ctx, got.data()));
        host_conv_bias_relu(x, w1, b1, mid, n, ic, hw, hw, oc1, 3, 1);
        host_conv_bias_relu(mid, w2, b2, want, n, oc1, hw, hw, oc2, 1, 0);
        double num = 0, den = 0;
        for (size_t i = 0; i < got.size(); ++i) {
            num += ((double)got[i] - want[i]) * ((double)got[i] - want[i]);
            den += (double)want[i] * want[i];
        }
        const double rel = sqrt(num / (den > 0 ? den : 1));
        printf("relative L2 difference to the host loop: %.3e\n", rel);
        REQUIRE(rel < 1e-5 && den > 0);
        common.PrintStats();
        pool.PrintStats();
    }
    fc_context_destroy(ctx);
    printf("feather chain ok\n");
    return 0;
}
