// feather::ConvolutionLayer / feather::ReluLayer -- conv layers as nodes of the FeatherCNN-style graph interface that
// the reference carries (layer.h:29-84, utility/blob.h:24-119) but never compiles.  A node reads its bottom Blob
// and writes its top Blob, both in DEVICE memory, so consecutive layers run without a host round trip; a ReLU
// that follows a convolution is fused into the convolution's last kernel (Layer::TryFuse / Fuse, layer.h:44-50)
// together with the per-channel bias (bias_term of conv_layer.h:46-48).
#pragma once

#include <stdio.h>

#include <string>

#include "fastconv_b200.h"
#include "layer.h"

namespace feather {

// ReLU exists only fused into the producer of its input: after Fuse() its Forward is a no-op and its top blob IS the
// producer's top blob; unfused it reports -1 (there is no stand-alone activation kernel in the library).
class ReluLayer : public Layer {
public:
    ReluLayer(const std::string &name, const RuntimeParameter<float> *rt_param)
        : Layer(name, "ReLU", rt_param), fused_into(NULL) {}
    int Forward() { return fused_into ? 0 : -1; }
    Layer *fused_into;
};

class ConvolutionLayer : public Layer {
public:
    // weights [oc][ic/group][kh][kw] and bias [oc] (or NULL) are HOST arrays, copied at Init()
    ConvolutionLayer(const std::string &name, const RuntimeParameter<float> *rt_param, const float *weights,
                     const float *bias, size_t oc, size_t kh, size_t kw, size_t stride, size_t pad, size_t group = 1,
                     int algorithm = FC_ALGO_AUTO, int math_mode = FC_MATH_FP32_MIRRORED)
        : Layer(name, "Convolution", rt_param), weights_(weights), bias_(bias), oc_(oc), kh_(kh), kw_(kw),
          stride_(stride), pad_(pad), group_(group), algorithm_(algorithm), math_mode_(math_mode), relu_(0), conv_(NULL) {
        _fusible = true;
        _top.push_back(name);
    }
    ~ConvolutionLayer() {
        if (conv_) fc_conv_destroy(conv_);
    }

    int Fuse(Layer *next_layer) {
        if (next_layer->type() != "ReLU") return 0;
        relu_ = 1;
        static_cast<ReluLayer *>(next_layer)->fused_into = this;
        return 1;
    }

    int GenerateTopBlobs() {
        if (_bottom.size() != 1) return -1;
        const Blob<float> *in = _bottom_blobs[_bottom[0]];
        fc_conv_desc d = descriptor(in);
        int oh = 0, ow = 0;
        if (fc_conv_output_size(&d, &oh, &ow) != FC_OK) return -1;
        Blob<float> *&top = _top_blobs[_top[0]];
        if (top == NULL) top = new Blob<float>(&private_mempool, in->num(), oc_, oh, ow, _top[0]);
        top->ReshapeWithRealloc((int)in->num(), (int)oc_, oh, ow);
        return top->data() != NULL ? 0 : -1;
    }

    int Init() {
        if (conv_) return 0;
        const Blob<float> *in = _bottom_blobs[_bottom[0]];
        fc_conv_desc d = descriptor(in);
        if (fc_conv_create(_ctx, &d, algorithm_, math_mode_, weights_, &conv_) != FC_OK ||
            fc_conv_set_epilogue(conv_, bias_, relu_) != FC_OK) {
            fprintf(stderr, "feather::ConvolutionLayer %s: %s\n", _name.c_str(), fc_last_error());
            return -1;
        }
        return 0;
    }

    // asynchronous on the context's stream: the next node may be enqueued right away
    int Forward() {
        const Blob<float> *in = _bottom_blobs[_bottom[0]];
        return fc_conv_forward_device(conv_, in->data(), _top_blobs[_top[0]]->data()) == FC_OK ? 0 : -1;
    }

    fc_conv *planned() const { return conv_; }

private:
    fc_conv_desc descriptor(const Blob<float> *in) const {
        fc_conv_desc d;
        d.batch = (int)in->num(); d.ic = (int)in->channels(); d.ih = (int)in->height(); d.iw = (int)in->width();
        d.oc = (int)oc_; d.kh = (int)kh_; d.kw = (int)kw_; d.sh = d.sw = (int)stride_;
        d.pad_left = d.pad_right = d.pad_top = d.pad_bottom = (int)pad_;
        d.group = (int)group_;
        return d;
    }

    const float *weights_, *bias_;
    size_t oc_, kh_, kw_, stride_, pad_, group_;
    int algorithm_, math_mode_, relu_;
    fc_conv *conv_;
};

}  // namespace feather
