// feather::Layer -- the FeatherCNN-style graph node interface of the reference (layer.h:29-84): named
// bottom/top blobs, Init/Forward/ForwardReshape/GenerateTopBlobs/Fuse.  The reference does not compile
// this file (it needs a missing rt_param.h); here it is a small working base over device Blobs so that
// conv layers can be chained on the GPU without host round trips.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "rt_param.h"
#include "utility/blob.h"

namespace feather {

class Layer {
public:
    Layer(const std::string &name, const std::string &type, const RuntimeParameter<float> *rt_param)
        : _name(name), _type(type), _fusible(false), _inplace(false), num_threads(rt_param->num_threads()),
          common_mempool(rt_param->common_mempool()), private_mempool(rt_param->context()), _ctx(rt_param->context()) {}
    virtual ~Layer() {
        for (std::map<std::string, Blob<float> *>::iterator it = _top_blobs.begin(); it != _top_blobs.end(); ++it)
            delete it->second;
    }

    int SetupBottomBlob(const Blob<float> *p_blob, std::string name) {
        if (_bottom_blobs.find(name) != _bottom_blobs.end()) return -1;
        _bottom_blobs[name] = p_blob;
        _bottom.push_back(name);
        return 0;
    }
    int ReplaceBottomBlob(std::string old_bottom, std::string new_bottom, const Blob<float> *p_blob) {
        std::map<std::string, const Blob<float> *>::iterator it = _bottom_blobs.find(old_bottom);
        if (it == _bottom_blobs.end()) return -1;
        _bottom_blobs.erase(it);
        _bottom_blobs[new_bottom] = p_blob;
        for (size_t i = 0; i < _bottom.size(); ++i)
            if (_bottom[i] == old_bottom) _bottom[i] = new_bottom;
        return 0;
    }
    int TryFuse(Layer *next_layer) { return _fusible ? Fuse(next_layer) : 0; }
    virtual int Fuse(Layer *) { return 0; }
    virtual int GenerateTopBlobs() { return 0; }
    virtual int Init() { return 0; }
    virtual int Forward() { return 0; }
    virtual int ForwardReshape() { return GenerateTopBlobs() == 0 ? Forward() : -1; }

    std::string name() { return _name; }
    std::string type() { return _type; }
    std::string bottom(size_t i) { return i < _bottom.size() ? _bottom[i] : std::string(); }
    size_t bottom_size() { return _bottom.size(); }
    std::string top(size_t i) { return i < _top.size() ? _top[i] : std::string(); }
    size_t top_size() { return _top.size(); }
    size_t top_blob_size() { return _top_blobs.size(); }
    const Blob<float> *top_blob(std::string name) {
        std::map<std::string, Blob<float> *>::iterator it = _top_blobs.find(name);
        return it == _top_blobs.end() ? NULL : it->second;
    }
    const Blob<float> *top_blob(size_t idx) { return idx < _top.size() ? top_blob(_top[idx]) : NULL; }
    size_t weight_blob_num() const { return _weight_blobs.size(); }
    const Blob<float> *weight_blob(size_t i) const { return i < _weight_blobs.size() ? _weight_blobs[i] : NULL; }
    bool fusible() const { return _fusible; }

protected:
    std::string _name, _type;
    std::vector<std::string> _bottom, _top;
    std::map<std::string, const Blob<float> *> _bottom_blobs;
    std::map<std::string, Blob<float> *> _top_blobs;
    std::vector<Blob<float> *> _weight_blobs;
    bool _fusible, _inplace;
    size_t num_threads;
    CommonMemPool<float> *common_mempool;
    PrivateMemPool<float> private_mempool;
    fc_context *_ctx;
};

}  // namespace feather
