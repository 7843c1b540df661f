// feather::Blob -- an fp32 NCHW tensor handle (reference: utility/blob.h:24-119), here over DEVICE memory
// from a PrivateMemPool.  Kept for code written against the FeatherCNN-style Layer interface (layer.h).
#pragma once

#include <assert.h>
#include <stdio.h>

#include <string>

#include "mempool.h"

namespace feather {

template <class Dtype>
class Blob {
public:
    Blob() : _data(NULL), _num(0), _channels(0), _height(0), _width(0), _pool(NULL) {}
    Blob(PrivateMemPool<Dtype> *pool, size_t num, size_t channels, size_t height, size_t width, std::string name = "")
        : _data(NULL), _num(num), _channels(channels), _height(height), _width(width), _name(name), _pool(pool) {}
    ~Blob() { Free(); }

    void Alloc() {
        if (_data == NULL && _pool != NULL && data_size() > 0) _pool->Alloc(&_data, data_size() * sizeof(Dtype));
    }
    void Free() {
        if (_data != NULL && _pool != NULL) _pool->Free(&_data);
        _data = NULL;
    }
    void Realloc(size_t elem_size) {
        Free();
        if (_pool != NULL && elem_size > 0) _pool->Alloc(&_data, elem_size * sizeof(Dtype));
    }
    void ReshapeWithRealloc(int num, int channels, int height, int width) {
        const size_t old = data_size();
        _num = num; _channels = channels; _height = height; _width = width;
        if (data_size() > old || _data == NULL) Realloc(data_size());
    }
    void ReshapeWithRealloc(const Blob<Dtype> *b) {
        ReshapeWithRealloc((int)b->num(), (int)b->channels(), (int)b->height(), (int)b->width());
    }
    // host -> device / device -> host copies of the whole tensor
    bool CopyData(fc_context *ctx, const Dtype *host) {
        return fc_memcpy_h2d(ctx, _data, host, data_size() * sizeof(Dtype)) == FC_OK;
    }
    bool ReadData(fc_context *ctx, Dtype *host) const {
        return fc_memcpy_d2h(ctx, host, _data, data_size() * sizeof(Dtype)) == FC_OK;
    }
    void CopyShape(const Blob<Dtype> *b) {
        _num = b->num(); _channels = b->channels(); _height = b->height(); _width = b->width();
    }

    Dtype *data() const { return _data; }
    size_t data_size() const { return _num * _channels * _height * _width; }
    std::string name() { return _name; }
    size_t num() const { return _num; }
    size_t channels() const { return _channels; }
    size_t height() const { return _height; }
    size_t width() const { return _width; }
    void PrintBlobInfo() const {
        printf("----BlobInfo----\nShape in nchw (%zu %zu %zu %zu)\n----------------\n", _num, _channels, _height, _width);
    }

private:
    Dtype *_data;
    size_t _num, _channels, _height, _width;
    std::string _name;
    PrivateMemPool<Dtype> *_pool;
};

}  // namespace feather
