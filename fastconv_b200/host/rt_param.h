// Runtime parameters handed to feather::Layer (the reference's layer.h:19 includes an rt_param.h that is
// not in its tree; only a shared scratch pool and a thread count are implied, layer.h:79-83).
#pragma once

#include "fastconv_b200.h"
#include "utility/mempool.h"

template <typename Dtype>
class RuntimeParameter {
public:
    RuntimeParameter(fc_context *ctx, CommonMemPool<Dtype> *pool, size_t threads = 1)
        : _ctx(ctx), _common_mempool(pool), _num_threads(threads) {}
    fc_context *context() const { return _ctx; }
    CommonMemPool<Dtype> *common_mempool() const { return _common_mempool; }
    size_t num_threads() const { return _num_threads; }

private:
    fc_context *_ctx;
    CommonMemPool<Dtype> *_common_mempool;
    size_t _num_threads;
};
