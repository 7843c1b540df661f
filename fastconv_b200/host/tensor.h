// Placeholder kept for source compatibility: the reference's tensor.h is an empty Tensor<Dtype> stub.
#pragma once

template <typename Dtype>
class Tensor {
public:
    Tensor() {}
};
