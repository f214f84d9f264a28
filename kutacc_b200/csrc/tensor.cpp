// Tensor descriptor, TensorWrapper and the plain-C descriptor helpers.
#include "common.h"

namespace kutacc {

// The constructor checks dim against both vector lengths (reference: src/tensor/tensor.h:32-33).
Tensor::Tensor(void *data, std::vector<int64_t> &&sizes, std::vector<int64_t> &&strides, int64_t dim, DType dtype)
    : dim_(dim), data_(data), sizes_(std::move(sizes)), strides_(std::move(strides)), dtype_(dtype)
{
    KUTACC_CHECK(dim_ == (int64_t)sizes_.size(), dim_, " ", sizes_.size());
    KUTACC_CHECK(dim_ == (int64_t)strides_.size(), dim_, " ", strides_.size());
}

int64_t Tensor::numel() const
{
    if (dim_ == 0) return 0;
    int64_t n = 1;
    for (int64_t s : sizes_) n *= s;
    return n;
}

TensorWrapper::TensorWrapper(void *data_ptr, std::vector<int64_t> &&sizes, std::vector<int64_t> &&strides,
                             int64_t dim, DType dtype)
{
    tensor_ = new Tensor(data_ptr, std::move(sizes), std::move(strides), dim, dtype);
}
TensorWrapper::TensorWrapper() { tensor_ = nullptr; }
TensorWrapper::~TensorWrapper() { delete static_cast<Tensor *>(tensor_); }

}  // namespace kutacc

extern "C" {

kutacc_tensor_h kutacc_b200_tensor_create(void *data, int64_t dim, const int64_t *sizes, const int64_t *strides,
                                          int dtype)
{
    if (dim < 0 || (dim > 0 && (sizes == nullptr || strides == nullptr))) {
        KUTACC_CHECK(false, "kutacc_b200_tensor_create: bad dim or null sizes/strides");
        return nullptr;
    }
    std::vector<int64_t> sz(sizes, sizes + dim), st(strides, strides + dim);
    return new kutacc::Tensor(data, std::move(sz), std::move(st), dim, (kutacc::DType)dtype);
}

void kutacc_b200_tensor_destroy(kutacc_tensor_h t) { delete kutacc::as_tensor(t); }

}  // extern "C"
