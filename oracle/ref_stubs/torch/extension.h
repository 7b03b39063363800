// Stand-in for <torch/extension.h>, for the oracle only: just enough of the tensor interface for
// the host wrappers of the reference's classification/mmcls_custom/models/backbones/cuda_new/
// bi_wkv_kernel.cu (:370-443) to compile without the torch headers.  A Tensor here is a raw
// device pointer with up to three sizes; zeros_like allocates with cudaMalloc and frees with the
// last copy.  The dispatch macro instantiates float only.
#pragma once
#include <cuda_runtime.h>
#include <cassert>
#include <cstdint>
#include <memory>
#include <vector>

namespace torch {
struct Tensor {
    void* ptr = nullptr;
    int64_t sizes[3] = {1, 1, 1};
    int dims = 0;
    std::shared_ptr<void> owner;     // set when this stand-in allocated the memory

    template <typename T>
    T* data_ptr() const { return static_cast<T*>(ptr); }
    int64_t size(int i) const { return sizes[i]; }
    int type() const { return 0; }
    int64_t numel() const {
        int64_t n = 1;
        for (int i = 0; i < dims; ++i) n *= sizes[i];
        return n;
    }
};
inline Tensor wrap(void* p, int64_t a, int64_t b = -1, int64_t c = -1) {
    Tensor t;
    t.ptr = p;
    t.sizes[0] = a; t.dims = 1;
    if (b >= 0) { t.sizes[1] = b; t.dims = 2; }
    if (c >= 0) { t.sizes[2] = c; t.dims = 3; }
    return t;
}
inline Tensor zeros_like(const Tensor& like) {
    Tensor t = like;
    void* p = nullptr;
    const size_t bytes = static_cast<size_t>(like.numel()) * sizeof(float);
    cudaMalloc(&p, bytes);
    cudaMemset(p, 0, bytes);
    t.ptr = p;
    t.owner = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    return t;
}
}  // namespace torch

#define AT_DISPATCH_FLOATING_TYPES(TYPE, NAME, ...) \
    {                                               \
        (void)(TYPE);                               \
        using scalar_t = float;                     \
        (__VA_ARGS__)();                            \
    }
