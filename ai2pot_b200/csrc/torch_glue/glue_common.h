// Shared helpers of the torch-op glue: argument checks, raw pointers, current stream, workspace.
// The glue registers the reference's own op names and argument lists (TORCH_LIBRARY) and forwards
// to the C ABI in include/ai2pot_b200.h. It holds no math.
#pragma once
#include <torch/library.h>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/autograd/custom_function.h>

#include "../../../include/ai2pot_b200.h"

namespace ai2b_glue {

inline void check(int rc, const char *what)
{
    TORCH_CHECK(rc == AI2B_OK, what, " failed (", rc, "): ", ai2b_last_error_string());
}

inline void require_cuda(const at::Tensor &t, const char *name)
{
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor: this build has no CPU path");
}

inline const int *iptr(const at::Tensor &t, const char *name)
{
    require_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be int32");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    return t.data_ptr<int>();
}

template <typename T>
inline const T *fptr(const at::Tensor &t, const at::Tensor &like, const char *name)
{
    require_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == like.scalar_type(), name, " must have the dtype of brcs");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    return t.data_ptr<T>();
}

inline void *stream() { return (void *)at::cuda::getCurrentCUDAStream().stream(); }

inline at::Tensor workspace(size_t bytes, const at::Tensor &like)
{
    return at::empty({(int64_t)(bytes < 256 ? 256 : bytes)}, like.options().dtype(at::kByte));
}

}  // namespace ai2b_glue
