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

// g[B] @ parts[k][B, n_k] for every k in one launch (what a training op's backward returns per parameter
// tensor); results are views into one flat tensor, in the order of `parts`
inline std::vector<at::Tensor> weighted_sums(const at::Tensor &g, const std::vector<at::Tensor> &parts)
{
    const int B = (int)g.numel(), np = (int)parts.size();
    std::vector<int> n(np);
    std::vector<const void *> ptr(np);
    int64_t total = 0;
    for (int k = 0; k < np; k++) { n[k] = B ? (int)(parts[k].numel() / B) : 0; ptr[k] = parts[k].data_ptr(); total += n[k]; }
    at::Tensor flat = at::zeros({total}, g.options());
    if (B > 0 && total > 0) {
        int rc;
        if (g.scalar_type() == at::kDouble)
            rc = ai2b_weighted_sum_rows_f64(np, (const double *const *)ptr.data(), n.data(), B, g.data_ptr<double>(), flat.data_ptr<double>(), stream());
        else
            rc = ai2b_weighted_sum_rows_f32(np, (const float *const *)ptr.data(), n.data(), B, g.data_ptr<float>(), flat.data_ptr<float>(), stream());
        TORCH_CHECK(rc == AI2B_OK, "ai2b_weighted_sum_rows: ", ai2b_last_error_string());
    }
    std::vector<at::Tensor> out(np);
    int64_t off = 0;
    for (int k = 0; k < np; k++) { out[k] = flat.narrow(0, off, n[k]); off += n[k]; }
    return out;
}

// ZBL parameters of an op call (zbl_rmax <= 0: no correction)
struct ZblArgs {
    double rmax, rmin;
    const at::Tensor &cks, &dks;
};

// adds the ZBL pair correction onto e[B], f[B,Np+nghost,3] and, if defined, v[B,9]
inline void apply_zbl(const ZblArgs &z, at::Tensor &e, at::Tensor &f, const at::Tensor &v, const at::Tensor &binum,
                      const at::Tensor &bilist, const at::Tensor &bnumneigh, const at::Tensor &bfirstneigh, const at::Tensor &brcs,
                      const at::Tensor &btypes, const at::Tensor &type_map, int64_t nghost)
{
    if (z.rmax <= 0.0) return;
    const int B = (int)binum.size(0), npad = (int)bnumneigh.size(1), umax = (int)bfirstneigh.size(2), ntypes = (int)type_map.size(0);
    TORCH_CHECK(z.cks.numel() >= (int64_t)ntypes * ntypes * 4 && z.dks.numel() >= (int64_t)ntypes * ntypes * 4,
                "zbl_cks / zbl_dks must hold ntypes * ntypes * 4 values");
    int rc;
    if (brcs.scalar_type() == at::kDouble)
        rc = ai2b_zbl_efv_f64(e.data_ptr<double>(), f.data_ptr<double>(), v.defined() ? v.data_ptr<double>() : nullptr, B, npad,
                              iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                              fptr<double>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, iptr(type_map, "type_map"), umax,
                              (int)nghost, z.rmax, z.rmin, fptr<double>(z.cks, brcs, "zbl_cks"), fptr<double>(z.dks, brcs, "zbl_dks"),
                              stream());
    else
        rc = ai2b_zbl_efv_f32(e.data_ptr<float>(), f.data_ptr<float>(), v.defined() ? v.data_ptr<float>() : nullptr, B, npad,
                              iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                              fptr<float>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, iptr(type_map, "type_map"), umax,
                              (int)nghost, (float)z.rmax, (float)z.rmin, fptr<float>(z.cks, brcs, "zbl_cks"),
                              fptr<float>(z.dks, brcs, "zbl_dks"), stream());
    check(rc, "ai2b_zbl_efv");
}

}  // namespace ai2b_glue
