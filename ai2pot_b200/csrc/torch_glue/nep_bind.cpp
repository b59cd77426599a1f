// libnep_bind.so: nep::nepToEFVOp, nep::nepToEFOp, nep::nepToDescriptorsOp with the reference's
// argument lists (source/descriptor/nep/bind/nep_bind.cc:26-133,278-330) over the C ABI.
// num_neurons and the descriptor count are derived from the weight shapes exactly as
// source/descriptor/nep/src/nepOp.cc:980-981 does.
#include "glue_common.h"

using namespace ai2b_glue;
using torch::autograd::variable_list;

namespace {

variable_list nep_efv(bool with_virial, int64_t cs, int64_t n_r, int64_t n_a, int64_t l_max, const at::Tensor &coeffs,
                      const at::Tensor &w0, const at::Tensor &b0, const at::Tensor &w1, const at::Tensor &bias,
                      const at::Tensor &binum, const at::Tensor &bilist, const at::Tensor &bnumneigh, const at::Tensor &bfirstneigh,
                      const at::Tensor &brcs, const at::Tensor &btypes, const at::Tensor &type_map, int64_t nghost, double rc_r,
                      double rc_a, const at::Tensor &qs, const ZblArgs &zbl)
{
    require_cuda(brcs, "brcs");
    c10::cuda::CUDAGuard guard(brcs.device());
    const int B = (int)binum.size(0), npad = (int)bnumneigh.size(1), umax = (int)bfirstneigh.size(2), ntypes = (int)type_map.size(0);
    const int nneu = (int)(w1.numel() / ntypes);
    at::Tensor e = at::empty({B}, brcs.options()), f = at::empty({B, npad + nghost, 3}, brcs.options());
    at::Tensor v = with_virial ? at::empty({B, 9}, brcs.options()) : at::Tensor();
    const bool f64 = brcs.scalar_type() == at::kDouble;
    TORCH_CHECK(f64 || brcs.scalar_type() == at::kFloat, "brcs must be float32 or float64");
    at::Tensor ws = workspace(ai2b_nep_workspace_bytes(B, ntypes, (int)n_r, (int)n_a, (int)cs, f64 ? 1 : 0), brcs);
    int rc;
    if (f64)
        rc = ai2b_nep_efv_f64(e.data_ptr<double>(), f.data_ptr<double>(), with_virial ? v.data_ptr<double>() : nullptr, (int)cs, (int)n_r,
                              (int)n_a, (int)l_max, nneu, fptr<double>(coeffs, brcs, "coeffs"), fptr<double>(w0, brcs, "w0"),
                              fptr<double>(b0, brcs, "b0"), fptr<double>(w1, brcs, "w1"), fptr<double>(bias, brcs, "type_bias"), B, npad,
                              iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                              fptr<double>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, umax, (int)nghost, rc_r, rc_a,
                              fptr<double>(qs, brcs, "q_scaler"), ws.data_ptr(), (size_t)ws.numel(), stream());
    else
        rc = ai2b_nep_efv_f32(e.data_ptr<float>(), f.data_ptr<float>(), with_virial ? v.data_ptr<float>() : nullptr, (int)cs, (int)n_r,
                              (int)n_a, (int)l_max, nneu, fptr<float>(coeffs, brcs, "coeffs"), fptr<float>(w0, brcs, "w0"),
                              fptr<float>(b0, brcs, "b0"), fptr<float>(w1, brcs, "w1"), fptr<float>(bias, brcs, "type_bias"), B, npad,
                              iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                              fptr<float>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, umax, (int)nghost, (float)rc_r, (float)rc_a,
                              fptr<float>(qs, brcs, "q_scaler"), ws.data_ptr(), (size_t)ws.numel(), stream());
    check(rc, "ai2b_nep_efv");
    apply_zbl(zbl, e, f, v, binum, bilist, bnumneigh, bfirstneigh, brcs, btypes, type_map, nghost);
    if (with_virial) return {e, f, v};
    return {e, f};
}

variable_list nep_desc(int64_t cs, int64_t n_r, int64_t n_a, int64_t l_max, const at::Tensor &coeffs, const at::Tensor &binum,
                       const at::Tensor &bilist, const at::Tensor &bnumneigh, const at::Tensor &bfirstneigh, const at::Tensor &brcs,
                       const at::Tensor &btypes, const at::Tensor &type_map, int64_t nghost, double rc_r, double rc_a)
{
    require_cuda(brcs, "brcs");
    c10::cuda::CUDAGuard guard(brcs.device());
    const int B = (int)binum.size(0), npad = (int)bnumneigh.size(1), umax = (int)bfirstneigh.size(2), ntypes = (int)type_map.size(0);
    const int nd = l_max == 0 ? (int)n_r : (int)(n_r + n_a * l_max);
    at::Tensor d = at::empty({B, npad, nd}, brcs.options());
    const bool f64 = brcs.scalar_type() == at::kDouble;
    at::Tensor ws = workspace(ai2b_nep_workspace_bytes(B, ntypes, (int)n_r, (int)n_a, (int)cs, f64 ? 1 : 0), brcs);
    int rc;
    if (f64)
        rc = ai2b_nep_descriptors_f64(d.data_ptr<double>(), (int)cs, (int)n_r, (int)n_a, (int)l_max, fptr<double>(coeffs, brcs, "coeffs"), B,
                                      npad, iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"),
                                      iptr(bfirstneigh, "bfirstneigh"), fptr<double>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, umax,
                                      (int)nghost, rc_r, rc_a, ws.data_ptr(), (size_t)ws.numel(), stream());
    else
        rc = ai2b_nep_descriptors_f32(d.data_ptr<float>(), (int)cs, (int)n_r, (int)n_a, (int)l_max, fptr<float>(coeffs, brcs, "coeffs"), B,
                                      npad, iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"),
                                      iptr(bfirstneigh, "bfirstneigh"), fptr<float>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes, umax,
                                      (int)nghost, (float)rc_r, (float)rc_a, ws.data_ptr(), (size_t)ws.numel(), stream());
    check(rc, "ai2b_nep_descriptors");
    return {d};
}

}  // namespace

#define NEP_EFV_ARGS                                                                                                         \
    int64_t chebyshev_size, int64_t n_radial_basis, int64_t n_angular_basis, int64_t l_max, const at::Tensor &coeffs_tensor, \
        const at::Tensor &w0_tensor, const at::Tensor &b0_tensor, const at::Tensor &w1_tensor,                               \
        const at::Tensor &type_bias_tensor, const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor,                 \
        const at::Tensor &bnumneigh_tensor, const at::Tensor &bfirstneigh_tensor, const at::Tensor &brcs_tensor,             \
        const at::Tensor &btypes_tensor, const at::Tensor &type_map_tensor, int64_t nghost, double rmax_radial,              \
        double rmax_angular, const at::Tensor &q_scaler_tensor, double zbl_rmax, double zbl_rmin,                            \
        const at::Tensor &zbl_cks_tensor, const at::Tensor &zbl_dks_tensor
#define NEP_EFV_PASS                                                                                                         \
    chebyshev_size, n_radial_basis, n_angular_basis, l_max, coeffs_tensor, w0_tensor, b0_tensor, w1_tensor, type_bias_tensor, \
        binum_tensor, bilist_tensor, bnumneigh_tensor, bfirstneigh_tensor, brcs_tensor, btypes_tensor, type_map_tensor,      \
        nghost, rmax_radial, rmax_angular, q_scaler_tensor, ZblArgs{zbl_rmax, zbl_rmin, zbl_cks_tensor, zbl_dks_tensor}

#include "nep_loss_glue.inc"

TORCH_LIBRARY(nep, m)
{
    register_nep_loss_ops(m);
    m.def("nepToEFVOp", [](NEP_EFV_ARGS) {
        return nep_efv(true, NEP_EFV_PASS);
    });
    m.def("nepToEFOp", [](NEP_EFV_ARGS) {
        return nep_efv(false, NEP_EFV_PASS);
    });
    m.def("nepToDescriptorsOp",
          [](int64_t chebyshev_size, int64_t n_radial_basis, int64_t n_angular_basis, int64_t l_max, const at::Tensor &coeffs_tensor,
             const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor, const at::Tensor &bnumneigh_tensor,
             const at::Tensor &bfirstneigh_tensor, const at::Tensor &brcs_tensor, const at::Tensor &btypes_tensor,
             const at::Tensor &type_map_tensor, int64_t nghost, double rmax_radial, double rmax_angular) {
              return nep_desc(chebyshev_size, n_radial_basis, n_angular_basis, l_max, coeffs_tensor, binum_tensor, bilist_tensor,
                              bnumneigh_tensor, bfirstneigh_tensor, brcs_tensor, btypes_tensor, type_map_tensor, nghost, rmax_radial,
                              rmax_angular);
          });
}
