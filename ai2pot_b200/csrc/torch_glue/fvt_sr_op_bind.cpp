// libfvt_sr_op_bind.so: fvt::ForceSrOp and fvt::VirialSrOp (source/fvt/bind/fvt_sr_op_bind.cc:9-46;
// forward/backward semantics source/fvt/src/force_sr_op.cc:11-179, virial_sr_op.cc:10-163) over
// the C ABI. Differentiable like the reference ops; the backward applies the +1/-1 (force) and
// -r / -dE (virial) Jacobians without materialising them.
#include "glue_common.h"

using namespace ai2b_glue;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

namespace {

struct ForceSrFunction : public torch::autograd::Function<ForceSrFunction> {
    static variable_list forward(AutogradContext *ctx, const at::Tensor &binum, const at::Tensor &bilist, const at::Tensor &bnumneigh,
                                 const at::Tensor &bfirstneigh, int64_t nghost, int64_t umax, const at::Tensor &de)
    {
        require_cuda(de, "bdei_drij");
        c10::cuda::CUDAGuard guard(de.device());
        const int B = (int)bilist.size(0), npad = (int)bilist.size(1);
        at::Tensor d = de.contiguous();
        at::Tensor force = at::empty({B, npad + nghost, 3}, d.options());
        int rc = d.scalar_type() == at::kDouble
                     ? ai2b_fvt_force_fwd_f64(force.data_ptr<double>(), B, npad, (int)nghost, (int)umax, iptr(binum, "binum"),
                                              iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                                              d.data_ptr<double>(), stream())
                     : ai2b_fvt_force_fwd_f32(force.data_ptr<float>(), B, npad, (int)nghost, (int)umax, iptr(binum, "binum"),
                                              iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                                              d.data_ptr<float>(), stream());
        check(rc, "ai2b_fvt_force_fwd");
        ctx->save_for_backward({binum, bilist, bnumneigh, bfirstneigh});
        ctx->saved_data["nghost"] = nghost;
        ctx->saved_data["umax"] = umax;
        return {force};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grads)
    {
        auto saved = ctx->get_saved_variables();
        const at::Tensor &binum = saved[0], &bilist = saved[1], &bnumneigh = saved[2], &bfirstneigh = saved[3];
        const int64_t nghost = ctx->saved_data["nghost"].toInt(), umax = ctx->saved_data["umax"].toInt();
        at::Tensor g = grads[0].contiguous();
        c10::cuda::CUDAGuard guard(g.device());
        const int B = (int)bilist.size(0), npad = (int)bilist.size(1);
        at::Tensor out = at::empty({B, npad, umax, 3}, g.options());
        int rc = g.scalar_type() == at::kDouble
                     ? ai2b_fvt_force_bwd_f64(out.data_ptr<double>(), B, npad, (int)nghost, (int)umax, iptr(binum, "binum"),
                                              iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                                              g.data_ptr<double>(), stream())
                     : ai2b_fvt_force_bwd_f32(out.data_ptr<float>(), B, npad, (int)nghost, (int)umax, iptr(binum, "binum"),
                                              iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"),
                                              g.data_ptr<float>(), stream());
        check(rc, "ai2b_fvt_force_bwd");
        return {at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), out};
    }
};

struct VirialSrFunction : public torch::autograd::Function<VirialSrFunction> {
    static variable_list forward(AutogradContext *ctx, const at::Tensor &bnumneigh, const at::Tensor &brcs, int64_t umax,
                                 const at::Tensor &de)
    {
        require_cuda(de, "bdei_drij");
        c10::cuda::CUDAGuard guard(de.device());
        const int B = (int)bnumneigh.size(0), npad = (int)bnumneigh.size(1);
        at::Tensor d = de.contiguous(), r = brcs.contiguous();
        at::Tensor virial = at::empty({B, 3, 3}, d.options());
        int rc = d.scalar_type() == at::kDouble
                     ? ai2b_fvt_virial_fwd_f64(virial.data_ptr<double>(), B, npad, (int)umax, iptr(bnumneigh, "bnumneigh"),
                                               fptr<double>(r, d, "brcs"), d.data_ptr<double>(), stream())
                     : ai2b_fvt_virial_fwd_f32(virial.data_ptr<float>(), B, npad, (int)umax, iptr(bnumneigh, "bnumneigh"),
                                               fptr<float>(r, d, "brcs"), d.data_ptr<float>(), stream());
        check(rc, "ai2b_fvt_virial_fwd");
        ctx->save_for_backward({bnumneigh, r, d});
        ctx->saved_data["umax"] = umax;
        return {virial};
    }
    static variable_list backward(AutogradContext *ctx, variable_list grads)
    {
        auto saved = ctx->get_saved_variables();
        const at::Tensor &bnumneigh = saved[0], &r = saved[1], &d = saved[2];
        const int64_t umax = ctx->saved_data["umax"].toInt();
        at::Tensor g = grads[0].contiguous();
        c10::cuda::CUDAGuard guard(g.device());
        const int B = (int)bnumneigh.size(0), npad = (int)bnumneigh.size(1);
        at::Tensor gde = at::empty({B, npad, umax, 3}, g.options()), grc = at::empty({B, npad, umax, 3}, g.options());
        int rc = g.scalar_type() == at::kDouble
                     ? ai2b_fvt_virial_bwd_f64(gde.data_ptr<double>(), grc.data_ptr<double>(), B, npad, (int)umax,
                                               iptr(bnumneigh, "bnumneigh"), r.data_ptr<double>(), d.data_ptr<double>(),
                                               g.data_ptr<double>(), stream())
                     : ai2b_fvt_virial_bwd_f32(gde.data_ptr<float>(), grc.data_ptr<float>(), B, npad, (int)umax,
                                               iptr(bnumneigh, "bnumneigh"), r.data_ptr<float>(), d.data_ptr<float>(),
                                               g.data_ptr<float>(), stream());
        check(rc, "ai2b_fvt_virial_bwd");
        // the reference returns the gradient w.r.t. rcs as well (virial_sr_op.cc:87-163)
        return {at::Tensor(), grc, at::Tensor(), gde};
    }
};

}  // namespace

TORCH_LIBRARY(fvt, m)
{
    m.def("ForceSrOp", [](const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor, const at::Tensor &bnumneigh_tensor,
                          const at::Tensor &bfirstneigh_tensor, int64_t nghost, int64_t umax_num_neighs,
                          const at::Tensor &bdei_drij_tensor) {
        return ForceSrFunction::apply(binum_tensor, bilist_tensor, bnumneigh_tensor, bfirstneigh_tensor, nghost, umax_num_neighs,
                                      bdei_drij_tensor);
    });
    m.def("VirialSrOp", [](const at::Tensor &bnumneigh_tensor, const at::Tensor &brcs_tensor, int64_t umax_num_neighs,
                           const at::Tensor &bdei_drij_tensor) {
        return VirialSrFunction::apply(bnumneigh_tensor, brcs_tensor, umax_num_neighs, bdei_drij_tensor);
    });
}
