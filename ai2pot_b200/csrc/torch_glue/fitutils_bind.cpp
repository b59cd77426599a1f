// libfitutils_bind.so: fitutils::targetStatisticsOp, allTypeDescriptorsStatisticsOp,
// eachTypeDescriptorsStatisticsOp, allTypeDescriptorsMaxminOp with the reference's argument lists and
// result lists (source/descriptor/fitutils/bind/fitutils_bind.cc:25-80, src/descriptorsStatisticsOp.cc:
// 82-187,198-304,319-410, src/targetStatisticsOp.cc:28-127) over the C ABI. Not differentiable, as there.
#include "glue_common.h"

using namespace ai2b_glue;
using torch::autograd::variable_list;

namespace {

struct Dims {
    int B, npad, nd;
    bool f64;
};
Dims desc_dims(const at::Tensor &binum, const at::Tensor &bdesc)
{
    require_cuda(bdesc, "bdescriptors");
    TORCH_CHECK(bdesc.dim() == 3 && bdesc.is_contiguous(), "bdescriptors must be a contiguous [B, Np, nd] tensor");
    TORCH_CHECK(bdesc.scalar_type() == at::kDouble || bdesc.scalar_type() == at::kFloat, "bdescriptors must be float32 or float64");
    return Dims{(int)binum.size(0), (int)bdesc.size(1), (int)bdesc.size(2), bdesc.scalar_type() == at::kDouble};
}

variable_list stats(const at::Tensor &binum, const at::Tensor *bilist, const at::Tensor *btypes, int64_t ntypes, const at::Tensor &bdesc)
{
    const Dims d = desc_dims(binum, bdesc);
    c10::cuda::CUDAGuard guard(bdesc.device());
    const bool each = btypes != nullptr;
    auto iopt = bdesc.options().dtype(at::kInt);
    at::Tensor n = each ? at::zeros({ntypes}, iopt) : at::zeros({}, iopt);
    at::Tensor mean = each ? at::zeros({ntypes, d.nd}, bdesc.options()) : at::zeros({d.nd}, bdesc.options());
    at::Tensor m2 = at::zeros_like(mean);
    int rc;
    if (d.f64)
        rc = each ? ai2b_desc_stats_each_f64(n.data_ptr<int>(), mean.data_ptr<double>(), m2.data_ptr<double>(), d.B, d.npad, d.nd,
                                             iptr(binum, "binum"), iptr(*bilist, "bilist"), iptr(*btypes, "btypes"), (int)ntypes,
                                             bdesc.data_ptr<double>(), stream())
                  : ai2b_desc_stats_all_f64(n.data_ptr<int>(), mean.data_ptr<double>(), m2.data_ptr<double>(), d.B, d.npad, d.nd,
                                            iptr(binum, "binum"), bdesc.data_ptr<double>(), stream());
    else
        rc = each ? ai2b_desc_stats_each_f32(n.data_ptr<int>(), mean.data_ptr<float>(), m2.data_ptr<float>(), d.B, d.npad, d.nd,
                                             iptr(binum, "binum"), iptr(*bilist, "bilist"), iptr(*btypes, "btypes"), (int)ntypes,
                                             bdesc.data_ptr<float>(), stream())
                  : ai2b_desc_stats_all_f32(n.data_ptr<int>(), mean.data_ptr<float>(), m2.data_ptr<float>(), d.B, d.npad, d.nd,
                                            iptr(binum, "binum"), bdesc.data_ptr<float>(), stream());
    check(rc, "ai2b_desc_stats");
    return {n, mean, m2};
}

}  // namespace

TORCH_LIBRARY(fitutils, m)
{
    m.def("targetStatisticsOp", [](const at::Tensor &binum_tensor, const at::Tensor &betot_dft_tensor, const at::Tensor &bforce_dft_tensor) {
        require_cuda(betot_dft_tensor, "betot_dft");
        c10::cuda::CUDAGuard guard(betot_dft_tensor.device());
        const int B = (int)binum_tensor.size(0), npad = (int)bforce_dft_tensor.size(1);
        at::Tensor n = at::zeros({}, betot_dft_tensor.options().dtype(at::kInt)), out = at::zeros({3}, betot_dft_tensor.options());
        at::Tensor e = betot_dft_tensor.contiguous(), f = bforce_dft_tensor.contiguous();
        int rc;
        if (e.scalar_type() == at::kDouble)
            rc = ai2b_target_stats_f64(n.data_ptr<int>(), out.data_ptr<double>(), B, npad, iptr(binum_tensor, "binum"), e.data_ptr<double>(),
                                       fptr<double>(f, e, "bforce_dft"), stream());
        else
            rc = ai2b_target_stats_f32(n.data_ptr<int>(), out.data_ptr<float>(), B, npad, iptr(binum_tensor, "binum"), e.data_ptr<float>(),
                                       fptr<float>(f, e, "bforce_dft"), stream());
        check(rc, "ai2b_target_stats");
        return variable_list{n, out[0], out[1], out[2]};
    });
    m.def("allTypeDescriptorsStatisticsOp", [](const at::Tensor &binum_tensor, const at::Tensor &bdescriptors_tensor) {
        return stats(binum_tensor, nullptr, nullptr, 1, bdescriptors_tensor);
    });
    m.def("eachTypeDescriptorsStatisticsOp", [](const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor,
                                                const at::Tensor &btypes_tensor, int64_t ntypes, const at::Tensor &bdescriptors_tensor) {
        return stats(binum_tensor, &bilist_tensor, &btypes_tensor, ntypes, bdescriptors_tensor);
    });
    m.def("allTypeDescriptorsMaxminOp", [](const at::Tensor &binum_tensor, const at::Tensor &bdescriptors_tensor) {
        const Dims d = desc_dims(binum_tensor, bdescriptors_tensor);
        c10::cuda::CUDAGuard guard(bdescriptors_tensor.device());
        at::Tensor mx = at::zeros({d.nd}, bdescriptors_tensor.options()), mn = at::zeros({d.nd}, bdescriptors_tensor.options());
        int rc = d.f64 ? ai2b_desc_maxmin_f64(mx.data_ptr<double>(), mn.data_ptr<double>(), d.B, d.npad, d.nd, iptr(binum_tensor, "binum"),
                                              bdescriptors_tensor.data_ptr<double>(), stream())
                       : ai2b_desc_maxmin_f32(mx.data_ptr<float>(), mn.data_ptr<float>(), d.B, d.npad, d.nd, iptr(binum_tensor, "binum"),
                                              bdescriptors_tensor.data_ptr<float>(), stream());
        check(rc, "ai2b_desc_maxmin");
        return variable_list{mx, mn};
    });
}
