// libmtpr_bind.so: the mtpr:: torch ops of the hot path, with the reference's names and
// argument lists (source/descriptor/mtpr/bind/mtpr_bind.cc:30-567), over the C ABI.
//   mtpr::set_ai2pot_path, mtpr::mtpParamOp, mtpr::linearMtpToEFVOp, mtpr::linearMtpToEFOp,
//   mtpr::linearMtpToDescriptorsOp, mtpr::linearMtpToLossOp, mtpr::linearMtpToEFLossOp
#include "glue_common.h"

#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <tuple>
#include <vector>

using namespace ai2b_glue;
using torch::autograd::variable_list;

namespace {

std::string g_ai2pot_path;

// template directory, as source/descriptor/mtpr/src/mtpParam.cc:36-42 resolves it
std::string template_dir()
{
    const char *env = std::getenv("AI2POT_PATH");
    if (env) return std::string(env) + "/source/descriptor/mtpr/MTP_templates/";
    return g_ai2pot_path + "/_data/MTP_templates/";
}

std::string template_file(int level)
{
    TORCH_CHECK(level >= 2 && level <= 28 && level % 2 == 0, "mtp level must be an even number (2 ~ 28)");
    char name[64];
    if (level <= 4) snprintf(name, sizeof(name), "depreciated-0%d.almtp", level);
    else snprintf(name, sizeof(name), "%02d.almtp", level);
    return template_dir() + name;
}

// Compiled programs are cached per (alpha tables, device). An entry keeps references to the three
// table tensors it was compiled from: while it is cached their storage cannot be freed, so another
// model's tables can never appear at the same addresses, and a hit is confirmed by the tensors'
// version counters (an in-place edit of a table recompiles). The cache holds the most recently used
// MAX_PROGRAMS entries; an evicted program is destroyed (cudaFree waits for work that still uses it).
struct ProgEntry {
    at::Tensor basic, times, map;
    int64_t vb, vt, vm;
    int nm, nmus, dev;
    ai2b_mtp_program *prog;
    uint64_t used;
};
constexpr size_t MAX_PROGRAMS = 16;
std::vector<ProgEntry> g_programs;
uint64_t g_clock = 0;
std::mutex g_mutex;

int64_t version_of(const at::Tensor &t) { return t.is_inference() ? 0 : (int64_t)t._version(); }

const ai2b_mtp_program *program_for(int nm, const at::Tensor &basic, const at::Tensor &times, const at::Tensor &map, int nmus,
                                    int dev)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    for (auto &e : g_programs)
        if (e.basic.data_ptr() == basic.data_ptr() && e.times.data_ptr() == times.data_ptr() && e.map.data_ptr() == map.data_ptr() &&
            e.basic.sizes() == basic.sizes() && e.times.sizes() == times.sizes() && e.map.sizes() == map.sizes() && e.nm == nm &&
            e.nmus == nmus && e.dev == dev && e.vb == version_of(basic) && e.vt == version_of(times) && e.vm == version_of(map)) {
            e.used = ++g_clock;
            return e.prog;
        }
    at::Tensor hb = basic.to(at::kCPU, at::kInt).contiguous(), ht = times.to(at::kCPU, at::kInt).contiguous(),
               hm = map.to(at::kCPU, at::kInt).contiguous();
    ai2b_mtp_program *prog = nullptr;
    check(ai2b_mtp_program_create(nm, (int)basic.size(0), hb.data_ptr<int>(), (int)times.size(0), ht.data_ptr<int>(), (int)map.size(0),
                                  hm.data_ptr<int>(), nmus, &prog),
          "ai2b_mtp_program_create");
    if (g_programs.size() >= MAX_PROGRAMS) {
        size_t old = 0;
        for (size_t i = 1; i < g_programs.size(); i++)
            if (g_programs[i].used < g_programs[old].used) old = i;
        ai2b_mtp_program_destroy(g_programs[old].prog);
        g_programs.erase(g_programs.begin() + old);
    }
    g_programs.push_back(ProgEntry{basic, times, map, version_of(basic), version_of(times), version_of(map), nm, nmus, dev, prog,
                                   ++g_clock});
    return prog;
}

struct Nb {
    int B, npad, umax, ntypes;
};

template <typename T>
variable_list efv_impl(bool with_virial, int64_t cs, double scaling, const at::Tensor &coeffs, const at::Tensor &lin,
                       const at::Tensor &bias, int64_t nm, const at::Tensor &basic, const at::Tensor &times, const at::Tensor &map,
                       int64_t nmus, const at::Tensor &binum, const at::Tensor &bilist, const at::Tensor &bnumneigh,
                       const at::Tensor &bfirstneigh, const at::Tensor &brcs, const at::Tensor &btypes, const at::Tensor &type_map,
                       int64_t nghost, double rmax, double rmin, const at::Tensor &qs)
{
    require_cuda(brcs, "brcs");
    c10::cuda::CUDAGuard guard(brcs.device());
    const int B = (int)binum.size(0), npad = (int)bnumneigh.size(1), umax = (int)bfirstneigh.size(2), ntypes = (int)type_map.size(0);
    const ai2b_mtp_program *prog = program_for((int)nm, basic, times, map, (int)nmus, brcs.get_device());
    // outputs shaped as the reference allocates them (src/linearMtpOp.cc:2890-2892)
    at::Tensor e = at::empty({B}, brcs.options()), f = at::empty({B, npad + nghost, 3}, brcs.options());
    at::Tensor v = with_virial ? at::empty({B, 9}, brcs.options()) : at::Tensor();
    at::Tensor ws = workspace(ai2b_mtp_workspace_bytes(prog, B, npad, ntypes), brcs);
    auto fn = [&](auto tag) {
        using U = decltype(tag);
        if constexpr (std::is_same<U, double>::value)
            return ai2b_mtp_efv_f64(prog, e.data_ptr<double>(), f.data_ptr<double>(), with_virial ? v.data_ptr<double>() : nullptr,
                                    (int)cs, scaling, fptr<double>(coeffs, brcs, "coeffs"), fptr<double>(lin, brcs, "linear_coeffs"),
                                    fptr<double>(bias, brcs, "type_bias"), B, npad, iptr(binum, "binum"), iptr(bilist, "bilist"),
                                    iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"), fptr<double>(brcs, brcs, "brcs"),
                                    iptr(btypes, "btypes"), ntypes, umax, (int)nghost, rmax, rmin, fptr<double>(qs, brcs, "q_scaler"),
                                    ws.data_ptr(), (size_t)ws.numel(), stream());
        else
            return ai2b_mtp_efv_f32(prog, e.data_ptr<float>(), f.data_ptr<float>(), with_virial ? v.data_ptr<float>() : nullptr,
                                    (int)cs, (float)scaling, fptr<float>(coeffs, brcs, "coeffs"), fptr<float>(lin, brcs, "linear_coeffs"),
                                    fptr<float>(bias, brcs, "type_bias"), B, npad, iptr(binum, "binum"), iptr(bilist, "bilist"),
                                    iptr(bnumneigh, "bnumneigh"), iptr(bfirstneigh, "bfirstneigh"), fptr<float>(brcs, brcs, "brcs"),
                                    iptr(btypes, "btypes"), ntypes, umax, (int)nghost, (float)rmax, (float)rmin,
                                    fptr<float>(qs, brcs, "q_scaler"), ws.data_ptr(), (size_t)ws.numel(), stream());
    };
    check(fn(T{}), "ai2b_mtp_efv");
    if (with_virial) return {e, f, v};
    return {e, f};
}

variable_list efv_dispatch(bool with_virial, int64_t cs, double scaling, const at::Tensor &coeffs, const at::Tensor &lin,
                           const at::Tensor &bias, int64_t nm, const at::Tensor &basic, const at::Tensor &times,
                           const at::Tensor &map, int64_t nmus, const at::Tensor &binum, const at::Tensor &bilist,
                           const at::Tensor &bnumneigh, const at::Tensor &bfirstneigh, const at::Tensor &brcs,
                           const at::Tensor &btypes, const at::Tensor &type_map, int64_t nghost, double rmax, double rmin,
                           const at::Tensor &qs, const ZblArgs &zbl)
{
    TORCH_CHECK(brcs.scalar_type() == at::kDouble || brcs.scalar_type() == at::kFloat, "brcs must be float32 or float64");
    variable_list out = brcs.scalar_type() == at::kDouble
        ? efv_impl<double>(with_virial, cs, scaling, coeffs, lin, bias, nm, basic, times, map, nmus, binum, bilist, bnumneigh,
                           bfirstneigh, brcs, btypes, type_map, nghost, rmax, rmin, qs)
        : efv_impl<float>(with_virial, cs, scaling, coeffs, lin, bias, nm, basic, times, map, nmus, binum, bilist, bnumneigh,
                          bfirstneigh, brcs, btypes, type_map, nghost, rmax, rmin, qs);
    // the reference's CUDA op adds the correction before its kernels accumulate (linearMtpOp.cc:2920-2947);
    // the sum is the same in either order
    apply_zbl(zbl, out[0], out[1], with_virial ? out[2] : at::Tensor(), binum, bilist, bnumneigh, bfirstneigh, brcs, btypes, type_map,
              nghost);
    return out;
}

variable_list descriptors_dispatch(int64_t cs, double scaling, const at::Tensor &coeffs, int64_t nm, const at::Tensor &basic,
                                   const at::Tensor &times, const at::Tensor &map, int64_t nmus, const at::Tensor &binum,
                                   const at::Tensor &bilist, const at::Tensor &bnumneigh, const at::Tensor &bfirstneigh,
                                   const at::Tensor &brcs, const at::Tensor &btypes, const at::Tensor &type_map, int64_t nghost,
                                   double rmax, double rmin)
{
    require_cuda(brcs, "brcs");
    c10::cuda::CUDAGuard guard(brcs.device());
    const int B = (int)binum.size(0), npad = (int)bnumneigh.size(1), umax = (int)bfirstneigh.size(2), ntypes = (int)type_map.size(0);
    const ai2b_mtp_program *prog = program_for((int)nm, basic, times, map, (int)nmus, brcs.get_device());
    at::Tensor d = at::empty({B, npad, map.size(0)}, brcs.options());
    at::Tensor ws = workspace(ai2b_mtp_workspace_bytes(prog, B, npad, ntypes), brcs);
    int rc;
    if (brcs.scalar_type() == at::kDouble)
        rc = ai2b_mtp_descriptors_f64(prog, d.data_ptr<double>(), (int)cs, scaling, fptr<double>(coeffs, brcs, "coeffs"), B, npad,
                                      iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"),
                                      iptr(bfirstneigh, "bfirstneigh"), fptr<double>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes,
                                      umax, (int)nghost, rmax, rmin, ws.data_ptr(), (size_t)ws.numel(), stream());
    else
        rc = ai2b_mtp_descriptors_f32(prog, d.data_ptr<float>(), (int)cs, (float)scaling, fptr<float>(coeffs, brcs, "coeffs"), B, npad,
                                      iptr(binum, "binum"), iptr(bilist, "bilist"), iptr(bnumneigh, "bnumneigh"),
                                      iptr(bfirstneigh, "bfirstneigh"), fptr<float>(brcs, brcs, "brcs"), iptr(btypes, "btypes"), ntypes,
                                      umax, (int)nghost, (float)rmax, (float)rmin, ws.data_ptr(), (size_t)ws.numel(), stream());
    check(rc, "ai2b_mtp_descriptors");
    return {d};
}

// mtpParamOp: the seven tensors of src/mtpParamOp.cc:24-72 (CPU int32): alpha_moments_count,
// alpha_index_basic, alpha_index_times, alpha_moment_mapping, num_mus4moms, mus4moms, nmus
variable_list mtp_param(int64_t level)
{
    const std::string file = template_file((int)level);
    int counts[5];
    check(ai2b_mtp_parse_almtp(file.c_str(), counts, nullptr, nullptr, nullptr), "ai2b_mtp_parse_almtp");
    auto opt = at::TensorOptions().dtype(at::kInt);
    at::Tensor basic = at::zeros({counts[1], 4}, opt), times = at::zeros({counts[2], 4}, opt), map = at::zeros({counts[3]}, opt);
    check(ai2b_mtp_parse_almtp(file.c_str(), counts, basic.data_ptr<int>(), times.data_ptr<int>(), map.data_ptr<int>()),
          "ai2b_mtp_parse_almtp");
    // radial-function indices every moment depends on (src/mtpParam.cc _get_mus4all_mom_dp)
    const int nm = counts[0];
    std::vector<std::set<int>> mus(nm);
    const int *pb = basic.data_ptr<int>(), *pt = times.data_ptr<int>();
    for (int i = 0; i < counts[1]; i++) mus[i].insert(pb[4 * i]);
    for (int t = 0; t < counts[2]; t++) {
        const int a = pt[4 * t], b = pt[4 * t + 1], d = pt[4 * t + 3];
        mus[d].insert(mus[a].begin(), mus[a].end());
        mus[d].insert(mus[b].begin(), mus[b].end());
    }
    size_t mx = 0;
    for (auto &s : mus) mx = std::max(mx, s.size());
    at::Tensor num = at::zeros({nm}, opt), all = at::full({nm, (int64_t)mx}, -1, opt);
    for (int m = 0; m < nm; m++) {
        num.data_ptr<int>()[m] = (int)mus[m].size();
        int k = 0;
        for (int v : mus[m]) all.data_ptr<int>()[m * mx + k++] = v;
    }
    return {at::tensor(counts[0], opt), basic, times, map, num, all, at::tensor(counts[4], opt)};
}

}  // namespace

#include "mtpr_loss_glue.inc"

TORCH_LIBRARY(mtpr, m)
{
    m.def("set_ai2pot_path", [](const std::string &path) { g_ai2pot_path = path; });
    m.def("mtpParamOp", [](int64_t mtp_level) { return mtp_param(mtp_level); });
    m.def("linearMtpToEFVOp",
          [](int64_t chebyshev_size, double scaling, const at::Tensor &coeffs_tensor, const at::Tensor &linear_coeffs_tensor,
             const at::Tensor &type_bias_tensor, int64_t alpha_moments_count, const at::Tensor &alpha_index_basic_tensor,
             const at::Tensor &alpha_index_times_tensor, const at::Tensor &alpha_moment_mapping_tensor, int64_t nmus,
             const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor, const at::Tensor &bnumneigh_tensor,
             const at::Tensor &bfirstneigh_tensor, const at::Tensor &brcs_tensor, const at::Tensor &btypes_tensor,
             const at::Tensor &type_map_tensor, int64_t nghost, double rmax, double rmin, const at::Tensor &q_scaler_tensor,
             double zbl_rmax, double zbl_rmin, const at::Tensor &zbl_cks_tensor, const at::Tensor &zbl_dks_tensor) {
              return efv_dispatch(true, chebyshev_size, scaling, coeffs_tensor, linear_coeffs_tensor, type_bias_tensor,
                                  alpha_moments_count, alpha_index_basic_tensor, alpha_index_times_tensor,
                                  alpha_moment_mapping_tensor, nmus, binum_tensor, bilist_tensor, bnumneigh_tensor,
                                  bfirstneigh_tensor, brcs_tensor, btypes_tensor, type_map_tensor, nghost, rmax, rmin,
                                  q_scaler_tensor, ZblArgs{zbl_rmax, zbl_rmin, zbl_cks_tensor, zbl_dks_tensor});
          });
    m.def("linearMtpToEFOp",
          [](int64_t chebyshev_size, double scaling, const at::Tensor &coeffs_tensor, const at::Tensor &linear_coeffs_tensor,
             const at::Tensor &type_bias_tensor, int64_t alpha_moments_count, const at::Tensor &alpha_index_basic_tensor,
             const at::Tensor &alpha_index_times_tensor, const at::Tensor &alpha_moment_mapping_tensor, int64_t nmus,
             const at::Tensor &binum_tensor, const at::Tensor &bilist_tensor, const at::Tensor &bnumneigh_tensor,
             const at::Tensor &bfirstneigh_tensor, const at::Tensor &brcs_tensor, const at::Tensor &btypes_tensor,
             const at::Tensor &type_map_tensor, int64_t nghost, double rmax, double rmin, const at::Tensor &q_scaler_tensor,
             double zbl_rmax, double zbl_rmin, const at::Tensor &zbl_cks_tensor, const at::Tensor &zbl_dks_tensor) {
              return efv_dispatch(false, chebyshev_size, scaling, coeffs_tensor, linear_coeffs_tensor, type_bias_tensor,
                                  alpha_moments_count, alpha_index_basic_tensor, alpha_index_times_tensor,
                                  alpha_moment_mapping_tensor, nmus, binum_tensor, bilist_tensor, bnumneigh_tensor,
                                  bfirstneigh_tensor, brcs_tensor, btypes_tensor, type_map_tensor, nghost, rmax, rmin,
                                  q_scaler_tensor, ZblArgs{zbl_rmax, zbl_rmin, zbl_cks_tensor, zbl_dks_tensor});
          });
    m.def("linearMtpToDescriptorsOp",
          [](int64_t chebyshev_size, double scaling, const at::Tensor &coeffs_tensor, int64_t alpha_moments_count,
             const at::Tensor &alpha_index_basic_tensor, const at::Tensor &alpha_index_times_tensor,
             const at::Tensor &alpha_moment_mapping_tensor, int64_t nmus, const at::Tensor &binum_tensor,
             const at::Tensor &bilist_tensor, const at::Tensor &bnumneigh_tensor, const at::Tensor &bfirstneigh_tensor,
             const at::Tensor &brcs_tensor, const at::Tensor &btypes_tensor, const at::Tensor &type_map_tensor, int64_t nghost,
             double rmax, double rmin) {
              return descriptors_dispatch(chebyshev_size, scaling, coeffs_tensor, alpha_moments_count, alpha_index_basic_tensor,
                                          alpha_index_times_tensor, alpha_moment_mapping_tensor, nmus, binum_tensor, bilist_tensor,
                                          bnumneigh_tensor, bfirstneigh_tensor, brcs_tensor, btypes_tensor, type_map_tensor, nghost,
                                          rmax, rmin);
          });
    register_loss_ops(m);
}
