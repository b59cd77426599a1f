// TEST INFRASTRUCTURE — not part of the shipped library.
//
// C entry points over the UNMODIFIED reference CPU implementation (lhycms/AI2Pot),
// compiled from the reference's own headers where they lie (nothing is copied):
//   source/nblist/include/{structure,binLinkedList,neighborList}.h
//   source/descriptor/mtpr/include/{linearMtp_cpu_launcher,linearMtpLoss_cpu_launcher}.h
//   source/descriptor/mtpr/src/mtpParam.cc
//   source/descriptor/nep/include/{nep_cpu_launcher,nepLoss_cpu_launcher}.h
//   source/fvt/include/{force_sr,virial_sr}.h
//   source/descriptor/correction/include/zbl.h
//   source/descriptor/fitutils/include/{descriptorsStatistics,targetStatistics}.h
// The resulting shared object (oracle/_ref/libai2pot_ref.so) is used only by the
// tests, the smoke check and the CPU-baseline leg of the benchmark, as the checker
// and the timed CPU baseline; the product never loads it.
//
// Every function here is a thin call into a reference launcher; argument meaning is
// the reference's (see the cited launcher).
#include <cstring>
#include <cstdlib>
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>
#include <algorithm>

#include "nblist/include/structure.h"
#include "nblist/include/neighborList.h"
#include "descriptor/mtpr/include/mtpParam.h"
#include "descriptor/mtpr/include/linearMtp_cpu_launcher.h"
#include "descriptor/mtpr/include/linearMtpLoss_cpu_launcher.h"
#include "descriptor/nep/include/nep_cpu_launcher.h"
#include "descriptor/nep/include/nepLoss_cpu_launcher.h"
#include "fvt/include/force_sr.h"
#include "fvt/include/virial_sr.h"
#include "descriptor/correction/include/zbl.h"
#include "descriptor/fitutils/include/descriptorsStatistics.h"
#include "descriptor/fitutils/include/targetStatistics.h"

namespace {

template <typename T>
int nblist_impl(int natoms, const T *cell, const int *types, const T *coords, int is_cart,
                double rcut, const int *pbc, int sort, int umax,
                int *numneigh, int *firstneigh, T *rcs, int *types_out, int *max_nn)
{
    // nblist/bind/nblist_bind.cc:87-136 (float build casts rcut to float first)
    ai2pot::Structure<T> structure(natoms, const_cast<T *>(cell), const_cast<int *>(types),
                                   const_cast<T *>(coords), is_cart != 0);
    bool pbc_xyz[3] = {pbc[0] != 0, pbc[1] != 0, pbc[2] != 0};
    ai2pot::NeighborList<T> nl(structure, (T)rcut, pbc_xyz, sort != 0);
    int mx = nl.get_max_num_neigh_atoms();
    if (max_nn) *max_nn = mx;
    if (mx > umax) return -1;          // the reference would overrun its buffers here
    if (!numneigh) return 0;           // count-only query
    int inum = 0, nghost = 0;
    std::vector<int> ilist(natoms);
    nl.find_info4mlff(inum, ilist.data(), numneigh, firstneigh, rcs, types_out, nghost, umax);
    return 0;
}

}  // namespace

extern "C" {

// ---- neighbour list: nblist/include/neighborList.h:178-189,532-578 -------------------
int ref_nblist_f64(int natoms, const double *cell, const int *types, const double *coords,
                   int is_cart, double rcut, const int *pbc, int sort, int umax,
                   int *numneigh, int *firstneigh, double *rcs, int *types_out, int *max_nn)
{
    return nblist_impl<double>(natoms, cell, types, coords, is_cart, rcut, pbc, sort, umax,
                               numneigh, firstneigh, rcs, types_out, max_nn);
}
int ref_nblist_f32(int natoms, const float *cell, const int *types, const float *coords,
                   int is_cart, double rcut, const int *pbc, int sort, int umax,
                   int *numneigh, int *firstneigh, float *rcs, int *types_out, int *max_nn)
{
    return nblist_impl<float>(natoms, cell, types, coords, is_cart, rcut, pbc, sort, umax,
                              numneigh, firstneigh, rcs, types_out, max_nn);
}

// ---- .almtp parser: descriptor/mtpr/src/mtpParam.cc:80-200 ---------------------------
// Two-call protocol: counts first (arrays NULL), then the arrays.
int ref_mtp_param_file(const char *filename, int *counts /*[5]: nm, nb, nt, ns, nmus*/,
                       int *basic, int *times, int *mapping)
{
    try {
        ai2pot::mtpr::MtpParam p{std::string(filename)};
        counts[0] = p.alpha_moments_count();
        counts[1] = p.alpha_index_basic_count();
        counts[2] = p.alpha_index_times_count();
        counts[3] = p.alpha_scalar_moments();
        counts[4] = p.nmus();
        if (basic) std::memcpy(basic, p.alpha_index_basic(), sizeof(int) * 4 * counts[1]);
        if (times) std::memcpy(times, p.alpha_index_times(), sizeof(int) * 4 * counts[2]);
        if (mapping) std::memcpy(mapping, p.alpha_moment_mapping(), sizeof(int) * counts[3]);
    } catch (...) {
        return -1;
    }
    return 0;
}

// ---- linear MTP: descriptor/mtpr/include/linearMtp_cpu_launcher.h:128-345 ------------
#define MTP_TABLE_ARGS                                                                       \
    int alpha_moments_count, int alpha_index_basic_count, const int *alpha_index_basic,      \
    int alpha_index_times_count, const int *alpha_index_times, int alpha_scalar_moments,     \
    const int *alpha_moment_mapping, int nmus
#define MTP_TABLE_PASS                                                                       \
    alpha_moments_count, alpha_index_basic_count, (const int (*)[4])alpha_index_basic,       \
    alpha_index_times_count, (const int (*)[4])alpha_index_times, alpha_scalar_moments,      \
    alpha_moment_mapping, nmus
#define NB_ARGS(T)                                                                           \
    int batch_size, int natoms_pad, int *binum, int *bilist, int *bnumneigh,                 \
    int *bfirstneigh, T *brcs, int *btypes, int ntypes, int *type_map, int umax, int nghost
#define NB_PASS(T)                                                                           \
    batch_size, natoms_pad, binum, bilist, bnumneigh, bfirstneigh, (T (*)[3])brcs, btypes,   \
    ntypes, type_map, umax, nghost

#define DEF_MTP(T, SUF)                                                                      \
void ref_mtp_efv_##SUF(T *betot, T *bforce, T *bvirial, int chebyshev_size, T scaling,       \
                       T *coeffs, T *linear_coeffs, T *type_bias, MTP_TABLE_ARGS,            \
                       NB_ARGS(T), T rmax, T rmin, T *q_scaler)                              \
{                                                                                            \
    ai2pot::mtpr::find_efv_cpu_launcher<T>(betot, (T (*)[3])bforce, bvirial, chebyshev_size, \
        scaling, coeffs, linear_coeffs, type_bias, MTP_TABLE_PASS, NB_PASS(T), rmax, rmin,   \
        q_scaler);                                                                           \
}                                                                                            \
void ref_mtp_ef_##SUF(T *betot, T *bforce, int chebyshev_size, T scaling, T *coeffs,         \
                      T *linear_coeffs, T *type_bias, MTP_TABLE_ARGS, NB_ARGS(T), T rmax,    \
                      T rmin, T *q_scaler)                                                   \
{                                                                                            \
    ai2pot::mtpr::find_ef_cpu_launcher<T>(betot, (T (*)[3])bforce, chebyshev_size, scaling,  \
        coeffs, linear_coeffs, type_bias, MTP_TABLE_PASS, NB_PASS(T), rmax, rmin, q_scaler); \
}                                                                                            \
void ref_mtp_descriptors_##SUF(T *bdesc, int chebyshev_size, T scaling, T *coeffs,           \
                               MTP_TABLE_ARGS, NB_ARGS(T), T rmax, T rmin)                   \
{                                                                                            \
    ai2pot::mtpr::find_descriptors_cpu_launcher<T>(bdesc, chebyshev_size, scaling, coeffs,   \
        MTP_TABLE_PASS, NB_PASS(T), rmax, rmin);                                             \
}                                                                                            \
/* descriptor/mtpr/include/linearMtpLoss_cpu_launcher.h:152-533 */                           \
void ref_mtp_loss_##SUF(T *bloss, int batch_size, int natoms_pad, int *binum, int *bilist,   \
                        T e_w, T f_w, T v_w, T *betot_ml, T *betot_dft, T *bforce_ml,        \
                        T *bforce_dft, T *bvirial_ml, T *bvirial_dft)                        \
{                                                                                            \
    ai2pot::mtpr::find_loss_cpu_launcher<T>(bloss, batch_size, natoms_pad, binum, bilist,    \
        e_w, f_w, v_w, betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft,       \
        bvirial_ml, bvirial_dft);                                                            \
}                                                                                            \
void ref_mtp_ef_loss_##SUF(T *bloss, int batch_size, int natoms_pad, int *binum,             \
                           int *bilist, T e_w, T f_w, T *betot_ml, T *betot_dft,             \
                           T *bforce_ml, T *bforce_dft)                                      \
{                                                                                            \
    ai2pot::mtpr::find_ef_loss_cpu_launcher<T>(bloss, batch_size, natoms_pad, binum, bilist, \
        e_w, f_w, betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft);           \
}                                                                                            \
void ref_mtp_loss_backward_##SUF(T *dcoeffs, T *dlinear, T *dbias, T e_w, T f_w, T v_w,      \
                                 T *betot_ml, T *betot_dft, T *bforce_ml, T *bforce_dft,     \
                                 T *bvirial_ml, T *bvirial_dft, int chebyshev_size,          \
                                 T scaling, T *coeffs, T *linear_coeffs, T *type_bias,       \
                                 MTP_TABLE_ARGS, NB_ARGS(T), T rmax, T rmin, T *q_scaler)    \
{                                                                                            \
    ai2pot::mtpr::find_loss_backward_cpu_launcher<T>(dcoeffs, dlinear, dbias, e_w, f_w, v_w, \
        betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft, bvirial_ml,          \
        bvirial_dft, chebyshev_size, scaling, coeffs, linear_coeffs, type_bias,              \
        MTP_TABLE_PASS, NB_PASS(T), rmax, rmin, q_scaler);                                   \
}                                                                                            \
void ref_mtp_ef_loss_backward_##SUF(T *dcoeffs, T *dlinear, T *dbias, T e_w, T f_w,          \
                                    T *betot_ml, T *betot_dft, T *bforce_ml, T *bforce_dft,  \
                                    int chebyshev_size, T scaling, T *coeffs,                \
                                    T *linear_coeffs, T *type_bias, MTP_TABLE_ARGS,          \
                                    NB_ARGS(T), T rmax, T rmin, T *q_scaler)                 \
{                                                                                            \
    ai2pot::mtpr::find_ef_loss_backward_cpu_launcher<T>(dcoeffs, dlinear, dbias, e_w, f_w,   \
        betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft, chebyshev_size,      \
        scaling, coeffs, linear_coeffs, type_bias, MTP_TABLE_PASS, NB_PASS(T), rmax, rmin,   \
        q_scaler);                                                                           \
}

DEF_MTP(double, f64)
DEF_MTP(float, f32)

// ---- NEP: descriptor/nep/include/nep_cpu_launcher.h:116-317 --------------------------
#define DEF_NEP(T, SUF)                                                                      \
void ref_nep_efv_##SUF(T *betot, T *bforce, T *bvirial, int chebyshev_size, int n_radial,    \
                       int n_angular, int l_max, int num_neurons, T *coeffs, T *w0, T *b0,   \
                       T *w1, T *type_bias, NB_ARGS(T), T rmax_radial, T rmax_angular,       \
                       T *q_scaler)                                                          \
{                                                                                            \
    ai2pot::nep::find_efv_cpu_launcher<T>(betot, (T (*)[3])bforce, bvirial, chebyshev_size,  \
        n_radial, n_angular, l_max, num_neurons, coeffs, w0, b0, w1, type_bias, NB_PASS(T),  \
        rmax_radial, rmax_angular, q_scaler);                                                \
}                                                                                            \
void ref_nep_ef_##SUF(T *betot, T *bforce, int chebyshev_size, int n_radial, int n_angular,  \
                      int l_max, int num_neurons, T *coeffs, T *w0, T *b0, T *w1,            \
                      T *type_bias, NB_ARGS(T), T rmax_radial, T rmax_angular, T *q_scaler)  \
{                                                                                            \
    ai2pot::nep::find_ef_cpu_launcher<T>(betot, (T (*)[3])bforce, chebyshev_size, n_radial,  \
        n_angular, l_max, num_neurons, coeffs, w0, b0, w1, type_bias, NB_PASS(T),            \
        rmax_radial, rmax_angular, q_scaler);                                                \
}                                                                                            \
void ref_nep_descriptors_##SUF(T *bdesc, int chebyshev_size, int n_radial, int n_angular,    \
                               int l_max, T *coeffs, NB_ARGS(T), T rmax_radial,              \
                               T rmax_angular)                                               \
{                                                                                            \
    ai2pot::nep::find_descriptors_cpu_launcher<T>(bdesc, chebyshev_size, n_radial,           \
        n_angular, l_max, coeffs, NB_PASS(T), rmax_radial, rmax_angular);                    \
}

DEF_NEP(double, f64)
DEF_NEP(float, f32)

// ---- NEP loss gradient: descriptor/nep/include/nepLoss_cpu_launcher.h:69-160,213-330 ------------------
#define DEF_NEP_LOSS(T, SUF)                                                                 \
void ref_nep_loss_backward_##SUF(T *dcoeffs, T *dw0, T *db0, T *dw1, T *dbias, T e_w, T f_w, T v_w, \
                                 T *betot_ml, T *betot_dft, T *bforce_ml, T *bforce_dft,     \
                                 T *bvirial_ml, T *bvirial_dft, int chebyshev_size, int n_radial, \
                                 int n_angular, int l_max, int num_neurons, T *coeffs, T *w0, T *b0, \
                                 T *w1, T *type_bias, NB_ARGS(T), T rmax_radial, T rmax_angular, \
                                 T *q_scaler)                                                \
{                                                                                            \
    ai2pot::nep::find_loss_backward_cpu_launcher<T>(dcoeffs, dw0, db0, dw1, dbias, e_w, f_w, v_w, \
        betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft, bvirial_ml, bvirial_dft, \
        chebyshev_size, n_radial, n_angular, l_max, num_neurons, coeffs, w0, b0, w1, type_bias, \
        NB_PASS(T), rmax_radial, rmax_angular, q_scaler);                                    \
}                                                                                            \
void ref_nep_ef_loss_backward_##SUF(T *dcoeffs, T *dw0, T *db0, T *dw1, T *dbias, T e_w, T f_w, \
                                    T *betot_ml, T *betot_dft, T *bforce_ml, T *bforce_dft,  \
                                    int chebyshev_size, int n_radial, int n_angular, int l_max, \
                                    int num_neurons, T *coeffs, T *w0, T *b0, T *w1, T *type_bias, \
                                    NB_ARGS(T), T rmax_radial, T rmax_angular, T *q_scaler)  \
{                                                                                            \
    ai2pot::nep::find_ef_loss_backward_cpu_launcher<T>(dcoeffs, dw0, db0, dw1, dbias, e_w, f_w, \
        betot_ml, betot_dft, (T (*)[3])bforce_ml, (T (*)[3])bforce_dft, chebyshev_size, n_radial, \
        n_angular, l_max, num_neurons, coeffs, w0, b0, w1, type_bias, NB_PASS(T), rmax_radial, \
        rmax_angular, q_scaler);                                                             \
}

DEF_NEP_LOSS(double, f64)
DEF_NEP_LOSS(float, f32)

// ---- fvt: fvt/include/force_sr.h:50-81, virial_sr.h:24-51 (values only) ---------------
#define DEF_FVT(T, SUF)                                                                      \
void ref_fvt_force_##SUF(T *force, int inum, int *ilist, int *numneigh, int *firstneigh,     \
                         int nghost, int umax, T *dei_drij)                                  \
{                                                                                            \
    std::vector<T> der((size_t)(inum + nghost) * 3 * inum * umax);                           \
    ai2pot::fvt::ForceSr<T>::find_val_der(force, der.data(), inum, ilist, numneigh,          \
        firstneigh, nghost, umax, dei_drij);                                                 \
}                                                                                            \
void ref_fvt_virial_##SUF(T *virial, int inum, int *numneigh, T *rcs, int umax, T *dei_drij) \
{                                                                                            \
    std::vector<T> d1((size_t)9 * inum * umax), d2((size_t)9 * inum * umax);                 \
    ai2pot::fvt::VirialSr<T>::find_val_der(virial, d1.data(), d2.data(), inum, numneigh,     \
        rcs, umax, dei_drij);                                                                \
}

DEF_FVT(double, f64)
DEF_FVT(float, f32)

// ---- ZBL pair correction: descriptor/correction/include/zbl.h -----------------------------------
// zbl_efv: the complete correction as the reference's CUDA path applies it
// (descriptor/correction/gpu/include/zbl.cuh:423-500: energy, force on the centre atom, virial, per
// directed pair), composed here from the reference's own CPU pair methods
// (PairZBL::add_atomic_energy_one / add_atomic_force_one / add_virial_one, zbl.h:330-395).
// zbl_cpu_efv / zbl_cpu_ef: GroupZBL::correct_efv / correct_ef exactly as the CPU ops call them
// (zbl.h:491-622; correct_efv adds the energy only, correct_ef energy and force).
#define DEF_ZBL(T, SUF)                                                                              \
void ref_zbl_efv_##SUF(T *etot, T *force, T *virial, int inum, int *ilist, int *numneigh,            \
                       int *firstneigh, T *rcs, int *types, int ntypes, int *type_map, int umax,     \
                       int nghost, T rmax, T rmin, T *cks, T *dks)                                   \
{                                                                                                    \
    (void)nghost;                                                                                    \
    for (int ii = 0; ii < inum; ii++) {                                                              \
        const int ci = ilist[ii], ti = types[ci];                                                    \
        for (int jj = 0; jj < numneigh[ii]; jj++) {                                                  \
            const int tj = types[firstneigh[(size_t)ii * umax + jj]];                                \
            T vec[3] = {rcs[((size_t)ii * umax + jj) * 3], rcs[((size_t)ii * umax + jj) * 3 + 1],    \
                        rcs[((size_t)ii * umax + jj) * 3 + 2]};                                      \
            const T dist = std::sqrt(std::pow(vec[0], 2) + std::pow(vec[1], 2) + std::pow(vec[2], 2)); \
            if (dist > rmax) continue;                                                               \
            const int k = ti * ntypes + tj;                                                          \
            ai2pot::correction::PairZBL<T> pz(type_map[ti], type_map[tj], rmax, rmin, cks + 4 * k, dks + 4 * k); \
            pz.add_atomic_energy_one(*etot, dist);                                                   \
            pz.add_atomic_force_one(force + 3 * ci, vec);                                            \
            if (virial) pz.add_virial_one(virial, vec);                                              \
        }                                                                                            \
    }                                                                                                \
}                                                                                                    \
void ref_zbl_cpu_efv_##SUF(T *etot, T *force, T *virial, int inum, int *ilist, int *numneigh,        \
                           int *firstneigh, T *rcs, int *types, int ntypes, int *type_map, int umax, \
                           int nghost, T rmax, T rmin, T *cks, T *dks)                               \
{                                                                                                    \
    ai2pot::correction::GroupZBL<T> g(ntypes, type_map, type_map, rmax, rmin, cks, dks);             \
    g.correct_efv(*etot, force, virial, inum, ilist, numneigh, firstneigh, (T(*)[3])rcs, types,      \
                  ntypes, type_map, umax, nghost);                                                   \
}                                                                                                    \
void ref_zbl_cpu_ef_##SUF(T *etot, T *force, int inum, int *ilist, int *numneigh, int *firstneigh,   \
                          T *rcs, int *types, int ntypes, int *type_map, int umax, int nghost,       \
                          T rmax, T rmin, T *cks, T *dks)                                            \
{                                                                                                    \
    ai2pot::correction::GroupZBL<T> g(ntypes, type_map, type_map, rmax, rmin, cks, dks);             \
    g.correct_ef(*etot, force, inum, ilist, numneigh, firstneigh, (T(*)[3])rcs, types, ntypes,       \
                 type_map, umax, nghost);                                                            \
}

DEF_ZBL(double, f64)
DEF_ZBL(float, f32)

// ---- dataset statistics: descriptor/fitutils/include/descriptorsStatistics.h:76-205, targetStatistics.h:44-80
#define DEF_STATS(T, SUF)                                                                            \
void ref_desc_stats_all_##SUF(int *natoms, T *mean, T *m2, int B, int npad, int nd, int *binum, T *bdesc) \
{                                                                                                    \
    ai2pot::fitutils::AllTypeDescriptorsStatistics<T>::find_descriptors_statistics(natoms, mean, m2, B, npad, nd, binum, bdesc); \
}                                                                                                    \
void ref_desc_stats_each_##SUF(int *natoms, T *mean, T *m2, int B, int npad, int nd, int *binum,     \
                               int *bilist, int *btypes, int ntypes, T *bdesc)                       \
{                                                                                                    \
    ai2pot::fitutils::EachTypeDescriptorsStatistics<T>::find_descriptors_statistics(natoms, mean, m2, B, npad, nd, binum, bilist, \
                                                                                    btypes, ntypes, bdesc); \
}                                                                                                    \
void ref_desc_maxmin_##SUF(T *mx, T *mn, int B, int npad, int nd, int *binum, T *bdesc)              \
{                                                                                                    \
    ai2pot::fitutils::AllTypeDescriptorsMaxmin<T>::find_descriptors_maxmin(mx, mn, B, npad, nd, binum, bdesc); \
}                                                                                                    \
void ref_target_stats_##SUF(int *natoms, T *out3, int B, int npad, int *binum, T *etot, T *force)    \
{                                                                                                    \
    ai2pot::fitutils::TargetStatistics<T>::find_ef_statistics(natoms, out3, out3 + 1, out3 + 2, B, npad, binum, etot, (T(*)[3])force); \
}

DEF_STATS(double, f64)
DEF_STATS(float, f32)

}  // extern "C"
