/* ai2pot_b200 — C ABI of the B200 (sm_100a) per-atom evaluation path.
 *
 * Drop-in boundary: each entry point below takes what the reference's own raw-pointer
 * launcher for the same step takes (cited per function, paths relative to the reference
 * project root), plus a CUDA stream and — where the kernels need scratch — a caller-owned
 * workspace. Plain pointers and sizes only; no torch types.
 *
 * Conventions
 *  - Every function returns AI2B_OK (0) or a negative AI2B_ERR_* code and never throws;
 *    ai2b_last_error_string() gives the message of the calling thread's last failure.
 *  - Pointers named d_* are DEVICE pointers on the current device unless stated otherwise.
 *  - Calls are stream-ordered and do not synchronise; `stream` is a cudaStream_t passed as
 *    void* (NULL = the legacy default stream).
 *  - The hot calls allocate nothing: outputs and workspace come from the caller. Handles
 *    (ai2b_mtp_program) own small device tables allocated at create time.
 *  - Suffix _f32 / _f64 selects the float type of rcs, parameters and outputs, exactly as the
 *    reference dispatches on brcs.scalar_type().
 *  - Batched neighbour tensors use the reference layout: binum[B], bilist[B,Np],
 *    bnumneigh[B,Np], bfirstneigh[B,Np,umax] (padding -1), brcs[B,Np,umax,3] (r_j - r_i),
 *    btypes[B,Np+nghost]; forces [B,Np+nghost,3] indexed by atom id; virial [B,9] row-major.
 */
#ifndef AI2POT_B200_H
#define AI2POT_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AI2B_OK 0
#define AI2B_ERR_INVALID (-1)      /* bad argument (NULL pointer, negative size, unsupported value) */
#define AI2B_ERR_UNSUPPORTED (-2)  /* valid in the reference but outside this build's limits       */
#define AI2B_ERR_CUDA (-3)         /* a CUDA runtime call failed                                    */
#define AI2B_ERR_WORKSPACE (-4)    /* workspace missing or too small                                */
#define AI2B_ERR_OVERFLOW (-5)     /* a neighbour row would exceed umax (list truncated)            */
#define AI2B_ERR_TIMEOUT (-6)      /* a bounded device-side wait gave up                            */

const char *ai2b_last_error_string(void);
int ai2b_version(void);

/* ------------------------------------------------------------------------------------------
 * Linear MTP
 * ---------------------------------------------------------------------------------------- */

/* Compiled form of the alpha tables (replaces passing d_alpha_index_basic / _times /
 * _moment_mapping to every launch: source/descriptor/mtpr/gpu/include/
 * linearMtp_torch_launcher.h:24-55 takes them per call; source/descriptor/mtpr/src/
 * mtpParam.cc:80-200 produces them). Tables are HOST pointers, int32, row-major [n][4].
 * Limits: monomial degree <= 8 (template level <= 20), nmus <= 8. */
typedef struct ai2b_mtp_program ai2b_mtp_program;
int ai2b_mtp_program_create(int alpha_moments_count, int alpha_index_basic_count,
                            const int *alpha_index_basic, int alpha_index_times_count,
                            const int *alpha_index_times, int alpha_scalar_moments,
                            const int *alpha_moment_mapping, int nmus,
                            ai2b_mtp_program **out);
void ai2b_mtp_program_destroy(ai2b_mtp_program *prog);

/* Parser of the .almtp template files (source/descriptor/mtpr/src/mtpParam.cc:80-200).
 * Two-call protocol: with the array pointers NULL only counts[5] = {alpha_moments_count,
 * alpha_index_basic_count, alpha_index_times_count, alpha_scalar_moments, nmus} is filled. */
int ai2b_mtp_parse_almtp(const char *filename, int *counts, int *alpha_index_basic,
                         int *alpha_index_times, int *alpha_moment_mapping);

/* Scratch bytes the MTP calls below need for a batch of `batch_size` structures padded to
 * `natoms_pad` atoms, for a model with `ntypes` species: per-structure atom offsets, a
 * zero-padded copy of the radial coefficients, and two [atoms][dense moments] arrays that carry
 * the basic moments and their adjoints between the three kernels of a call. */
size_t ai2b_mtp_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int natoms_pad,
                                int ntypes);

/* Energy + force + virial. Replaces find_efv_torch_launcher<T>
 * (source/descriptor/mtpr/gpu/include/linearMtp_torch_launcher.h:24-55, .cuh:27-100) and the
 * CPU launcher (source/descriptor/mtpr/include/linearMtp_cpu_launcher.h:128-203).
 * Outputs are overwritten (zeroed, then accumulated). d_bvirial may be NULL: energy + force
 * only (find_ef_torch_launcher, linearMtp_torch_launcher.h:58-88). */
#define AI2B_DECL_MTP_EFV(SUF, T)                                                              \
    int ai2b_mtp_efv_##SUF(const ai2b_mtp_program *prog, T *d_betot, T *d_bforce, T *d_bvirial, \
                           int chebyshev_size, T scaling, const T *d_coeffs,                   \
                           const T *d_linear_coeffs, const T *d_type_bias, int batch_size,     \
                           int natoms_pad, const int *d_binum, const int *d_bilist,            \
                           const int *d_bnumneigh, const int *d_bfirstneigh, const T *d_brcs,  \
                           const int *d_btypes, int ntypes, int umax, int nghost, T rmax,      \
                           T rmin, const T *d_q_scaler, void *d_workspace,                     \
                           size_t workspace_bytes, void *stream);
AI2B_DECL_MTP_EFV(f64, double)
AI2B_DECL_MTP_EFV(f32, float)

/* Scalar basis values [B, Np, alpha_scalar_moments] (not divided by q_scaler). Replaces
 * find_descriptors_torch_launcher<T> (linearMtp_torch_launcher.h:90-118) /
 * find_descriptors_cpu_launcher (linearMtp_cpu_launcher.h:284-345). */
#define AI2B_DECL_MTP_DESC(SUF, T)                                                             \
    int ai2b_mtp_descriptors_##SUF(const ai2b_mtp_program *prog, T *d_bdescriptors,            \
                                   int chebyshev_size, T scaling, const T *d_coeffs,           \
                                   int batch_size, int natoms_pad, const int *d_binum,         \
                                   const int *d_bilist, const int *d_bnumneigh,                \
                                   const int *d_bfirstneigh, const T *d_brcs,                  \
                                   const int *d_btypes, int ntypes, int umax, int nghost,      \
                                   T rmax, T rmin, void *d_workspace, size_t workspace_bytes,  \
                                   void *stream);
AI2B_DECL_MTP_DESC(f64, double)
AI2B_DECL_MTP_DESC(f32, float)

/* Training path. ai2b_mtp_loss_*: per-structure weighted MSE loss[B] and the batch RMSEs
 * rmse[3] = {energy, force, virial} (LinearMtpLoss<T>::find_loss / find_ef_loss,
 * source/descriptor/mtpr/include/linearMtpLoss.h:138-210; RMSE definitions
 * source/descriptor/mtpr/src/linearMtpOp.cc:885-911). d_bvirial_ml / d_bvirial_dft NULL gives
 * the energy + force variant. Needs 32 bytes of workspace.
 * ai2b_mtp_loss_backward_*: analytic gradient of every structure's loss w.r.t. coeffs
 * [B,ntypes*ntypes*nmus*chebyshev_size], linear_coeffs [B,alpha_scalar_moments] and type_bias
 * [B,ntypes] (find_loss_backward / find_ef_loss_backward, linearMtpLoss.h:212-569; CUDA
 * launcher gpu/include/linearMtpLoss.cuh:1015). The model E/F/V of the same inputs are passed
 * in (the reference recomputes them inside its backward). Outputs are overwritten.
 * d_bforce_ml has row stride natoms_pad + nghost, d_bforce_dft natoms_pad; nghost must be 0
 * for the gradient. Workspace: ai2b_mtp_loss_workspace_bytes. */
size_t ai2b_mtp_loss_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int natoms_pad,
                                     int ntypes);
#define AI2B_DECL_MTP_LOSS(SUF, T)                                                               \
    int ai2b_mtp_loss_##SUF(T *d_bloss, T *d_rmse, int batch_size, int natoms_pad, int nghost,   \
                            const int *d_binum, const int *d_bilist, T e_weight, T f_weight,     \
                            T v_weight, const T *d_betot_ml, const T *d_betot_dft,               \
                            const T *d_bforce_ml, const T *d_bforce_dft, const T *d_bvirial_ml,  \
                            const T *d_bvirial_dft, void *d_workspace, size_t workspace_bytes,   \
                            void *stream);                                                       \
    int ai2b_mtp_loss_backward_##SUF(                                                            \
        const ai2b_mtp_program *prog, T *d_bloss_der2coeffs, T *d_bloss_der2linear_coeffs,       \
        T *d_bloss_der2type_bias, T e_weight, T f_weight, T v_weight, const T *d_betot_ml,       \
        const T *d_betot_dft, const T *d_bforce_ml, const T *d_bforce_dft,                       \
        const T *d_bvirial_ml, const T *d_bvirial_dft, int chebyshev_size, T scaling,            \
        const T *d_coeffs, const T *d_linear_coeffs, const T *d_type_bias, int batch_size,       \
        int natoms_pad, const int *d_binum, const int *d_bilist, const int *d_bnumneigh,         \
        const int *d_bfirstneigh, const T *d_brcs, const int *d_btypes, int ntypes, int umax,    \
        int nghost, T rmax, T rmin, const T *d_q_scaler, void *d_workspace,                      \
        size_t workspace_bytes, void *stream);
AI2B_DECL_MTP_LOSS(f64, double)
AI2B_DECL_MTP_LOSS(f32, float)

/* ------------------------------------------------------------------------------------------
 * Neighbour list
 * ---------------------------------------------------------------------------------------- */

/* Builds the padded neighbour tensors of ONE structure from positions. Replaces the CPU-only
 * chain Structure -> NeighborList -> find_info4mlff that the Python module calls
 * (source/nblist/bind/nblist_bind.cc:35-207; source/nblist/include/neighborList.h:178-189,
 * 532-578; binLinkedList.h:983-1031). Same membership rule and the same rcs bits as the
 * reference; the order inside a row is unspecified.
 *   h_cell[9]   HOST, rows = lattice vectors          h_pbc[3]  HOST, periodic flags
 *   d_coords    [natoms,3] Cartesian (is_cart != 0) or fractional
 *   outputs     d_numneigh[natoms], d_firstneigh[natoms,umax] (pad -1), d_rcs[natoms,umax,3] (pad 0)
 *   d_status    int[2]: {largest neighbour count found, 1 if a row exceeded umax}. A row that
 *               would exceed umax is truncated to umax entries (the reference overruns its
 *               buffers there, neighborList.h:550); the caller reads d_status to detect it.
 * Workspace: ai2b_nblist_workspace_bytes(natoms, is_f64). */
size_t ai2b_nblist_workspace_bytes(int natoms, int is_f64);
int ai2b_nblist_build_f64(int natoms, const double *h_cell, const double *d_coords, int is_cart,
                          double rcut, const int *h_pbc, int umax, int *d_numneigh,
                          int *d_firstneigh, double *d_rcs, int *d_status, void *d_workspace,
                          size_t workspace_bytes, void *stream);
int ai2b_nblist_build_f32(int natoms, const float *h_cell, const float *d_coords, int is_cart,
                          double rcut, const int *h_pbc, int umax, int *d_numneigh,
                          int *d_firstneigh, float *d_rcs, int *d_status, void *d_workspace,
                          size_t workspace_bytes, void *stream);

/* Neighbour build for a local domain with ghost atoms (what the LAMMPS pair style assembles on
 * the host from its full list, interface/lammps/AI2POT/pair_ai2pot.cpp:175-249): rows for the
 * first `ncentres` atoms, all `natoms` atoms as candidates; neighbour indices are positions in
 * d_coords (ghosts >= ncentres). Outputs sized [ncentres, ...]. Same workspace size as the
 * plain build for `natoms`. */
int ai2b_nblist_build_ghost_f64(int natoms, int ncentres, const double *h_cell,
                                const double *d_coords, int is_cart, double rcut,
                                const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh,
                                double *d_rcs, int *d_status, void *d_workspace,
                                size_t workspace_bytes, void *stream);
int ai2b_nblist_build_ghost_f32(int natoms, int ncentres, const float *h_cell,
                                const float *d_coords, int is_cart, double rcut,
                                const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh,
                                float *d_rcs, int *d_status, void *d_workspace,
                                size_t workspace_bytes, void *stream);

/* As ai2b_nblist_build_ghost_*, for the centre range [centre_begin, centre_end) only: row 0 of
 * the outputs belongs to atom centre_begin, outputs are sized [centre_end - centre_begin, ...], all
 * natoms atoms are candidates. A domain that is evaluated in several passes (interior centres while
 * the halo is in flight, boundary centres after it: the role LAMMPS' communication plays around
 * interface/lammps/AI2POT/pair_ai2pot.cpp:175-249) calls this once per pass. reuse_bins != 0: the
 * workspace still holds the binning of an earlier call with the same atoms, cell, cutoff and flags,
 * so only the row pass runs and d_status is accumulated into instead of being reset.
 * h_open_extent (may be NULL): fractional coordinates {lo0, lo1, lo2, hi0, hi1, hi2} that bound the
 * atoms along the non-periodic axes (entries of periodic axes are ignored). With it the bin grid is
 * sized on the host and the build needs no reduction over the positions; atoms outside the bounds
 * are still handled correctly (they share the edge bins). */
int ai2b_nblist_build_range_f64(int natoms, int centre_begin, int centre_end,
                                const double *h_cell, const double *d_coords, int is_cart,
                                double rcut, const int *h_pbc, const double *h_open_extent,
                                int umax, int reuse_bins,
                                int *d_numneigh, int *d_firstneigh, double *d_rcs,
                                int *d_status, void *d_workspace, size_t workspace_bytes,
                                void *stream);
int ai2b_nblist_build_range_f32(int natoms, int centre_begin, int centre_end,
                                const float *h_cell, const float *d_coords, int is_cart,
                                double rcut, const int *h_pbc, const double *h_open_extent,
                                int umax, int reuse_bins,
                                int *d_numneigh, int *d_firstneigh, float *d_rcs, int *d_status,
                                void *d_workspace, size_t workspace_bytes, void *stream);

/* Neighbour lists of a padded batch of small periodic structures in ONE launch: what the
 * reference's dataset does frame by frame on the host before padding every array to the largest
 * structure (ai2pot/data/mlffdataset.py:61-90, each frame through
 * source/nblist/bind/nblist_bind.cc:35-207). Same membership rule, image arithmetic and row
 * contents as ai2b_nblist_build_*; every (centre, atom, image) triple of the reference's supercell
 * is tested, so it is meant for cells of up to a few thousand atoms.
 *   d_binum[B]            atoms of each structure (<= natoms_pad)
 *   d_cells[B][9]         lattice vectors of each structure, rows = a0, a1, a2 (device)
 *   d_coords[B][Np][3]    positions (Cartesian, or fractional if !is_cart); padded slots unused
 *   h_pbc[3]              periodic flags, shared by the batch
 * Outputs, fully written (padding included): d_bilist[B][Np] (0..n-1, pad 0), d_bnumneigh[B][Np],
 * d_bfirstneigh[B][Np][umax] (pad -1), d_brcs[B][Np][umax][3] (pad 0); d_status[0] = largest
 * neighbour count, d_status[1] bit 0 = a row was truncated to umax, bit 1 = a cell more than 500
 * times thinner than the cutoff was skipped. No workspace. */
int ai2b_nblist_build_batch_f64(int batch_size, int natoms_pad, const int *d_binum,
                                const double *d_cells, const double *d_coords, int is_cart,
                                double rcut, const int *h_pbc, int umax, int *d_bilist,
                                int *d_bnumneigh, int *d_bfirstneigh, double *d_brcs,
                                int *d_status, void *stream);
int ai2b_nblist_build_batch_f32(int batch_size, int natoms_pad, const int *d_binum,
                                const float *d_cells, const float *d_coords, int is_cart,
                                double rcut, const int *h_pbc, int umax, int *d_bilist,
                                int *d_bnumneigh, int *d_bfirstneigh, float *d_brcs,
                                int *d_status, void *stream);

/* Orders every row by distance, in place (the reference's sort=true argument,
 * source/nblist/include/neighborList.h:290-335). Ties keep their build order. */
int ai2b_nblist_sort_rows_f64(int natoms, int umax, const int *d_numneigh, int *d_firstneigh,
                              double *d_rcs, void *stream);
int ai2b_nblist_sort_rows_f32(int natoms, int umax, const int *d_numneigh, int *d_firstneigh,
                              float *d_rcs, void *stream);

/* NEP energy + force + virial without a workspace argument (no counterpart in the reference).
 * For hosts that cannot give this library device memory of its own: an MD driver calling from
 * inside its timestep loop, where an allocation would stall the whole device, or a program
 * whose device memory is owned by its own pool. The scratch of ai2b_nep_efv_f32 lives in a
 * 128 KiB array inside the library image (held by every GPU that loads the library until the
 * process exits). Same arguments and results as ai2b_nep_efv_f32 otherwise.
 *  - allocates nothing; the first call on a device resolves the array's device address and
 *    should be made outside any stream capture;
 *  - returns AI2B_ERR_WORKSPACE when  256-rounded 4*(batch_size+1)  +  256-rounded
 *    4*ntypes^2*(n_radial+n_angular)*(chebyshev_size <= 8 ? 8 : 16)  exceeds 128 KiB;
 *  - every call rewrites the scratch it reads, so nothing needs clearing between calls;
 *  - all calls on a device share the array: calls that overlap on the GPU race. */
int ai2b_nep_efv_static_scratch_f32(float *d_betot, float *d_bforce, float *d_bvirial,
                                    int chebyshev_size, int n_radial, int n_angular, int l_max,
                                    int num_neurons, const float *d_coeffs, const float *d_w0,
                                    const float *d_b0, const float *d_w1, const float *d_type_bias,
                                    int batch_size, int natoms_pad, const int *d_binum,
                                    const int *d_bilist, const int *d_bnumneigh,
                                    const int *d_bfirstneigh, const float *d_brcs,
                                    const int *d_btypes, int ntypes, int umax, int nghost,
                                    float rmax_radial, float rmax_angular, const float *d_q_scaler,
                                    void *stream);

/* ------------------------------------------------------------------------------------------
 * fvt: scatter of per-pair energy gradients dE_i/dr_ij [B,Np,umax,3] into forces / virial
 * ---------------------------------------------------------------------------------------- */

/* force[B,Np+nghost,3]: F[i] += d, F[nbr] -= d (fvt::ForceSr<T>::find_val_der,
 * source/fvt/include/force_sr.h:50-81); _bwd gives dL/d(dei_drij) from dL/dforce without the
 * dense Jacobian the reference stores (find_der_backward, force_sr.h:99-123).
 * virial[B,9]: V[a,b] -= d_a r_b (fvt::VirialSr<T>::find_val_der, virial_sr.h:24-51); _bwd gives
 * dL/d(dei_drij) and, if d_grcs != NULL, dL/d(rcs). Outputs are overwritten. */
#define AI2B_DECL_FVT(SUF, T)                                                                    \
    int ai2b_fvt_force_fwd_##SUF(T *d_bforce, int batch_size, int natoms_pad, int nghost,        \
                                 int umax, const int *d_binum, const int *d_bilist,              \
                                 const int *d_bnumneigh, const int *d_bfirstneigh,               \
                                 const T *d_bdei_drij, void *stream);                            \
    int ai2b_fvt_force_bwd_##SUF(T *d_grad_dei_drij, int batch_size, int natoms_pad, int nghost, \
                                 int umax, const int *d_binum, const int *d_bilist,              \
                                 const int *d_bnumneigh, const int *d_bfirstneigh,               \
                                 const T *d_grad_force, void *stream);                           \
    int ai2b_fvt_virial_fwd_##SUF(T *d_bvirial, int batch_size, int natoms_pad, int umax,        \
                                  const int *d_bnumneigh, const T *d_brcs, const T *d_bdei_drij, \
                                  void *stream);                                                 \
    int ai2b_fvt_virial_bwd_##SUF(T *d_grad_dei_drij, T *d_grad_rcs, int batch_size,             \
                                  int natoms_pad, int umax, const int *d_bnumneigh,              \
                                  const T *d_brcs, const T *d_bdei_drij, const T *d_grad_virial, \
                                  void *stream);
AI2B_DECL_FVT(f64, double)
AI2B_DECL_FVT(f32, float)

/* NEP training path: analytic gradient of every structure's loss (same definition as
 * ai2b_mtp_loss_*, NepLoss<T>::find_loss / find_ef_loss, source/descriptor/nep/include/
 * nepLoss.h:139-215) w.r.t. coeffs [B, ntypes*ntypes*(n_radial+n_angular)*chebyshev_size],
 * w0 [B, ntypes*num_neurons*num_descriptors], b0 and w1 [B, ntypes*num_neurons], type_bias
 * [B, ntypes]. Replaces find_loss_backward_cpu_launcher / find_ef_loss_backward_cpu_launcher
 * (source/descriptor/nep/include/nepLoss_cpu_launcher.h:69-160, 213-330; CUDA
 * gpu/include/nepLoss.cuh:1163,1942). The model E/F/V of the same inputs are passed in;
 * d_bvirial_ml / d_bvirial_dft NULL gives the energy + force variant. Outputs are overwritten;
 * nghost must be 0. ai2b_nep_loss_*: loss[B] as ai2b_mtp_loss_* (same formula) and rmse[3] with
 * the NEP ops' energy RMSE, which is per atom: sqrt(mean_b ((E_b - E*_b) / n_b)^2)
 * (find_efv_rmse_cpu_launcher, nepLoss_cpu_launcher.h:355-411). */
#define AI2B_DECL_NEP_LOSS(SUF, T)                                                               \
    int ai2b_nep_loss_##SUF(T *d_bloss, T *d_rmse, int batch_size, int natoms_pad, int nghost,   \
                            const int *d_binum, const int *d_bilist, T e_weight, T f_weight,     \
                            T v_weight, const T *d_betot_ml, const T *d_betot_dft,               \
                            const T *d_bforce_ml, const T *d_bforce_dft, const T *d_bvirial_ml,  \
                            const T *d_bvirial_dft, void *d_workspace, size_t workspace_bytes,   \
                            void *stream);                                                       \
    int ai2b_nep_loss_backward_##SUF(                                                            \
        T *d_bloss_der2coeffs, T *d_bloss_der2w0, T *d_bloss_der2b0, T *d_bloss_der2w1,          \
        T *d_bloss_der2type_bias, T e_weight, T f_weight, T v_weight, const T *d_betot_ml,       \
        const T *d_betot_dft, const T *d_bforce_ml, const T *d_bforce_dft,                       \
        const T *d_bvirial_ml, const T *d_bvirial_dft, int chebyshev_size, int n_radial_basis,   \
        int n_angular_basis, int l_max, int num_neurons, const T *d_coeffs, const T *d_w0,       \
        const T *d_b0, const T *d_w1, int batch_size, int natoms_pad, const int *d_binum,        \
        const int *d_bilist, const int *d_bnumneigh, const int *d_bfirstneigh, const T *d_brcs,  \
        const int *d_btypes, int ntypes, int umax, int nghost, T rmax_radial, T rmax_angular,    \
        const T *d_q_scaler, void *stream);
AI2B_DECL_NEP_LOSS(f64, double)
AI2B_DECL_NEP_LOSS(f32, float)

/* ------------------------------------------------------------------------------------------
 * ZBL screened-Coulomb pair correction, added onto etot[B], force[B,Np+nghost,3] and (if not NULL)
 * virial[B,9] of a preceding MTP / NEP evaluation of the same batch. Replaces
 * correct_zbl_efv_torch_launcher<T> / correct_zbl_ef_torch_launcher<T>
 * (source/descriptor/correction/gpu/include/zbl_torch_launcher.h, kernels zbl.cuh:423-690) with
 * the pair functions of source/descriptor/correction/include/zbl.h:276-395. d_type_map[ntypes]
 * holds the atomic numbers, d_cks / d_dks [ntypes*ntypes*4] the screening coefficients.
 * The reference's CPU ops differ from its CUDA ops here: GroupZBL::correct_efv adds the energy
 * only (zbl.h:545-548) and the CPU MTP launcher then zeroes even that; these entry points follow
 * the CUDA path (energy, force, virial).
 * ---------------------------------------------------------------------------------------- */
#define AI2B_DECL_ZBL(SUF, T)                                                                    \
    int ai2b_zbl_efv_##SUF(T *d_betot, T *d_bforce, T *d_bvirial, int batch_size,                \
                           int natoms_pad, const int *d_binum, const int *d_bilist,              \
                           const int *d_bnumneigh, const int *d_bfirstneigh, const T *d_brcs,    \
                           const int *d_btypes, int ntypes, const int *d_type_map, int umax,     \
                           int nghost, T zbl_rmax, T zbl_rmin, const T *d_cks, const T *d_dks,   \
                           void *stream);
AI2B_DECL_ZBL(f64, double)
AI2B_DECL_ZBL(f32, float)

/* ------------------------------------------------------------------------------------------
 * Dataset statistics for the descriptor scaler and the target normaliser (the pre-training pass).
 * desc_stats_all / _each: AllTypeDescriptorsStatistics / EachTypeDescriptorsStatistics
 * <T>::find_descriptors_statistics (source/descriptor/fitutils/include/descriptorsStatistics.h:
 * 76-167; CUDA launchers gpu/include/descriptorsStatistics_torch_launcher.h): atom count(s),
 * mean[ (ntypes,) nd ] and M2 = sum (x - mean)^2 of bdescriptors[B,Np,nd] over the listed atoms
 * (per centre type btypes[b*Np + bilist[b*Np + i]] for _each). desc_maxmin:
 * AllTypeDescriptorsMaxmin<T>::find_descriptors_maxmin (:177-205; max starts at FLT_MIN, min at
 * FLT_MAX as there). target_stats: TargetStatistics<T>::find_ef_statistics
 * (targetStatistics.h:44-80): d_out3 = {mean, M2 of E_b / n_b over structures, sum of squared
 * force components}. Sums are accumulated in double (the reference sums sequentially in T).
 * ---------------------------------------------------------------------------------------- */
#define AI2B_DECL_STATS(SUF, T)                                                                  \
    int ai2b_desc_stats_all_##SUF(int *d_natoms, T *d_mean, T *d_m2, int batch_size,             \
                                  int natoms_pad, int descriptor_dim, const int *d_binum,        \
                                  const T *d_bdescriptors, void *stream);                        \
    int ai2b_desc_stats_each_##SUF(int *d_natoms, T *d_mean, T *d_m2, int batch_size,            \
                                   int natoms_pad, int descriptor_dim, const int *d_binum,       \
                                   const int *d_bilist, const int *d_btypes, int ntypes,         \
                                   const T *d_bdescriptors, void *stream);                       \
    int ai2b_desc_maxmin_##SUF(T *d_max, T *d_min, int batch_size, int natoms_pad,               \
                               int descriptor_dim, const int *d_binum, const T *d_bdescriptors,  \
                               void *stream);                                                    \
    int ai2b_target_stats_##SUF(int *d_natoms, T *d_out3, int batch_size, int natoms_pad,        \
                                const int *d_binum, const T *d_betot_dft, const T *d_bforce_dft, \
                                void *stream);
AI2B_DECL_STATS(f64, double)
AI2B_DECL_STATS(f32, float)

/* ------------------------------------------------------------------------------------------
 * Reduction of per-structure gradients: d_out[off_k + i] = sum_b d_w[b] * parts[k][b * n[k] + i],
 * off_k = n[0] + ... + n[k-1], for up to 8 row-major [batch_size][n[k]] device arrays in ONE
 * launch (d_w NULL: plain sums). This is the `grad_out[B] @ per-structure gradient` product that
 * the backward of every training op forms once per parameter tensor (source/descriptor/nep/src/
 * nepOp.cc:2335-2339, 3464-3468; source/descriptor/mtpr/src/linearMtpOp.cc, the *LossOp
 * backward functions). h_parts / h_n are HOST arrays of nparts device pointers / row lengths.
 * ---------------------------------------------------------------------------------------- */
#define AI2B_DECL_WSUM(SUF, T)                                                                   \
    int ai2b_weighted_sum_rows_##SUF(int nparts, const T *const *h_parts, const int *h_n,        \
                                     int batch_size, const T *d_w, T *d_out, void *stream);
AI2B_DECL_WSUM(f64, double)
AI2B_DECL_WSUM(f32, float)

/* ------------------------------------------------------------------------------------------
 * Device-resident input path for a molecular-dynamics host: replaces
 * PairAI2Pot::construct_mlff_input + the tensor traffic of PairAI2Pot::compute
 * (interface/lammps/AI2POT/pair_ai2pot.cpp:175-249, 383-471). Unlike the entry points above a
 * session owns its device and pinned buffers (they grow with the atom counts and are reused, so
 * a steady-state step allocates nothing) and its own stream, takes HOST arrays in the host
 * program's layout, and returns when the results are on the host.
 *   h_x[nlocal+nghost][3]      positions as the host keeps them (double; ghosts carry the
 *                              periodic images, no cell is needed)
 *   h_model_type[nlocal+nghost] model type index of every atom (lmp2model_type_map applied)
 *   h_f[nlocal+nghost][3]      += forces, ghosts included (the host reverse-communicates them)
 *   h_eng                      += energy (may be NULL);  h_virial6 += xx,yy,zz,xy,xz,yz if
 *                              want_virial (pair_ai2pot.cpp:461-468)
 *   h_max_neighbours           largest neighbour count found (may be NULL); more than umax
 *                              returns AI2B_ERR_OVERFLOW (the reference overruns its rows)
 * The neighbour rows are built on the device every step from the positions (r_j - r_i in
 * double, stored as float, as the host loop does), with the model cutoff; pairs the host's list
 * holds beyond the cutoff (skin) contribute nothing in either case. Models are single precision,
 * as in pair_ai2pot.cpp. The MTP variant borrows the program handle (keep it alive).
 * ---------------------------------------------------------------------------------------- */
typedef struct ai2b_md_session ai2b_md_session;
int ai2b_md_session_create_nep(ai2b_md_session **out, int chebyshev_size, int n_radial,
                               int n_angular, int l_max, int num_neurons, int ntypes,
                               const float *h_coeffs, const float *h_w0, const float *h_b0,
                               const float *h_w1, const float *h_type_bias,
                               const float *h_q_scaler, float rmax_radial, float rmax_angular,
                               int umax);
int ai2b_md_session_create_mtp(ai2b_md_session **out, const ai2b_mtp_program *prog,
                               int chebyshev_size, float scaling, int ntypes, int nmus,
                               int alpha_scalar_moments, const float *h_coeffs,
                               const float *h_linear_coeffs, const float *h_type_bias,
                               const float *h_q_scaler, float rmax, float rmin, int umax);
void ai2b_md_session_destroy(ai2b_md_session *session);
int ai2b_md_session_compute(ai2b_md_session *session, int nlocal, int nghost, const double *h_x,
                            const int *h_model_type, int want_virial, double *h_f,
                            double *h_eng, double *h_virial6, int *h_max_neighbours);

/* Neighbour rows in single precision from double-precision positions (r_j - r_i formed in
 * double, rounded once: pair_ai2pot.cpp:232-235); otherwise as ai2b_nblist_build_ghost_f64. */
int ai2b_nblist_build_ghost_f64_rows32(int natoms, int ncentres, const double *h_cell,
                                       const double *d_coords, int is_cart, double rcut,
                                       const int *h_pbc, int umax, int *d_numneigh,
                                       int *d_firstneigh, float *d_rcs, int *d_status,
                                       void *d_workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * NEP (3-body terms, l_max <= 4, chebyshev_size <= 16)
 * ---------------------------------------------------------------------------------------- */

size_t ai2b_nep_workspace_bytes(int batch_size, int ntypes, int n_radial, int n_angular,
                                int chebyshev_size, int is_f64);

/* Energy + force + virial. Replaces nep::find_efv_torch_launcher<T>
 * (source/descriptor/nep/gpu/include/nep_torch_launcher.cuh:34-103) and the CPU launcher
 * (source/descriptor/nep/include/nep_cpu_launcher.h:186-257). Parameter layouts as in the
 * reference: coeffs[ntypes,ntypes,n_radial+n_angular,chebyshev_size], w0[ntypes,neurons,nd],
 * b0[ntypes,neurons], w1[ntypes,neurons], nd = n_radial + n_angular*l_max. Outputs are
 * overwritten. d_bvirial may be NULL: energy + force only (find_ef, nep_cpu_launcher.h:116-184). */
#define AI2B_DECL_NEP(SUF, T)                                                                    \
    int ai2b_nep_efv_##SUF(T *d_betot, T *d_bforce, T *d_bvirial, int chebyshev_size,            \
                           int n_radial, int n_angular, int l_max, int num_neurons,              \
                           const T *d_coeffs, const T *d_w0, const T *d_b0, const T *d_w1,       \
                           const T *d_type_bias, int batch_size, int natoms_pad,                 \
                           const int *d_binum, const int *d_bilist, const int *d_bnumneigh,      \
                           const int *d_bfirstneigh, const T *d_brcs, const int *d_btypes,       \
                           int ntypes, int umax, int nghost, T rmax_radial, T rmax_angular,      \
                           const T *d_q_scaler, void *d_workspace, size_t workspace_bytes,       \
                           void *stream);                                                        \
    /* same, ADDING onto d_betot, d_bforce, d_bvirial instead of overwriting them: what the     \
     * reference's own launchers do (they never zero their outputs, nep.h:320-529). Lets a      \
     * caller evaluate one system in several passes over disjoint sets of centres. */           \
    int ai2b_nep_efv_accumulate_##SUF(T *d_betot, T *d_bforce, T *d_bvirial, int chebyshev_size, \
                           int n_radial, int n_angular, int l_max, int num_neurons,              \
                           const T *d_coeffs, const T *d_w0, const T *d_b0, const T *d_w1,       \
                           const T *d_type_bias, int batch_size, int natoms_pad,                 \
                           const int *d_binum, const int *d_bilist, const int *d_bnumneigh,      \
                           const int *d_bfirstneigh, const T *d_brcs, const int *d_btypes,       \
                           int ntypes, int umax, int nghost, T rmax_radial, T rmax_angular,      \
                           const T *d_q_scaler, void *d_workspace, size_t workspace_bytes,       \
                           void *stream);                                                        \
    /* descriptors [B,Np,nd]: find_descriptors launcher, nep_cpu_launcher.h:259-317 */           \
    int ai2b_nep_descriptors_##SUF(T *d_bdescriptors, int chebyshev_size, int n_radial,          \
                                   int n_angular, int l_max, const T *d_coeffs, int batch_size,  \
                                   int natoms_pad, const int *d_binum, const int *d_bilist,      \
                                   const int *d_bnumneigh, const int *d_bfirstneigh,             \
                                   const T *d_brcs, const int *d_btypes, int ntypes, int umax,   \
                                   int nghost, T rmax_radial, T rmax_angular, void *d_workspace, \
                                   size_t workspace_bytes, void *stream);
AI2B_DECL_NEP(f64, double)
AI2B_DECL_NEP(f32, float)

/* ------------------------------------------------------------------------------------------
 * Halo exchange between neighbouring spatial domains by direct stores into the neighbour GPU's
 * memory (NVLink peer access). It does the job MPI does for the reference when LAMMPS runs the
 * pair style on several ranks: ghost positions before the evaluation, ghost forces back after it
 * (interface/lammps/AI2POT/pair_ai2pot.cpp:177-205, 452-455).
 *   ai2b_peer_push_rows_*  d_peer_dst[d_dst_index[k]][0..2] = d_src[d_src_index[k]][0..2] + h_shift3
 *                          for k < nrows (either index may be NULL = k; h_shift3 NULL = no shift),
 *                          then *d_peer_flag = flag_value with a system-scope release once every
 *                          row is written. d_peer_dst and d_peer_flag are addresses in the
 *                          NEIGHBOUR's memory as mapped into this process (peer access must be
 *                          enabled by whoever mapped them); d_counter is one zero-initialised
 *                          word of THIS device, private to the pushes of one stream.
 *   ai2b_peer_wait         holds the stream until *d_flag >= value (system-scope acquire polls).
 *                          Bounded: after max_polls polls (200 ns apart) it stores 1 to *d_status
 *                          and lets the stream go on, so nothing hangs; the host reads d_status
 *                          when it next synchronises and treats 1 as AI2B_ERR_TIMEOUT.
 *   ai2b_peer_exchange_*   both directions of an exchange in one launch: the two pushes (arguments
 *                          *_l to the lower neighbour, *_r to the upper one), both neighbours'
 *                          flags raised, then the bounded wait for this rank's two flags
 *                          (d_my_flag_l: raised by the lower neighbour, d_my_flag_r: by the upper).
 *   ai2b_peer_return_reduce_*  the closing exchange of a step in one launch: contiguous
 *                          ghost-force rows to the two neighbours' d_back arrays; this rank's
 *                          partial sums d_partial[nvalues] (energy, virial) written into row `rank`
 *                          of every rank's table ([nranks][16] values, d_peer_tables[q] = rank q's
 *                          table as mapped here, own entry = own table) with a flag per source
 *                          rank; after the bounded waits, d_force[d_back_index[k]] += d_back[k]
 *                          for the rows the neighbours pushed here, and d_reduced[nvalues] = sum
 *                          over the ranks' partials in rank order (identical on every rank).
 *                          nranks = 0 skips the reduction, nback = nrows = 0 the force part.
 * Use increasing flag values (a step counter): a flag is never reset.
 * ---------------------------------------------------------------------------------------- */
int ai2b_peer_push_rows_f32(const float *d_src, const int *d_src_index, const int *d_dst_index,
                            int nrows, const float *h_shift3, float *d_peer_dst,
                            int *d_peer_flag, int flag_value, unsigned *d_counter, void *stream);
int ai2b_peer_push_rows_f64(const double *d_src, const int *d_src_index, const int *d_dst_index,
                            int nrows, const double *h_shift3, double *d_peer_dst,
                            int *d_peer_flag, int flag_value, unsigned *d_counter, void *stream);
int ai2b_peer_wait(const int *d_flag, int value, long long max_polls, int *d_status,
                   void *stream);
#define AI2B_DECL_PEER_EXCHANGE(SUF, T)                                                          \
    int ai2b_peer_exchange_##SUF(const T *d_src_l, const int *d_src_index_l,                     \
                                 const int *d_dst_index_l, int nrows_l, const T *h_shift3_l,     \
                                 T *d_peer_dst_l, int *d_peer_flag_l, const T *d_src_r,          \
                                 const int *d_src_index_r, const int *d_dst_index_r,             \
                                 int nrows_r, const T *h_shift3_r, T *d_peer_dst_r,              \
                                 int *d_peer_flag_r, int flag_value, const int *d_my_flag_l,     \
                                 const int *d_my_flag_r, long long max_polls, int *d_status,     \
                                 unsigned *d_counter, void *stream);
AI2B_DECL_PEER_EXCHANGE(f64, double)
AI2B_DECL_PEER_EXCHANGE(f32, float)
#define AI2B_DECL_PEER_RETURN(SUF, T)                                                            \
    int ai2b_peer_return_reduce_##SUF(const T *d_src_l, int nrows_l, T *d_peer_dst_l,            \
                                      int *d_peer_flag_l, const T *d_src_r, int nrows_r,         \
                                      T *d_peer_dst_r, int *d_peer_flag_r, int flag_value,       \
                                      const int *d_my_flag_l, const int *d_my_flag_r,            \
                                      const T *d_back, const int *d_back_index, int nback,       \
                                      T *d_force, const T *d_partial, T *const *d_peer_tables,   \
                                      int *const *d_peer_table_flags, const T *d_my_table,       \
                                      const int *d_my_table_flags, T *d_reduced, int rank,       \
                                      int nranks, int nvalues, long long max_polls,              \
                                      int *d_status, unsigned *d_counter, void *stream);
AI2B_DECL_PEER_RETURN(f64, double)
AI2B_DECL_PEER_RETURN(f32, float)

#ifdef __cplusplus
}
#endif
#endif /* AI2POT_B200_H */
