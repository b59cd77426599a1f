// Device-resident input path for a molecular-dynamics host (the role of
// PairAI2Pot::construct_mlff_input + compute, interface/lammps/AI2POT/pair_ai2pot.cpp:175-249,383-471).
//
// The reference builds the seven input tensors on the host every step (a loop over the host's
// neighbour list forming r_j - r_i in double and storing float), uploads all of them, runs the
// model and downloads forces. Here a step uploads only the positions (double, as the host keeps
// them) and the model types of the nlocal + nghost atoms; the neighbour rows are built on the
// device (centres = local atoms, candidates = local + ghost atoms, no periodic images: the host's
// ghosts carry the periodicity), the model runs on them, and forces for all nlocal + nghost atoms
// come back for the host's reverse communication, with the energy and the six virial components
// in the host's order. Device and pinned buffers grow when the atom counts grow and are reused
// otherwise, so a steady-state step allocates nothing.
#include "common.cuh"

#include <vector>

using namespace ai2b;

struct ai2b_md_session {
    int kind = 0;   // 0 = NEP, 1 = linear MTP
    int ntypes = 0, umax = 0;
    double rcut = 0;
    // NEP
    int cs = 0, n_r = 0, n_a = 0, l_max = 0, nneu = 0;
    float rc_r = 0, rc_a = 0;
    float *d_coeffs = nullptr, *d_w0 = nullptr, *d_b0 = nullptr, *d_w1 = nullptr, *d_bias = nullptr, *d_qs = nullptr;
    // MTP
    const ai2b_mtp_program *prog = nullptr;
    float scaling = 0, rmax = 0, rmin = 0;
    float *d_lin = nullptr;
    // per-step buffers
    int cap_all = 0, cap_local = 0;
    double *d_x = nullptr;
    int *d_types = nullptr, *d_numneigh = nullptr, *d_firstneigh = nullptr, *d_ilist = nullptr, *d_binum = nullptr, *d_status = nullptr;
    float *d_rcs = nullptr, *d_force = nullptr, *d_ev = nullptr;
    void *d_nbws = nullptr, *d_ws = nullptr;
    size_t nbws = 0, ws = 0;
    float *h_force = nullptr, *h_ev = nullptr;
    int *h_small = nullptr;   // pinned: [0] = nlocal, [1..2] = status
    cudaStream_t stream = nullptr;
};

namespace {

__global__ void iota_kernel(int *out, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = i;
}

template <typename T>
int upload(T **dst, const T *src, size_t n)
{
    AI2B_CUDA(cudaMalloc((void **)dst, sizeof(T) * (n ? n : 1)));
    if (n) AI2B_CUDA(cudaMemcpy(*dst, src, sizeof(T) * n, cudaMemcpyHostToDevice));
    return AI2B_OK;
}

void release_step_buffers(ai2b_md_session *s)
{
    cudaFree(s->d_x); cudaFree(s->d_types); cudaFree(s->d_numneigh); cudaFree(s->d_firstneigh); cudaFree(s->d_ilist);
    cudaFree(s->d_rcs); cudaFree(s->d_force); cudaFree(s->d_nbws); cudaFree(s->d_ws);
    cudaFreeHost(s->h_force);
    s->d_x = nullptr; s->d_types = s->d_numneigh = s->d_firstneigh = s->d_ilist = nullptr;
    s->d_rcs = s->d_force = nullptr; s->d_nbws = s->d_ws = nullptr; s->h_force = nullptr;
    // nothing is usable until ensure_capacity has run to its end: a growth that failed half-way (out of
    // memory) must make the next call allocate afresh instead of running on freed or partial buffers
    s->cap_all = s->cap_local = 0;
}

int ensure_capacity(ai2b_md_session *s, int nlocal, int nall)
{
    if (nall <= s->cap_all && nlocal <= s->cap_local) return AI2B_OK;
    AI2B_CUDA(cudaStreamSynchronize(s->stream));
    release_step_buffers(s);
    const int call = nall + nall / 5 + 64, cloc = nlocal + nlocal / 5 + 64;   // 20 % head-room against regrowth every step
    AI2B_CUDA(cudaMalloc((void **)&s->d_x, sizeof(double) * 3 * call));
    AI2B_CUDA(cudaMalloc((void **)&s->d_types, sizeof(int) * call));
    AI2B_CUDA(cudaMalloc((void **)&s->d_numneigh, sizeof(int) * cloc));
    AI2B_CUDA(cudaMalloc((void **)&s->d_firstneigh, sizeof(int) * (size_t)cloc * s->umax));
    AI2B_CUDA(cudaMalloc((void **)&s->d_rcs, sizeof(float) * 3 * (size_t)cloc * s->umax));
    AI2B_CUDA(cudaMalloc((void **)&s->d_ilist, sizeof(int) * cloc));
    AI2B_CUDA(cudaMalloc((void **)&s->d_force, sizeof(float) * 3 * call));
    AI2B_CUDA(cudaMallocHost((void **)&s->h_force, sizeof(float) * 3 * call));
    s->nbws = ai2b_nblist_workspace_bytes(call, 1);
    AI2B_CUDA(cudaMalloc(&s->d_nbws, s->nbws));
    s->ws = s->kind == 0 ? ai2b_nep_workspace_bytes(1, s->ntypes, s->n_r, s->n_a, s->cs, 0)
                         : ai2b_mtp_workspace_bytes(s->prog, 1, cloc, s->ntypes);
    AI2B_CUDA(cudaMalloc(&s->d_ws, s->ws ? s->ws : 256));
    iota_kernel<<<(cloc + 255) / 256, 256, 0, s->stream>>>(s->d_ilist, cloc);
    AI2B_CUDA(cudaGetLastError());
    s->cap_all = call;
    s->cap_local = cloc;
    return AI2B_OK;
}

int common_init(ai2b_md_session *s)
{
    AI2B_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    AI2B_CUDA(cudaMalloc((void **)&s->d_ev, sizeof(float) * 16));
    AI2B_CUDA(cudaMalloc((void **)&s->d_binum, sizeof(int) * 4));
    AI2B_CUDA(cudaMalloc((void **)&s->d_status, sizeof(int) * 4));
    AI2B_CUDA(cudaMallocHost((void **)&s->h_ev, sizeof(float) * 16));
    AI2B_CUDA(cudaMallocHost((void **)&s->h_small, sizeof(int) * 8));
    return AI2B_OK;
}

}  // namespace

extern "C" int ai2b_md_session_create_nep(ai2b_md_session **out, int chebyshev_size, int n_radial, int n_angular, int l_max,
                                          int num_neurons, int ntypes, const float *h_coeffs, const float *h_w0, const float *h_b0,
                                          const float *h_w1, const float *h_type_bias, const float *h_q_scaler, float rmax_radial,
                                          float rmax_angular, int umax)
{
    AI2B_REQUIRE(out && h_coeffs && h_w0 && h_b0 && h_w1 && h_type_bias && h_q_scaler, AI2B_ERR_INVALID, "ai2b_md_session_create_nep: NULL argument");
    AI2B_REQUIRE(ntypes >= 1 && umax >= 1 && num_neurons >= 1 && rmax_radial > 0, AI2B_ERR_INVALID, "ai2b_md_session_create_nep: bad size");
    ai2b_md_session *s = new ai2b_md_session();
    s->kind = 0; s->ntypes = ntypes; s->umax = umax; s->rcut = rmax_radial > rmax_angular ? rmax_radial : rmax_angular;
    s->cs = chebyshev_size; s->n_r = n_radial; s->n_a = n_angular; s->l_max = l_max; s->nneu = num_neurons;
    s->rc_r = rmax_radial; s->rc_a = rmax_angular;
    const int nd = l_max == 0 ? n_radial : n_radial + n_angular * l_max;
    int rc = common_init(s);
    if (!rc) rc = upload(&s->d_coeffs, h_coeffs, (size_t)ntypes * ntypes * (n_radial + n_angular) * chebyshev_size);
    if (!rc) rc = upload(&s->d_w0, h_w0, (size_t)ntypes * num_neurons * nd);
    if (!rc) rc = upload(&s->d_b0, h_b0, (size_t)ntypes * num_neurons);
    if (!rc) rc = upload(&s->d_w1, h_w1, (size_t)ntypes * num_neurons);
    if (!rc) rc = upload(&s->d_bias, h_type_bias, (size_t)ntypes);
    if (!rc) rc = upload(&s->d_qs, h_q_scaler, (size_t)nd);
    if (rc) { ai2b_md_session_destroy(s); return rc; }
    *out = s;
    return AI2B_OK;
}

extern "C" int ai2b_md_session_create_mtp(ai2b_md_session **out, const ai2b_mtp_program *prog, int chebyshev_size, float scaling,
                                          int ntypes, int nmus, int alpha_scalar_moments, const float *h_coeffs,
                                          const float *h_linear_coeffs, const float *h_type_bias, const float *h_q_scaler, float rmax,
                                          float rmin, int umax)
{
    AI2B_REQUIRE(out && prog && h_coeffs && h_linear_coeffs && h_type_bias && h_q_scaler, AI2B_ERR_INVALID, "ai2b_md_session_create_mtp: NULL argument");
    AI2B_REQUIRE(ntypes >= 1 && umax >= 1 && nmus >= 1 && alpha_scalar_moments >= 1 && rmax > rmin, AI2B_ERR_INVALID,
                 "ai2b_md_session_create_mtp: bad size");
    ai2b_md_session *s = new ai2b_md_session();
    s->kind = 1; s->ntypes = ntypes; s->umax = umax; s->rcut = rmax; s->prog = prog; s->cs = chebyshev_size; s->scaling = scaling;
    s->rmax = rmax; s->rmin = rmin;
    int rc = common_init(s);
    if (!rc) rc = upload(&s->d_coeffs, h_coeffs, (size_t)ntypes * ntypes * nmus * chebyshev_size);
    if (!rc) rc = upload(&s->d_lin, h_linear_coeffs, (size_t)alpha_scalar_moments);
    if (!rc) rc = upload(&s->d_bias, h_type_bias, (size_t)ntypes);
    if (!rc) rc = upload(&s->d_qs, h_q_scaler, (size_t)alpha_scalar_moments);
    if (rc) { ai2b_md_session_destroy(s); return rc; }
    *out = s;
    return AI2B_OK;
}

extern "C" void ai2b_md_session_destroy(ai2b_md_session *s)
{
    if (!s) return;
    if (s->stream) cudaStreamSynchronize(s->stream);
    release_step_buffers(s);
    cudaFree(s->d_coeffs); cudaFree(s->d_w0); cudaFree(s->d_b0); cudaFree(s->d_w1); cudaFree(s->d_bias); cudaFree(s->d_qs);
    cudaFree(s->d_lin); cudaFree(s->d_ev); cudaFree(s->d_binum); cudaFree(s->d_status);
    cudaFreeHost(s->h_ev); cudaFreeHost(s->h_small);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

extern "C" int ai2b_md_session_compute(ai2b_md_session *s, int nlocal, int nghost, const double *h_x, const int *h_model_type,
                                       int want_virial, double *h_f, double *h_eng, double *h_virial6, int *h_max_neighbours)
{
    AI2B_REQUIRE(s && h_x && h_model_type && h_f, AI2B_ERR_INVALID, "ai2b_md_session_compute: NULL argument");
    AI2B_REQUIRE(nlocal >= 0 && nghost >= 0, AI2B_ERR_INVALID, "ai2b_md_session_compute: negative atom count");
    if (nlocal == 0) return AI2B_OK;
    const int nall = nlocal + nghost;
    if (int rc = ensure_capacity(s, nlocal, nall)) return rc;
    cudaStream_t st = s->stream;
    s->h_small[0] = nlocal;
    AI2B_CUDA(cudaMemcpyAsync(s->d_x, h_x, sizeof(double) * 3 * nall, cudaMemcpyHostToDevice, st));
    AI2B_CUDA(cudaMemcpyAsync(s->d_types, h_model_type, sizeof(int) * nall, cudaMemcpyHostToDevice, st));
    AI2B_CUDA(cudaMemcpyAsync(s->d_binum, s->h_small, sizeof(int), cudaMemcpyHostToDevice, st));
    const double cell[9] = {1, 0, 0, 0, 1, 0, 0, 0, 1};   // no periodic axis: only the extents of the atoms matter
    const int pbc[3] = {0, 0, 0};
    int rc = ai2b_nblist_build_ghost_f64_rows32(nall, nlocal, cell, s->d_x, 1, s->rcut, pbc, s->umax, s->d_numneigh, s->d_firstneigh,
                                                s->d_rcs, s->d_status, s->d_nbws, s->nbws, st);
    if (rc) return rc;
    float *d_vir = want_virial ? s->d_ev + 1 : nullptr;
    if (s->kind == 0)
        rc = ai2b_nep_efv_f32(s->d_ev, s->d_force, d_vir, s->cs, s->n_r, s->n_a, s->l_max, s->nneu, s->d_coeffs, s->d_w0, s->d_b0, s->d_w1,
                              s->d_bias, 1, nlocal, s->d_binum, s->d_ilist, s->d_numneigh, s->d_firstneigh, s->d_rcs, s->d_types, s->ntypes,
                              s->umax, nghost, s->rc_r, s->rc_a, s->d_qs, s->d_ws, s->ws, st);
    else
        rc = ai2b_mtp_efv_f32(s->prog, s->d_ev, s->d_force, d_vir, s->cs, s->scaling, s->d_coeffs, s->d_lin, s->d_bias, 1, nlocal,
                              s->d_binum, s->d_ilist, s->d_numneigh, s->d_firstneigh, s->d_rcs, s->d_types, s->ntypes, s->umax, nghost,
                              s->rmax, s->rmin, s->d_qs, s->d_ws, s->ws, st);
    if (rc) return rc;
    AI2B_CUDA(cudaMemcpyAsync(s->h_force, s->d_force, sizeof(float) * 3 * nall, cudaMemcpyDeviceToHost, st));
    AI2B_CUDA(cudaMemcpyAsync(s->h_ev, s->d_ev, sizeof(float) * 10, cudaMemcpyDeviceToHost, st));
    AI2B_CUDA(cudaMemcpyAsync(s->h_small + 1, s->d_status, sizeof(int) * 2, cudaMemcpyDeviceToHost, st));
    AI2B_CUDA(cudaStreamSynchronize(st));
    if (h_max_neighbours) *h_max_neighbours = s->h_small[1];
    AI2B_REQUIRE(!s->h_small[2], AI2B_ERR_OVERFLOW, "an atom has %d neighbours within the cutoff, umax is %d", s->h_small[1], s->umax);
    // pair_ai2pot.cpp:447-468: forces of all nlocal + nghost atoms are added, energy and virial accumulate
    for (size_t i = 0; i < (size_t)3 * nall; i++) h_f[i] += (double)s->h_force[i];
    if (h_eng) *h_eng += (double)s->h_ev[0];
    if (want_virial && h_virial6) {
        static const int pick[6] = {0, 4, 8, 1, 2, 5};
        for (int k = 0; k < 6; k++) h_virial6[k] += (double)s->h_ev[1 + pick[k]];
    }
    return AI2B_OK;
}
