// fvt: scatter of per-pair energy gradients dE_i/dr_ij into forces and the virial, and the
// matrix-free adjoints of both.
//
// Reference: source/fvt/include/force_sr.h:50-81 (F[i] += d, F[j] -= d), :99-123 (backward
// through a stored dense Jacobian of size [(N+nghost),3,N,umax] whose entries are +1 / -1),
// virial_sr.h:24-51 (V[a,b] -= d_a * r_b; Jacobians -r_b and -d_a). The dense Jacobians are
// never formed here: the backward kernels apply them directly
//   dL/dd[i,j,a]   = gF[i,a] - gF[nbr(i,j),a]              (force)
//   dL/dd[i,j,a]   = -sum_b gV[a,b] r[i,j,b]               (virial, w.r.t. dei_drij)
//   dL/dr[i,j,b]   = -sum_a gV[a,b] d[i,j,a]               (virial, w.r.t. rcs)
#include "common.cuh"

namespace ai2b {

template <typename T>
__global__ void fvt_force_fwd_kernel(T *__restrict__ force, int B, int npad, int nghost, int umax, const int *__restrict__ binum,
                                     const int *__restrict__ bilist, const int *__restrict__ numneigh,
                                     const int *__restrict__ firstneigh, const T *__restrict__ de)
{
    // one warp per centre slot, lanes over neighbours
    const int lane = threadIdx.x & 31;
    const long slot = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (slot >= (long)B * npad) return;
    const int b = (int)(slot / npad), ii = (int)(slot % npad);
    if (ii >= binum[b]) return;
    T *frc = force + (size_t)b * (npad + nghost) * 3;
    const int ci = bilist[slot], nn = min(numneigh[slot], umax);
    T s[3] = {0, 0, 0};
    for (int j = lane; j < nn; j += 32) {
        const int nj = firstneigh[slot * umax + j];
#pragma unroll
        for (int a = 0; a < 3; a++) {
            const T g = de[(slot * umax + j) * 3 + a];
            s[a] += g;
            atomicAdd(frc + 3 * nj + a, -g);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; a++) {
        s[a] = warp_sum(s[a]);
        if (lane == 0) atomicAdd(frc + 3 * ci + a, s[a]);
    }
}

template <typename T>
__global__ void fvt_force_bwd_kernel(T *__restrict__ gde, int B, int npad, int nghost, int umax, const int *__restrict__ binum,
                                     const int *__restrict__ bilist, const int *__restrict__ numneigh,
                                     const int *__restrict__ firstneigh, const T *__restrict__ gforce)
{
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;   // over [B, npad, umax]
    if (idx >= (long)B * npad * umax) return;
    const long slot = idx / umax;
    const int j = (int)(idx % umax), b = (int)(slot / npad), ii = (int)(slot % npad);
    T out[3] = {0, 0, 0};
    if (ii < binum[b] && j < numneigh[slot]) {
        const T *gf = gforce + (size_t)b * (npad + nghost) * 3;
        const int ci = bilist[slot], nj = firstneigh[idx];
#pragma unroll
        for (int a = 0; a < 3; a++) out[a] = gf[3 * ci + a] - gf[3 * nj + a];
    }
#pragma unroll
    for (int a = 0; a < 3; a++) gde[idx * 3 + a] = out[a];
}

template <typename T>
__global__ void fvt_virial_fwd_kernel(T *__restrict__ virial, int B, int npad, int umax, const int *__restrict__ numneigh,
                                      const T *__restrict__ rcs, const T *__restrict__ de)
{
    // grid.y = structure; block reduces its share of pairs, then 9 atomics.
    // The reference sums over every row of the padded batch (numneigh = 0 for padded atoms).
    __shared__ T sh[9][8];
    const int b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T v[9];
#pragma unroll
    for (int k = 0; k < 9; k++) v[k] = T(0);
    for (long p = (long)blockIdx.x * blockDim.x + threadIdx.x; p < (long)npad * umax; p += (long)gridDim.x * blockDim.x) {
        const long slot = (long)b * npad + p / umax;
        const int j = (int)(p % umax);
        if (j < numneigh[slot]) {
            const T *d = de + (slot * umax + j) * 3, *r = rcs + (slot * umax + j) * 3;
#pragma unroll
            for (int a = 0; a < 3; a++)
#pragma unroll
                for (int c = 0; c < 3; c++) v[3 * a + c] -= d[a] * r[c];
        }
    }
#pragma unroll
    for (int k = 0; k < 9; k++) {
        v[k] = warp_sum(v[k]);
        if (lane == 0) sh[k][warp] = v[k];
    }
    __syncthreads();
    if (threadIdx.x < 9) {
        T s = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) s += sh[threadIdx.x][w];
        atomicAdd(virial + 9 * b + threadIdx.x, s);
    }
}

template <typename T>
__global__ void fvt_virial_bwd_kernel(T *__restrict__ gde, T *__restrict__ grcs, int B, int npad, int umax,
                                      const int *__restrict__ numneigh, const T *__restrict__ rcs, const T *__restrict__ de,
                                      const T *__restrict__ gvirial)
{
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)B * npad * umax) return;
    const long slot = idx / umax;
    const int j = (int)(idx % umax), b = (int)(slot / npad);
    T od[3] = {0, 0, 0}, orr[3] = {0, 0, 0};
    if (j < numneigh[slot]) {
        const T *gv = gvirial + 9 * b;
#pragma unroll
        for (int a = 0; a < 3; a++)
#pragma unroll
            for (int c = 0; c < 3; c++) {
                od[a] -= gv[3 * a + c] * rcs[idx * 3 + c];
                orr[c] -= gv[3 * a + c] * de[idx * 3 + a];
            }
    }
#pragma unroll
    for (int a = 0; a < 3; a++) {
        gde[idx * 3 + a] = od[a];
        if (grcs) grcs[idx * 3 + a] = orr[a];
    }
}

}  // namespace ai2b

using namespace ai2b;

#define AI2B_DEF_FVT(SUF, T)                                                                                       \
    extern "C" int ai2b_fvt_force_fwd_##SUF(T *force, int B, int npad, int nghost, int umax, const int *binum,     \
                                            const int *bilist, const int *numneigh, const int *firstneigh,         \
                                            const T *de, void *stream)                                             \
    {                                                                                                              \
        AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0 && nghost >= 0, AI2B_ERR_INVALID, "fvt: negative size");      \
        if (B == 0 || npad + nghost == 0) return AI2B_OK;                                                          \
        AI2B_REQUIRE(force && binum && bilist && numneigh && firstneigh && de, AI2B_ERR_INVALID, "fvt: NULL");      \
        cudaStream_t st = (cudaStream_t)stream;                                                                    \
        AI2B_CUDA(cudaMemsetAsync(force, 0, sizeof(T) * 3 * (size_t)B * (npad + nghost), st));                     \
        if (npad == 0 || umax == 0) return AI2B_OK;                                                                \
        const long slots = (long)B * npad;                                                                         \
        fvt_force_fwd_kernel<T><<<(unsigned)((slots + 7) / 8), 256, 0, st>>>(force, B, npad, nghost, umax, binum,  \
                                                                            bilist, numneigh, firstneigh, de);     \
        AI2B_CUDA(cudaGetLastError());                                                                             \
        return AI2B_OK;                                                                                            \
    }                                                                                                              \
    extern "C" int ai2b_fvt_force_bwd_##SUF(T *gde, int B, int npad, int nghost, int umax, const int *binum,       \
                                            const int *bilist, const int *numneigh, const int *firstneigh,         \
                                            const T *gforce, void *stream)                                         \
    {                                                                                                              \
        AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0 && nghost >= 0, AI2B_ERR_INVALID, "fvt: negative size");      \
        const long n = (long)B * npad * umax;                                                                      \
        if (n == 0) return AI2B_OK;                                                                                \
        AI2B_REQUIRE(gde && binum && bilist && numneigh && firstneigh && gforce, AI2B_ERR_INVALID, "fvt: NULL");    \
        fvt_force_bwd_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(                    \
            gde, B, npad, nghost, umax, binum, bilist, numneigh, firstneigh, gforce);                              \
        AI2B_CUDA(cudaGetLastError());                                                                             \
        return AI2B_OK;                                                                                            \
    }                                                                                                              \
    extern "C" int ai2b_fvt_virial_fwd_##SUF(T *virial, int B, int npad, int umax, const int *numneigh,            \
                                             const T *rcs, const T *de, void *stream)                              \
    {                                                                                                              \
        AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0, AI2B_ERR_INVALID, "fvt: negative size");                     \
        if (B == 0) return AI2B_OK;                                                                                \
        AI2B_REQUIRE(virial, AI2B_ERR_INVALID, "fvt: NULL");                                                       \
        cudaStream_t st = (cudaStream_t)stream;                                                                    \
        AI2B_CUDA(cudaMemsetAsync(virial, 0, sizeof(T) * 9 * B, st));                                              \
        if (npad == 0 || umax == 0) return AI2B_OK;                                                                \
        AI2B_REQUIRE(numneigh && rcs && de, AI2B_ERR_INVALID, "fvt: NULL");                                        \
        long gx = ((long)npad * umax + 255) / 256;                                                                 \
        if (gx > 256) gx = 256;                                                                                    \
        fvt_virial_fwd_kernel<T><<<dim3((unsigned)gx, (unsigned)B), 256, 0, st>>>(virial, B, npad, umax, numneigh, \
                                                                                 rcs, de);                        \
        AI2B_CUDA(cudaGetLastError());                                                                             \
        return AI2B_OK;                                                                                            \
    }                                                                                                              \
    extern "C" int ai2b_fvt_virial_bwd_##SUF(T *gde, T *grcs, int B, int npad, int umax, const int *numneigh,      \
                                             const T *rcs, const T *de, const T *gvirial, void *stream)            \
    {                                                                                                              \
        AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0, AI2B_ERR_INVALID, "fvt: negative size");                     \
        const long n = (long)B * npad * umax;                                                                      \
        if (n == 0) return AI2B_OK;                                                                                \
        AI2B_REQUIRE(gde && numneigh && rcs && de && gvirial, AI2B_ERR_INVALID, "fvt: NULL");                      \
        fvt_virial_bwd_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(                   \
            gde, grcs, B, npad, umax, numneigh, rcs, de, gvirial);                                                 \
        AI2B_CUDA(cudaGetLastError());                                                                             \
        return AI2B_OK;                                                                                            \
    }

AI2B_DEF_FVT(f64, double)
AI2B_DEF_FVT(f32, float)
