// ZBL screened-Coulomb pair correction (energy, force on the centre atom, virial), added onto the
// outputs of an MTP or NEP evaluation when a model sets zbl_rmax > 0.
//
// Reference semantics: pair functions source/descriptor/correction/include/zbl.h:276-395
// (switch, screening function phi, pair energy, force, virial), applied per directed pair as the
// reference's CUDA path does (source/descriptor/correction/gpu/include/zbl.cuh:423-500):
//   E     += 1/2 E_pair(r),  E_pair = K Zi Zj / r * phi(r / a) * s(r)
//   F_i   += dE_pair/dr * r_vec / r            (r_vec = r_j - r_i; the pair is met again from j)
//   V_ab  += -1/2 r_a (dE_pair/dr r_b / r)
// for every listed neighbour with r <= rmax; a = 0.46848 / (Zi^0.23 + Zj^0.23), atomic numbers
// from type_map. One warp per centre atom, lanes = neighbours; energy and virial are summed per
// block before they touch global memory.
#include "common.cuh"

namespace ai2b {

constexpr int ZBL_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(ZBL_WARPS * 32)
zbl_kernel(T *__restrict__ etot, T *__restrict__ force, T *__restrict__ virial, int npad, const int *__restrict__ binum,
           const int *__restrict__ bilist, const int *__restrict__ numneigh, const int *__restrict__ firstneigh,
           const T *__restrict__ rcs, const int *__restrict__ btypes, int ntypes, const int *__restrict__ type_map, int umax,
           int nghost, T rmax, T rmin, const T *__restrict__ cks, const T *__restrict__ dks)
{
    __shared__ T acc[10];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 10) acc[threadIdx.x] = T(0);
    __syncthreads();
    const int inum = binum[b];
    const int *types = btypes + (size_t)b * (npad + nghost);
    T *frc = force + (size_t)b * (npad + nghost) * 3;
    const double KC = 14.399645;   // 1 / (4 pi eps0) in eV A (zbl.h:34)
    T e = T(0), v[9];
#pragma unroll
    for (int k = 0; k < 9; k++) v[k] = T(0);
    for (int ii = blockIdx.x * ZBL_WARPS + warp; ii < inum; ii += gridDim.x * ZBL_WARPS) {
        const size_t slot = (size_t)b * npad + ii;
        const int ci = bilist[slot];
        const int ti = types[ci];
        const int nn = min(numneigh[slot], umax);
        const double zi = (double)type_map[ti];
        const double pzi = pow(zi, 0.23);
        T fx = T(0), fy = T(0), fz = T(0);
        for (int j = lane; j < nn; j += 32) {
            const T *rc = rcs + (slot * umax + j) * 3;
            const T x = rc[0], y = rc[1], z = rc[2];
            const T r = gsqrt(x * x + y * y + z * z);
            if (!(r <= rmax) || !(r > T(0))) continue;
            const int tj = types[firstneigh[slot * umax + j]];
            const double zj = (double)type_map[tj];
            const T a = (T)(0.46848 / (pzi + pow(zj, 0.23)));
            const T *ck = cks + 4 * (ti * ntypes + tj), *dk = dks + 4 * (ti * ntypes + tj);
            const T xa = r / a;
            T phi = T(0), dphi = T(0);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const T ex = (T)exp((double)(-dk[k] * xa));
                phi += ck[k] * ex;
                dphi -= ck[k] * dk[k] / a * ex;
            }
            T sw = T(1), dsw = T(0);
            if (r >= rmin) {
                const T u = (r - rmin) / (rmax - rmin);
                sw = u * u * u * (T(-6) * u * u + T(15) * u - T(10)) + T(1);
                dsw = T(1) / (rmax - rmin) * (T(-30) * u * u * u * u + T(60) * u * u * u - T(30) * u * u);
            }
            const T A = (T)(KC * zi * zj / (double)r), dA = (T)(-KC * zi * zj / ((double)r * (double)r));
            e += T(0.5) * A * phi * sw;
            const T s = (dA * phi * sw + A * dphi * sw + A * phi * dsw) / r;   // dE/dr / r
            const T gx = s * x, gy = s * y, gz = s * z;
            fx += gx; fy += gy; fz += gz;
            if (virial) {
                v[0] -= T(0.5) * x * gx; v[1] -= T(0.5) * x * gy; v[2] -= T(0.5) * x * gz;
                v[3] -= T(0.5) * y * gx; v[4] -= T(0.5) * y * gy; v[5] -= T(0.5) * y * gz;
                v[6] -= T(0.5) * z * gx; v[7] -= T(0.5) * z * gy; v[8] -= T(0.5) * z * gz;
            }
        }
        fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
        if (lane == 0 && (fx != T(0) || fy != T(0) || fz != T(0))) {
            atomicAdd(frc + 3 * ci + 0, fx);
            atomicAdd(frc + 3 * ci + 1, fy);
            atomicAdd(frc + 3 * ci + 2, fz);
        }
    }
    e = warp_sum(e);
    if (lane == 0) atomicAdd(&acc[0], e);
    if (virial) {
#pragma unroll
        for (int k = 0; k < 9; k++) {
            const T s = warp_sum(v[k]);
            if (lane == 0) atomicAdd(&acc[1 + k], s);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(etot + b, acc[0]);
    else if (threadIdx.x < 10 && virial) atomicAdd(virial + 9 * b + threadIdx.x - 1, acc[threadIdx.x]);
}

template <typename T>
static int zbl_launch(T *etot, T *force, T *virial, int B, int npad, const int *binum, const int *bilist, const int *numneigh,
                      const int *firstneigh, const T *rcs, const int *types, int ntypes, const int *type_map, int umax, int nghost,
                      T rmax, T rmin, const T *cks, const T *dks, cudaStream_t st)
{
    AI2B_REQUIRE(etot && force && binum && bilist && numneigh && firstneigh && rcs && types && type_map && cks && dks,
                 AI2B_ERR_INVALID, "ai2b_zbl_efv: NULL argument");
    AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0 && ntypes >= 1 && nghost >= 0, AI2B_ERR_INVALID, "ai2b_zbl_efv: negative size");
    AI2B_REQUIRE(rmax > rmin && rmin >= T(0), AI2B_ERR_INVALID, "ai2b_zbl_efv: need 0 <= rmin < rmax");
    if (B == 0 || npad == 0) return AI2B_OK;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long bx = ((long)npad + ZBL_WARPS - 1) / ZBL_WARPS;
    const long cap = std::max(1L, (long)sms * 8 / B);
    if (bx > cap) bx = cap;
    AI2B_REQUIRE(B <= 65535, AI2B_ERR_UNSUPPORTED, "ai2b_zbl_efv: more than 65535 structures per call");
    zbl_kernel<T><<<dim3((unsigned)bx, (unsigned)B), ZBL_WARPS * 32, 0, st>>>(etot, force, virial, npad, binum, bilist, numneigh, firstneigh,
                                                                             rcs, types, ntypes, type_map, umax, nghost, rmax, rmin, cks, dks);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" int ai2b_zbl_efv_f64(double *etot, double *force, double *virial, int B, int npad, const int *binum, const int *bilist,
                                const int *numneigh, const int *firstneigh, const double *rcs, const int *types, int ntypes,
                                const int *type_map, int umax, int nghost, double rmax, double rmin, const double *cks,
                                const double *dks, void *stream)
{
    return zbl_launch<double>(etot, force, virial, B, npad, binum, bilist, numneigh, firstneigh, rcs, types, ntypes, type_map, umax,
                              nghost, rmax, rmin, cks, dks, (cudaStream_t)stream);
}
extern "C" int ai2b_zbl_efv_f32(float *etot, float *force, float *virial, int B, int npad, const int *binum, const int *bilist,
                                const int *numneigh, const int *firstneigh, const float *rcs, const int *types, int ntypes,
                                const int *type_map, int umax, int nghost, float rmax, float rmin, const float *cks,
                                const float *dks, void *stream)
{
    return zbl_launch<float>(etot, force, virial, B, npad, binum, bilist, numneigh, firstneigh, rcs, types, ntypes, type_map, umax,
                             nghost, rmax, rmin, cks, dks, (cudaStream_t)stream);
}
