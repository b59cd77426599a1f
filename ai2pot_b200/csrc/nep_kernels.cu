// NEP (3-body): descriptors, per-type network, force and virial on sm_100a.
//
// Reference semantics: source/descriptor/nep/include/basis.h:137-159,300-333,519-530 (radial
// functions), nep_utilities.h:25-31,100-383 (3-body coefficients, harmonic polynomials),
// nepBasis.h:57-196 (sums), nep.h:320-529 (network, force, virial).
//
// Eight lanes evaluate one centre atom (four atoms per warp). Lanes are neighbours:
//   1. radial pass over all neighbours: q_n = sum_j g_n(r_j); neighbours inside the angular
//      cutoff are compacted into a per-atom list (group ballot)
//   2. angular pass over that list: S_{mu,lm} = sum_j g_mu(r_j) B_lm(u_j) with u = r_vec/r
//      (B_lm is homogeneous of degree l, so B_lm(r_vec)/r^l = B_lm(u)); lane sums by a
//      transpose-reduce over the eight lanes
//   3. q_{mu,l} = sum_m w_m C_lm S^2, network forward/backward with lanes over neurons
//   4. force passes: radial  g = (sum_n dE/dq_n g'_n) u;
//      angular g = sum_mu [ g'_mu P u + g_mu/r (G - (u.G) u) ],  P = sum_lm e_lm B_lm(u),
//      G = sum_lm e_lm grad B_lm(u);  F_i += g, F_j -= g, V -= g (x) r
#include "common.cuh"
#include <cuda_pipeline.h>

#include <cstring>
#include <algorithm>

namespace ai2b {

constexpr int NEP_GROUP = 8;                  // lanes per atom
constexpr int NEP_APW = 32 / NEP_GROUP;       // atoms per warp
constexpr int NEP_WARPS = 4;
constexpr int NEP_APB = NEP_APW * NEP_WARPS;  // atoms per block
constexpr int NEP_NLM = 24;

enum NepMode { NEP_EFV = 0, NEP_EF = 1, NEP_DESC = 2 };

template <typename T>
struct NepArgs {
    T *etot, *force, *virial, *desc;
    const T *coeffs_pad;   // [ntypes*ntypes][n_r+n_a][CSP] zero-padded copy (workspace)
    const T *w0, *b0, *w1, *bias, *qs;
    const int *binum, *bilist, *numneigh, *firstneigh, *types;
    const T *rcs;
    const int *prefix;
    int B, npad, ntypes, umax, nghost, cs, n_r, n_a, l_max, nneu, nd, nS;
    T rc_r, rc_a;
};

// 3-body coefficients as the reference stores them: double literals, some written with an `f`
// suffix and therefore rounded to float first (nep_utilities.h:25-31).
__constant__ double c_C3B[NEP_NLM] = {
    0.238732414637843, (double)0.119366207318922f, (double)0.119366207318922f, (double)0.099471839432435f,
    0.596831036594608, (double)0.596831036594608f, (double)0.149207759148652f, (double)0.149207759148652f,
    0.139260575205408, (double)0.104445431404056f, (double)0.104445431404056f, (double)1.044454314040563f,
    1.044454314040563, (double)0.174075719006761f, (double)0.174075719006761f, (double)0.011190581936149f,
    0.223811638722978, (double)0.223811638722978f, (double)0.111905819361489f, (double)0.111905819361489f,
    1.566681471060845, (double)1.566681471060845f, (double)0.195835183882606f, (double)0.195835183882606f};

__device__ __forceinline__ float gtanh(float x) { return tanhf(x); }
__device__ __forceinline__ double gtanh(double x) { return tanh(x); }
// sin(pi x), cos(pi x): exact argument reduction, no slow path for large arguments
__device__ __forceinline__ void gsincospi(float x, float *s, float *c) { sincospif(x, s, c); }
__device__ __forceinline__ void gsincospi(double x, double *s, double *c) { sincospi(x, s, c); }

// f_k = fc (T_k(x)+1)/2 and d f_k / dr, k < CSP (entries >= cs meet zero coefficients)
template <typename T, int CSP>
__device__ __forceinline__ void nep_radial(T r, T rc, T (&f)[CSP], T (&df)[CSP])
{
    const T pi = T(3.14159265358979323846);
    T sn, cn;
    gsincospi(r / rc, &sn, &cn);
    const T fc = T(0.5) * (T(1) + cn), dfc = T(-0.5) * sn * pi / rc;
    const T s = r / rc - T(1);
    const T x = T(2) * s * s - T(1), xc = T(4) / rc * s;
    T t0 = T(1), t1 = x, d0 = T(0), d1 = T(1);
#pragma unroll
    for (int k = 0; k < CSP; k++) {
        T t, d;
        if (k == 0) { t = T(1); d = T(0); }
        else if (k == 1) { t = x; d = T(1); }
        else {
            t = T(2) * x * t1 - t0;
            d = T(2) * t1 + T(2) * x * d1 - d0;
            t0 = t1; t1 = t; d0 = d1; d1 = d;
        }
        const T v = (t + T(1)) * T(0.5), dv = xc * (d * T(0.5));
        f[k] = fc * v;
        df[k] = dfc * v + fc * dv;
    }
}

// A gradient component that is identically zero: accumulating it is skipped at compile time.
struct NepZero {};
template <typename T> __device__ __forceinline__ void nep_set(T &d, T v) { d = v; }
template <typename T> __device__ __forceinline__ void nep_set(T &d, NepZero) { d = T(0); }
template <typename T, int N>
__device__ __forceinline__ void nep_acc(const T (&e)[N], T v, T (&acc)[N])
{
#pragma unroll
    for (int i = 0; i < N; i++) acc[i] = fma(e[i], v, acc[i]);
}
template <typename T, int N>
__device__ __forceinline__ void nep_acc(const T (&)[N], NepZero, T (&)[N]) {}

// Harmonic polynomials b[l*l-1+m] (l = 1..4) at (x,y,z) and their Cartesian gradients (closed
// forms tabulated in nep_utilities.h:100-383), as a list X(index, value, d/dx, d/dy, d/dz) over
// the products defined by NEP_POLY_COMMON.
#define NEP_POLY_COMMON(x, y, z)                                                                       \
    const T r2 = x * x + y * y + z * z, x2 = x * x, y2 = y * y, z2 = z * z;                           \
    const T xy = x * y, xz = x * z, yz = y * z, xmy = x2 - y2;
#define NEP_Z NepZero{}
#define NEP_FOR_EACH_LM(X, x, y, z)                                                                    \
    X(0, z, NEP_Z, NEP_Z, T(1))                                                                        \
    X(1, x, T(1), NEP_Z, NEP_Z)                                                                        \
    X(2, y, NEP_Z, T(1), NEP_Z)                                                                        \
    X(3, T(3) * z2 - r2, T(-2) * x, T(-2) * y, T(4) * z)                                               \
    X(4, xz, z, NEP_Z, x)                                                                              \
    X(5, yz, NEP_Z, z, y)                                                                              \
    X(6, xmy, T(2) * x, T(-2) * y, NEP_Z)                                                              \
    X(7, T(2) * xy, T(2) * y, T(2) * x, NEP_Z)                                                         \
    X(8, (T(5) * z2 - T(3) * r2) * z, T(-6) * xz, T(-6) * yz, T(9) * z2 - T(3) * r2)                   \
    X(9, (T(5) * z2 - r2) * x, T(-2) * x2 + T(5) * z2 - r2, T(-2) * xy, T(8) * xz)                     \
    X(10, (T(5) * z2 - r2) * y, T(-2) * xy, T(-2) * y2 + T(5) * z2 - r2, T(8) * yz)                    \
    X(11, xmy * z, T(2) * xz, T(-2) * yz, xmy)                                                         \
    X(12, T(2) * xy * z, T(2) * yz, T(2) * xz, T(2) * xy)                                              \
    X(13, (x2 - T(3) * y2) * x, T(3) * xmy, T(-6) * xy, NEP_Z)                                         \
    X(14, (T(3) * x2 - y2) * y, T(6) * xy, T(3) * xmy, NEP_Z)                                          \
    X(15, (T(35) * z2 - T(30) * r2) * z2 + T(3) * r2 * r2, T(-60) * x * z2 + T(12) * r2 * x,           \
      T(-60) * y * z2 + T(12) * r2 * y, T(80) * z2 * z - T(48) * r2 * z)                               \
    X(16, (T(7) * z2 - T(3) * r2) * xz, T(-6) * x2 * z + T(7) * z2 * z - T(3) * r2 * z, T(-6) * xy * z, \
      T(15) * x * z2 - T(3) * r2 * x)                                                                  \
    X(17, (T(7) * z2 - T(3) * r2) * yz, T(-6) * xy * z, T(-6) * y2 * z + T(7) * z2 * z - T(3) * r2 * z, \
      T(15) * y * z2 - T(3) * r2 * y)                                                                  \
    X(18, (T(7) * z2 - r2) * xmy, T(-2) * x2 * x + T(2) * x * y2 + T(14) * x * z2 - T(2) * r2 * x,     \
      T(-2) * x2 * y + T(2) * y2 * y - T(14) * y * z2 + T(2) * r2 * y, T(12) * z * xmy)                \
    X(19, (T(7) * z2 - r2) * T(2) * xy, T(-4) * x2 * y + T(14) * y * z2 - T(2) * r2 * y,               \
      T(-4) * x * y2 + T(14) * x * z2 - T(2) * r2 * x, T(24) * xy * z)                                 \
    X(20, (x2 - T(3) * y2) * xz, T(3) * xmy * z, T(-6) * xy * z, (x2 - T(3) * y2) * x)                 \
    X(21, (T(3) * x2 - y2) * yz, T(6) * xy * z, T(3) * xmy * z, (T(3) * x2 - y2) * y)                  \
    X(22, xmy * xmy - T(4) * x2 * y2, T(4) * x2 * x - T(12) * x * y2, T(4) * y2 * y - T(12) * x2 * y, NEP_Z) \
    X(23, T(4) * xmy * xy, T(12) * x2 * y - T(4) * y2 * y, T(4) * x2 * x - T(12) * x * y2, NEP_Z)

template <typename T, bool GRAD>
__device__ __forceinline__ void nep_blm(T x, T y, T z, T (&b)[NEP_NLM], T (&g)[GRAD ? NEP_NLM : 1][3])
{
    NEP_POLY_COMMON(x, y, z)
#define NEP_SET(k, val, gx, gy, gz)                                                       \
    b[k] = (val);                                                                         \
    if constexpr (GRAD) { nep_set<T>(g[k][0], gx); nep_set<T>(g[k][1], gy); nep_set<T>(g[k][2], gz); }
    NEP_FOR_EACH_LM(NEP_SET, x, y, z)
#undef NEP_SET
}

// Sum over the 8 lanes of a group. `gmask` names exactly the group's lanes: the four groups of a
// warp run loops of different trip counts (their atoms have different neighbour counts), so a
// full-warp mask inside those loops would wait for lanes that never arrive.
template <typename T>
__device__ __forceinline__ T group_sum(T v, unsigned gmask)
{
    v += __shfl_xor_sync(gmask, v, 4);
    v += __shfl_xor_sync(gmask, v, 2);
    v += __shfl_xor_sync(gmask, v, 1);
    return v;
}
// 8 values per lane -> lane `sub` of each group holds the group total of v[sub]
template <typename T>
__device__ __forceinline__ T group_xreduce8(T (&v)[8], int sub, unsigned gmask)
{
    int o = 4;
#pragma unroll
    for (int h = 4; h >= 1; h >>= 1, o >>= 1) {
        const bool up = (sub & o) != 0;
#pragma unroll
        for (int i = 0; i < h; i++) {
            T send = up ? v[i] : v[i + h];
            T keep = up ? v[i + h] : v[i];
            v[i] = keep + __shfl_xor_sync(gmask, send, o);
        }
    }
    return v[0];
}

template <typename T>
__global__ void nep_pad_coeffs_kernel(const T *__restrict__ c, T *__restrict__ out, int rows, int cs, int csp)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * csp) return;
    int r = i / csp, k = i % csp;
    out[i] = k < cs ? c[r * cs + k] : T(0);
}

// zeroes up to three output arrays in one launch (instead of one memset per array)
template <typename T>
__global__ void nep_zero_kernel(T *__restrict__ a, size_t na, T *__restrict__ b, size_t nb, T *__restrict__ c, size_t nc)
{
    chain_release();
    chain_wait();
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = i0; i < na; i += step) a[i] = T(0);
    for (size_t i = i0; i < nb; i += step) b[i] = T(0);
    for (size_t i = i0; i < nc; i += step) c[i] = T(0);
}
template <typename T>
static int nep_zero_outputs(T *etot, size_t ne, T *force, size_t nf, T *virial, size_t nv, cudaStream_t st)
{
    const size_t n = ne + nf + nv;
    if (n == 0) return AI2B_OK;
    size_t blocks = (n + 4 * 256 - 1) / (4 * 256);
    if (blocks > 4096) blocks = 4096;
    AI2B_CUDA(launch_chained(nep_zero_kernel<T>, (unsigned)blocks, 256, 0, st, etot, ne, force, nf, virial, virial ? nv : size_t(0)));
    return AI2B_OK;
}

__global__ void nep_prefix_kernel(const int *__restrict__ binum, int B, int *__restrict__ prefix)
{
    // B is small (structures per batch): one thread is enough
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int s = 0;
        prefix[0] = 0;
        for (int b = 0; b < B; b++) { s += binum[b]; prefix[b + 1] = s; }
    }
}

__host__ __device__ inline int nep_atom_elems(int nd, int nS, int nneu)
{
    auto r4 = [](int n) { return (n + 3) & ~3; };
    return 2 * r4(nd) + 2 * r4(nS) + r4(nneu);   // q, Eq, S, ES, a
}

template <typename T, int CSP, int MODE>
__global__ void __launch_bounds__(NEP_WARPS * 32) nep_atom_kernel(const NepArgs<T> A)
{
    extern __shared__ __align__(16) unsigned char nep_smem[];
    __shared__ T blk_acc[10];   // energy + virial of the structure most of this block's atoms belong to
    __shared__ int blk_b;
    __shared__ T iqs[96];       // 1 / q_scaler (descriptor count <= 20 + 12*4 = 68)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane & (NEP_GROUP - 1), grp = lane / NEP_GROUP;
    const int slot_in_block = warp * NEP_APW + grp;
    const unsigned gmask_shift = grp * NEP_GROUP;
    const unsigned gmask = 0xffu << gmask_shift;
    auto r4 = [](int n) { return (n + 3) & ~3; };
    const int per_atom = nep_atom_elems(A.nd, A.nS, A.nneu);
    T *q = reinterpret_cast<T *>(nep_smem) + (size_t)slot_in_block * per_atom;
    T *Eq = q + r4(A.nd);
    T *S = Eq + r4(A.nd);
    T *ES = S + r4(A.nS);
    T *act = ES + r4(A.nS);
    unsigned short *alist = reinterpret_cast<unsigned short *>(reinterpret_cast<T *>(nep_smem) + (size_t)NEP_APB * per_atom) +
                            (size_t)slot_in_block * A.umax;
    const int ntot_n = A.n_r + A.n_a;
    const int nlm = A.l_max * A.l_max + 2 * A.l_max;
    if (MODE != NEP_DESC) {
        for (int k = threadIdx.x; k < A.nd; k += blockDim.x) iqs[k] = T(1) / A.qs[k];
        __syncthreads();
    }

    const int ntot = A.prefix[A.B];
    const int ngroups = gridDim.x * NEP_APB;
    const int gidx = blockIdx.x * NEP_APB + slot_in_block;
    // atoms are dealt to groups in contiguous chunks; all groups of a warp run the same trip count
    const int chunk = (ntot + ngroups - 1) / ngroups;

    for (int it = 0; it < chunk; it++) {
        const int t = gidx * chunk + it;
        const bool valid = t < ntot;
        int b = 0;
        if (valid) {
            int lo = 0, hi = A.B;
            while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (A.prefix[mid] <= t) lo = mid; else hi = mid; }
            b = lo;
        }
        const int ii = valid ? t - A.prefix[b] : 0;
        const size_t slot = (size_t)b * A.npad + ii;
        const int ci = valid ? A.bilist[slot] : 0;
        const int nn = valid ? min(A.numneigh[slot], A.umax) : 0;
        const int *types = A.types + (size_t)b * (A.npad + (MODE == NEP_DESC ? 0 : A.nghost));
        const int ti = valid ? types[ci] : 0;
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;
        const T *ctab = A.coeffs_pad + (size_t)ti * A.ntypes * ntot_n * CSP;

        if (MODE != NEP_DESC) {
            if (threadIdx.x == 0) blk_b = valid ? b : -1;
            if (threadIdx.x < 10) blk_acc[threadIdx.x] = T(0);
            __syncthreads();
        }
        for (int i = sub; i < A.nd; i += NEP_GROUP) q[i] = T(0);
        for (int i = sub; i < A.nS; i += NEP_GROUP) S[i] = T(0);
        __syncwarp();

        // ---- 1. radial pass + compaction of the angular neighbours -----------------------------
        int nang = 0;
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {
            const int j = j0 + sub;
            bool on = j < nn;
            T x = 0, y = 0, z = 0;
            int tj = 0;
            if (on) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; }
            const T r = gsqrt(x * x + y * y + z * z);
            on = on && r <= A.rc_r && r > T(0);
            if (on) tj = types[fn[j]];
            T f[CSP], df[CSP];
            nep_radial<T, CSP>(on ? r : A.rc_r, A.rc_r, f, df);
            const T *crow = ctab + (size_t)tj * ntot_n * CSP;
            for (int n = 0; n < A.n_r; n++) {
                T g = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k++) g = fma(crow[n * CSP + k], f[k], g);
                g = group_sum(on ? g : T(0), gmask);
                if (sub == (n & (NEP_GROUP - 1))) q[n] += g;
            }
            const bool ang = on && r <= A.rc_a && A.l_max > 0;
            const unsigned bal = (__ballot_sync(gmask, ang) >> gmask_shift) & 0xffu;
            if (ang) alist[nang + __popc(bal & ((1u << sub) - 1u))] = (unsigned short)j;
            nang += __popc(bal);
        }
        __syncwarp();

        // ---- 2. angular sums ------------------------------------------------------------------------
        for (int k0 = 0; k0 < nang; k0 += NEP_GROUP) {
            const bool on = k0 + sub < nang;
            T x = 0, y = 0, z = 0, rinv = 0, r = A.rc_a;
            int tj = 0;
            if (on) {
                const int j = alist[k0 + sub];
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
                r = gsqrt(x * x + y * y + z * z);
                rinv = T(1) / r;
                tj = types[fn[j]];
            }
            T f[CSP], df[CSP], bl[NEP_NLM], gdummy[1][3];
            nep_radial<T, CSP>(r, A.rc_a, f, df);
            nep_blm<T, false>(x * rinv, y * rinv, z * rinv, bl, gdummy);
            const T *crow = ctab + ((size_t)tj * ntot_n + A.n_r) * CSP;
            for (int mu = 0; mu < A.n_a; mu++) {
                T g = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k++) g = fma(crow[mu * CSP + k], f[k], g);
                if (!on) g = T(0);
#pragma unroll
                for (int c = 0; c < 3; c++) {
                    if (8 * c < nlm) {
                        T v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = g * bl[8 * c + i];
                        const T s = group_xreduce8<T>(v, sub, gmask);
                        if (8 * c + sub < nlm) S[mu * nlm + 8 * c + sub] += s;
                    }
                }
            }
        }
        __syncwarp();

        // ---- 3. angular descriptors, network -----------------------------------------------------------
        for (int p = sub; p < A.n_a * A.l_max; p += NEP_GROUP) {
            const int mu = p / A.l_max, l = p % A.l_max + 1;
            T acc = T(0);
            for (int mp = 0; mp < 2 * l + 1; mp++) {
                const int lm = l * l - 1 + mp;
                const T s = S[mu * nlm + lm];
                acc += (mp == 0 ? T(1) : T(2)) * (T)c_C3B[lm] * s * s;
            }
            q[A.n_r + p] = acc;
        }
        __syncwarp();
        if (MODE == NEP_DESC) {
            if (valid)
                for (int k = sub; k < A.nd; k += NEP_GROUP) A.desc[slot * A.nd + k] = q[k];
            __syncwarp();
            continue;
        }
        const T *W0 = A.w0 + (size_t)ti * A.nneu * A.nd, *B0 = A.b0 + (size_t)ti * A.nneu, *W1 = A.w1 + (size_t)ti * A.nneu;
        // network on the scaled descriptors q_k / q_scaler_k (kept in Eq until the backward pass overwrites it)
        for (int k = sub; k < A.nd; k += NEP_GROUP) Eq[k] = q[k] * iqs[k];
        __syncwarp();
        T es = T(0);
        for (int p = sub; p < A.nneu; p += NEP_GROUP) {
            const T *wrow = W0 + p * A.nd;
            T h0 = T(0), h1 = T(0);
            int k = 0;
            for (; k + 1 < A.nd; k += 2) {
                h0 = fma(wrow[k], Eq[k], h0);
                h1 = fma(wrow[k + 1], Eq[k + 1], h1);
            }
            if (k < A.nd) h0 = fma(wrow[k], Eq[k], h0);
            const T th = gtanh(h0 + h1 + B0[p]);
            es += W1[p] * th;
            act[p] = W1[p] * (T(1) - th * th);
        }
        es = group_sum(es, gmask);
        __syncwarp();
        for (int k = sub; k < A.nd; k += NEP_GROUP) {
            T a0 = T(0), a1 = T(0);
            int p = 0;
            for (; p + 1 < A.nneu; p += 2) {
                a0 = fma(act[p], W0[p * A.nd + k], a0);
                a1 = fma(act[p + 1], W0[(p + 1) * A.nd + k], a1);
            }
            if (p < A.nneu) a0 = fma(act[p], W0[p * A.nd + k], a0);
            Eq[k] = (a0 + a1) * iqs[k];
        }
        __syncwarp();
        for (int i = sub; i < A.nS; i += NEP_GROUP) {
            const int mu = i / nlm, lm = i % nlm;
            int l = 1;
            while ((l + 1) * (l + 1) - 1 <= lm) ++l;
            const int mp = lm - (l * l - 1);
            ES[i] = (mp == 0 ? T(1) : T(2)) * Eq[A.n_r + mu * A.l_max + l - 1] * T(2) * (T)c_C3B[lm] * S[i];
        }
        __syncwarp();

        // ---- 4. force / virial -------------------------------------------------------------------------
        T *frc = A.force + (size_t)b * (A.npad + A.nghost) * 3;
        T fcx = 0, fcy = 0, fcz = 0, vir[9];
#pragma unroll
        for (int k = 0; k < 9; k++) vir[k] = T(0);
        auto scatter = [&](bool on, int nj, T gx, T gy, T gz, T x, T y, T z) {
            if (!on) return;
            fcx += gx; fcy += gy; fcz += gz;
            atomicAdd(frc + 3 * nj + 0, -gx);
            atomicAdd(frc + 3 * nj + 1, -gy);
            atomicAdd(frc + 3 * nj + 2, -gz);
            if (MODE == NEP_EFV) {
                vir[0] -= gx * x; vir[1] -= gx * y; vir[2] -= gx * z;
                vir[3] -= gy * x; vir[4] -= gy * y; vir[5] -= gy * z;
                vir[6] -= gz * x; vir[7] -= gz * y; vir[8] -= gz * z;
            }
        };
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {     // radial part
            const int j = j0 + sub;
            bool on = j < nn;
            T x = 0, y = 0, z = 0;
            int nj = 0, tj = 0;
            if (on) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j]; }
            const T r = gsqrt(x * x + y * y + z * z);
            on = on && r <= A.rc_r && r > T(0);
            if (on) tj = types[nj];
            T f[CSP], df[CSP];
            nep_radial<T, CSP>(on ? r : A.rc_r, A.rc_r, f, df);
            const T *crow = ctab + (size_t)tj * ntot_n * CSP;
            T gr = T(0);
            for (int n = 0; n < A.n_r; n++) {
                T g = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k++) g = fma(crow[n * CSP + k], df[k], g);
                gr = fma(Eq[n], g, gr);
            }
            const T s = on ? gr / r : T(0);
            scatter(on, nj, s * x, s * y, s * z, x, y, z);
        }
        for (int k0 = 0; k0 < nang; k0 += NEP_GROUP) {   // angular part
            const bool on = k0 + sub < nang;
            T x = 0, y = 0, z = 0, rinv = 0, r = A.rc_a;
            int nj = 0, tj = 0;
            if (on) {
                const int j = alist[k0 + sub];
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
                r = gsqrt(x * x + y * y + z * z);
                rinv = T(1) / r;
                nj = fn[j];
                tj = types[nj];
            }
            const T ux = x * rinv, uy = y * rinv, uz = z * rinv;
            T f[CSP], df[CSP], bl[NEP_NLM], gb[NEP_NLM][3];
            nep_radial<T, CSP>(r, A.rc_a, f, df);
            nep_blm<T, true>(ux, uy, uz, bl, gb);
            const T *crow = ctab + ((size_t)tj * ntot_n + A.n_r) * CSP;
            T gx = 0, gy = 0, gz = 0;
            for (int mu = 0; mu < A.n_a; mu++) {
                T g = T(0), dg = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k++) {
                    const T cc = crow[mu * CSP + k];
                    g = fma(cc, f[k], g);
                    dg = fma(cc, df[k], dg);
                }
                T Pv = 0, Gx = 0, Gy = 0, Gz = 0;
                const T *es_mu = ES + mu * nlm;
#pragma unroll
                for (int lm = 0; lm < NEP_NLM; lm++) {
                    if (lm < nlm) {
                        const T e = es_mu[lm];
                        Pv = fma(e, bl[lm], Pv);
                        Gx = fma(e, gb[lm][0], Gx);
                        Gy = fma(e, gb[lm][1], Gy);
                        Gz = fma(e, gb[lm][2], Gz);
                    }
                }
                const T ug = ux * Gx + uy * Gy + uz * Gz;
                const T a = dg * Pv - g * rinv * ug, c = g * rinv;
                gx += a * ux + c * Gx;
                gy += a * uy + c * Gy;
                gz += a * uz + c * Gz;
            }
            scatter(on, nj, gx, gy, gz, x, y, z);
        }
        fcx = group_sum(fcx, gmask); fcy = group_sum(fcy, gmask); fcz = group_sum(fcz, gmask);
        if (MODE == NEP_EFV) {
#pragma unroll
            for (int k = 0; k < 9; k++) vir[k] = group_sum(vir[k], gmask);
        }
        if (sub == 0 && valid) {
            atomicAdd(frc + 3 * ci + 0, fcx);
            atomicAdd(frc + 3 * ci + 1, fcy);
            atomicAdd(frc + 3 * ci + 2, fcz);
            const bool local = b == blk_b;
            atomicAdd(local ? &blk_acc[0] : A.etot + b, es + A.bias[ti]);
            if (MODE == NEP_EFV) {
#pragma unroll
                for (int k = 0; k < 9; k++) atomicAdd(local ? &blk_acc[1 + k] : A.virial + 9 * b + k, vir[k]);
            }
        }
        __syncthreads();
        if (threadIdx.x < 10 && blk_b >= 0) {
            const T v = blk_acc[threadIdx.x];
            if (threadIdx.x == 0) atomicAdd(A.etot + blk_b, v);
            else if (MODE == NEP_EFV) atomicAdd(A.virial + 9 * blk_b + threadIdx.x - 1, v);
        }
    }
}

}  // namespace ai2b
#include "nep_fast.cuh"
#include "nep_loss.cuh"
#include "nep_loss_fast.cuh"
namespace ai2b {

// ---------------------------------------------------------------------------------------------
static size_t nep_ws_bytes(int B, int ntypes, int n_r, int n_a, int csp, size_t elem)
{
    size_t pre = (((size_t)(B > 0 ? B : 0) + 1) * sizeof(int) + 255) & ~size_t(255);
    size_t co = ((size_t)ntypes * ntypes * (n_r + n_a) * csp * elem + 255) & ~size_t(255);
    return pre + co;
}

static int nep_grid(const void *kern, size_t smem, int B, int npad, long *blocks)
{
    int sms = 148, dev = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NEP_WARPS * 32, smem));
    if (per_sm < 1) per_sm = 1;
    *blocks = (long)sms * per_sm;
    const long need_blocks = ((long)B * npad + NEP_APB - 1) / NEP_APB;
    if (*blocks > need_blocks) *blocks = need_blocks;
    return AI2B_OK;
}

// Specialised kernel for n_radial, n_angular <= NMAX. *done = false if the model's tables or the
// neighbour width do not fit its shared-memory plan (the general kernel then runs).
template <typename T, int CSP, int MODE, int NMAX>
static int launch_nep_fast(const NepArgs<T> &A, const T *coeffs, cudaStream_t st, bool *done)
{
    constexpr int MINB = sizeof(T) == 4 ? 4 : 2;
    constexpr bool NET = MODE != NEP_DESC;
    *done = false;
    if (A.ntypes > 16 || A.nneu > 256 || A.umax > 1024) return AI2B_OK;
    const size_t smem = ((size_t)nep_fast_table_elems<NMAX, CSP>(A.ntypes, A.nneu, NET) +
                         (size_t)NEP_APB * nep_fast_atom_elems<NMAX>(A.nneu, A.umax, NET)) * sizeof(T) +
                        (size_t)NEP_APB * A.umax * sizeof(unsigned short) + 16;
    if (smem > 96 * 1024) return AI2B_OK;
    auto kern = nep_fast_kernel<T, CSP, MODE, NMAX, MINB>;
    static KernelSetup setup;
    if (int rc = kernel_setup(setup, kern, smem)) return rc;
    long blocks = 0;
    int rc = nep_grid((const void *)kern, smem, A.B, A.npad, &blocks);
    if (rc != AI2B_OK) return rc;
    AI2B_CUDA(launch_chained(kern, (unsigned)blocks, NEP_WARPS * 32, smem, st, A, coeffs));
    *done = true;
    return AI2B_OK;
}

template <typename T, int CSP, int MODE>
static int launch_nep_csp(NepArgs<T> A, const T *coeffs, void *ws, size_t ws_bytes, cudaStream_t st)
{
    const size_t need = nep_ws_bytes(A.B, A.ntypes, A.n_r, A.n_a, CSP, sizeof(T));
    AI2B_REQUIRE(ws && ws_bytes >= need, AI2B_ERR_WORKSPACE, "NEP workspace too small: %zu < %zu bytes", ws_bytes, need);
    int *prefix = reinterpret_cast<int *>(ws);
    T *cpad = reinterpret_cast<T *>(reinterpret_cast<unsigned char *>(ws) + ((((size_t)A.B + 1) * sizeof(int) + 255) & ~size_t(255)));
    A.prefix = prefix;
    A.coeffs_pad = cpad;
    bool have_prefix = false;
    if constexpr (CSP == 8) {
        if (A.n_r <= 8 && A.n_a <= 8) {
            // the specialised kernel reads the atom offsets only for batches of several structures
            if (A.B > 1) {
                nep_prefix_kernel<<<1, 32, 0, st>>>(A.binum, A.B, prefix);
                have_prefix = true;
            }
            bool done = false;
            int rc = (A.n_r <= 4 && A.n_a <= 4) ? launch_nep_fast<T, CSP, MODE, 4>(A, coeffs, st, &done)
                                                : launch_nep_fast<T, CSP, MODE, 8>(A, coeffs, st, &done);
            if (rc != AI2B_OK || done) return rc;
        }
    }
    if (!have_prefix) nep_prefix_kernel<<<1, 32, 0, st>>>(A.binum, A.B, prefix);
    const int rows = A.ntypes * A.ntypes * (A.n_r + A.n_a);
    nep_pad_coeffs_kernel<T><<<(rows * CSP + 255) / 256, 256, 0, st>>>(coeffs, cpad, rows, A.cs, CSP);
    const size_t smem = (size_t)NEP_APB * (nep_atom_elems(A.nd, A.nS, A.nneu) * sizeof(T) + (size_t)A.umax * sizeof(unsigned short)) + 16;
    AI2B_REQUIRE(smem <= 200 * 1024, AI2B_ERR_UNSUPPORTED, "NEP model/umax need %zu bytes of shared memory per block", smem);
    auto kern = nep_atom_kernel<T, CSP, MODE>;
    static KernelSetup setup;
    if (int rc = kernel_setup(setup, kern, smem)) return rc;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_sm = 0;
    AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NEP_WARPS * 32, smem));
    if (per_sm < 1) per_sm = 1;
    long blocks = (long)sms * per_sm;
    const long need_blocks = ((long)A.B * A.npad + NEP_APB - 1) / NEP_APB;
    if (blocks > need_blocks) blocks = need_blocks;
    kern<<<(unsigned)blocks, NEP_WARPS * 32, smem, st>>>(A);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

template <typename T, int MODE>
static int launch_nep(NepArgs<T> A, const T *coeffs, void *ws, size_t ws_bytes, cudaStream_t st)
{
    AI2B_REQUIRE(A.cs >= 1 && A.cs <= 16, AI2B_ERR_UNSUPPORTED, "chebyshev_size %d outside 1..16", A.cs);
    AI2B_REQUIRE(A.l_max >= 0 && A.l_max <= 4, AI2B_ERR_INVALID, "l_max %d outside 0..4", A.l_max);
    AI2B_REQUIRE(A.n_r >= 0 && A.n_a >= 0 && A.n_r + A.n_a > 0 && A.nneu >= 1 && A.ntypes >= 1, AI2B_ERR_INVALID, "bad NEP sizes");
    AI2B_REQUIRE(A.B >= 0 && A.npad >= 0 && A.umax >= 0 && A.umax < 65536 && A.nghost >= 0, AI2B_ERR_INVALID, "bad batch sizes");
    if (A.B == 0 || A.npad == 0) return AI2B_OK;
    A.nd = A.l_max == 0 ? A.n_r : A.n_r + A.n_a * A.l_max;
    A.nS = A.l_max == 0 ? 0 : A.n_a * (A.l_max * A.l_max + 2 * A.l_max);
    if (A.cs <= 8) return launch_nep_csp<T, 8, MODE>(A, coeffs, ws, ws_bytes, st);
    return launch_nep_csp<T, 16, MODE>(A, coeffs, ws, ws_bytes, st);
}

}  // namespace ai2b

using namespace ai2b;

extern "C" size_t ai2b_nep_workspace_bytes(int batch_size, int ntypes, int n_radial, int n_angular, int chebyshev_size, int is_f64)
{
    return nep_ws_bytes(batch_size, ntypes, n_radial, n_angular, chebyshev_size <= 8 ? 8 : 16, is_f64 ? 8 : 4);
}

#define AI2B_DEF_NEP(SUF, T)                                                                                    \
    static int nep_efv_entry_##SUF(bool zero, T *etot, T *force, T *virial, int cs, int n_r, int n_a, int l_max, int nneu, \
                                   const T *coeffs, const T *w0, const T *b0, const T *w1, const T *bias,       \
                                   int B, int npad, const int *binum, const int *bilist, const int *numneigh,   \
                                   const int *firstneigh, const T *rcs, const int *types, int ntypes,           \
                                   int umax, int nghost, T rc_r, T rc_a, const T *qs, void *ws,                 \
                                   size_t ws_bytes, void *stream)                                               \
    {                                                                                                           \
        AI2B_REQUIRE(etot && force && coeffs && w0 && b0 && w1 && bias && qs && binum && bilist && numneigh &&  \
                         firstneigh && rcs && types, AI2B_ERR_INVALID, "ai2b_nep_efv: NULL argument");          \
        cudaStream_t st = (cudaStream_t)stream;                                                                 \
        if (zero && B > 0 && npad >= 0) {                                                                       \
            if (int rc = nep_zero_outputs<T>(etot, (size_t)B, force, 3 * (size_t)B * (npad + nghost), virial,   \
                                             virial ? 9 * (size_t)B : 0, st)) return rc;                        \
        }                                                                                                       \
        NepArgs<T> A{etot, force, virial, nullptr, nullptr, w0, b0, w1, bias, qs, binum, bilist, numneigh,      \
                     firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, n_r, n_a, l_max, nneu, \
                     0, 0, rc_r, rc_a};                                                                         \
        return virial ? launch_nep<T, NEP_EFV>(A, coeffs, ws, ws_bytes, st)                                     \
                      : launch_nep<T, NEP_EF>(A, coeffs, ws, ws_bytes, st);                                     \
    }                                                                                                           \
    extern "C" int ai2b_nep_efv_##SUF(T *etot, T *force, T *virial, int cs, int n_r, int n_a, int l_max, int nneu, \
                                      const T *coeffs, const T *w0, const T *b0, const T *w1, const T *bias,    \
                                      int B, int npad, const int *binum, const int *bilist, const int *numneigh, \
                                      const int *firstneigh, const T *rcs, const int *types, int ntypes,        \
                                      int umax, int nghost, T rc_r, T rc_a, const T *qs, void *ws,              \
                                      size_t ws_bytes, void *stream)                                            \
    {                                                                                                           \
        return nep_efv_entry_##SUF(true, etot, force, virial, cs, n_r, n_a, l_max, nneu, coeffs, w0, b0, w1, bias, B, npad, \
                                   binum, bilist, numneigh, firstneigh, rcs, types, ntypes, umax, nghost, rc_r, rc_a, qs, ws, \
                                   ws_bytes, stream);                                                           \
    }                                                                                                           \
    extern "C" int ai2b_nep_efv_accumulate_##SUF(T *etot, T *force, T *virial, int cs, int n_r, int n_a, int l_max, \
                                                 int nneu, const T *coeffs, const T *w0, const T *b0, const T *w1, \
                                                 const T *bias, int B, int npad, const int *binum, const int *bilist, \
                                                 const int *numneigh, const int *firstneigh, const T *rcs,      \
                                                 const int *types, int ntypes, int umax, int nghost, T rc_r, T rc_a, \
                                                 const T *qs, void *ws, size_t ws_bytes, void *stream)          \
    {                                                                                                           \
        return nep_efv_entry_##SUF(false, etot, force, virial, cs, n_r, n_a, l_max, nneu, coeffs, w0, b0, w1, bias, B, npad, \
                                   binum, bilist, numneigh, firstneigh, rcs, types, ntypes, umax, nghost, rc_r, rc_a, qs, ws, \
                                   ws_bytes, stream);                                                           \
    }                                                                                                           \
    extern "C" int ai2b_nep_descriptors_##SUF(T *desc, int cs, int n_r, int n_a, int l_max, const T *coeffs,    \
                                              int B, int npad, const int *binum, const int *bilist,             \
                                              const int *numneigh, const int *firstneigh, const T *rcs,         \
                                              const int *types, int ntypes, int umax, int nghost, T rc_r,       \
                                              T rc_a, void *ws, size_t ws_bytes, void *stream)                  \
    {                                                                                                           \
        AI2B_REQUIRE(desc && coeffs && binum && bilist && numneigh && firstneigh && rcs && types,               \
                     AI2B_ERR_INVALID, "ai2b_nep_descriptors: NULL argument");                                  \
        cudaStream_t st = (cudaStream_t)stream;                                                                 \
        const int nd = l_max == 0 ? n_r : n_r + n_a * l_max;                                                    \
        if (B > 0 && npad > 0) AI2B_CUDA(cudaMemsetAsync(desc, 0, sizeof(T) * (size_t)B * npad * nd, st));      \
        NepArgs<T> A{nullptr, nullptr, nullptr, desc, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,     \
                     binum, bilist, numneigh, firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost,   \
                     cs, n_r, n_a, l_max, 1, 0, 0, rc_r, rc_a};                                                 \
        return launch_nep<T, NEP_DESC>(A, coeffs, ws, ws_bytes, st);                                            \
    }

AI2B_DEF_NEP(f64, double)
AI2B_DEF_NEP(f32, float)

#define AI2B_DEF_NEP_LOSS(SUF, T)                                                                                   \
    extern "C" int ai2b_nep_loss_backward_##SUF(                                                                    \
        T *dco, T *dw0, T *db0, T *dw1, T *dbi, T e_w, T f_w, T v_w, const T *e_ml, const T *e_dft, const T *f_ml,  \
        const T *f_dft, const T *v_ml, const T *v_dft, int cs, int n_r, int n_a, int l_max, int nneu, const T *coeffs, \
        const T *w0, const T *b0, const T *w1, int B, int npad, const int *binum, const int *bilist,                \
        const int *numneigh, const int *firstneigh, const T *rcs, const int *types, int ntypes, int umax, int nghost, \
        T rc_r, T rc_a, const T *qs, void *stream)                                                                  \
    {                                                                                                               \
        AI2B_REQUIRE(dco && dw0 && db0 && dw1 && dbi && e_ml && e_dft && f_ml && f_dft && coeffs && w0 && b0 && w1 && \
                         qs && binum && bilist && numneigh && firstneigh && rcs && types, AI2B_ERR_INVALID,         \
                     "ai2b_nep_loss_backward: NULL argument");                                                      \
        AI2B_REQUIRE((v_ml == nullptr) == (v_dft == nullptr), AI2B_ERR_INVALID,                                     \
                     "ai2b_nep_loss_backward: pass both virial tensors or neither");                                \
        NepArgs<T> A{nullptr, nullptr, nullptr, nullptr, nullptr, w0, b0, w1, nullptr, qs, binum, bilist, numneigh, \
                     firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, n_r, n_a, l_max, nneu,     \
                     0, 0, rc_r, rc_a};                                                                             \
        NepLossArgs<T> L{dco, dw0, db0, dw1, dbi, e_ml, e_dft, f_ml, f_dft, v_ml, v_dft, e_w, f_w, v_w};           \
        return launch_nep_loss_backward<T>(A, coeffs, L, (cudaStream_t)stream);                                     \
    }
AI2B_DEF_NEP_LOSS(f64, double)
AI2B_DEF_NEP_LOSS(f32, float)

// ---------------------------------------------------------------------------------------------
// NEP energy/force/virial for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: a molecular-dynamics driver that calls
// the potential from inside its timestep loop, where a cudaMalloc would stall every stream on
// the device; or a program whose device memory belongs entirely to its own pool and which has
// no hook for a plugin's scratch buffer. For them the scratch of ai2b_nep_efv_f32 (the
// per-structure atom offsets and the zero-padded radial coefficients) lives in a fixed array
// that is part of the library image: every GPU that loads the library carries these 128 KiB
// until the process exits.
constexpr size_t NEP_STATIC_SCRATCH_BYTES = 128 * 1024;
static __device__ __align__(256) unsigned char g_nep_static_scratch[NEP_STATIC_SCRATCH_BYTES];

// Same arguments and results as ai2b_nep_efv_f32 minus the workspace pair.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress with
//    that device current) and keeps it; make that first call outside any stream capture.
//  * Sizes whose scratch exceeds the array are refused with AI2B_ERR_WORKSPACE:
//    4 * (batch_size + 1) + 4 * ntypes^2 * (n_radial + n_angular) * (chebyshev_size <= 8 ? 8 : 16),
//    each term rounded up to 256 bytes, must fit in 128 KiB.
//  * No cudaMalloc / cudaFree or allocating library routine is called. Both scratch regions are
//    fully rewritten by every call before they are read, so nothing has to start at zero; the
//    array keeps the last call's contents in between.
//  * All calls on a device share the one array: two calls whose kernels overlap on the GPU
//    (different streams, no ordering between them) race on it. Order them, or use
//    ai2b_nep_efv_f32 with separate workspaces.
extern "C" int ai2b_nep_efv_static_scratch_f32(float *etot, float *force, float *virial, int cs, int n_r, int n_a, int l_max,
                                               int nneu, const float *coeffs, const float *w0, const float *b0, const float *w1,
                                               const float *bias, int B, int npad, const int *binum, const int *bilist,
                                               const int *numneigh, const int *firstneigh, const float *rcs, const int *types,
                                               int ntypes, int umax, int nghost, float rc_r, float rc_a, const float *qs,
                                               void *stream)
{
    constexpr int MAX_DEVICES = 64;
    static void *scratch_of_device[MAX_DEVICES] = {nullptr};
    AI2B_REQUIRE(etot && force && coeffs && w0 && b0 && w1 && bias && qs && binum && bilist && numneigh && firstneigh && rcs && types,
                 AI2B_ERR_INVALID, "ai2b_nep_efv_static_scratch_f32: NULL argument");
    AI2B_REQUIRE(B >= 0 && ntypes >= 1 && n_r >= 0 && n_a >= 0 && cs >= 1 && cs <= 16, AI2B_ERR_INVALID,
                 "ai2b_nep_efv_static_scratch_f32: bad sizes");
    const size_t need = nep_ws_bytes(B, ntypes, n_r, n_a, cs <= 8 ? 8 : 16, sizeof(float));
    AI2B_REQUIRE(need <= NEP_STATIC_SCRATCH_BYTES, AI2B_ERR_WORKSPACE,
                 "ai2b_nep_efv_static_scratch_f32: this batch/model needs %zu bytes of scratch, the built-in array holds %zu; "
                 "use ai2b_nep_efv_f32 with a caller-owned workspace",
                 need, NEP_STATIC_SCRATCH_BYTES);
    int dev = 0;
    AI2B_CUDA(cudaGetDevice(&dev));
    AI2B_REQUIRE(dev >= 0 && dev < MAX_DEVICES, AI2B_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    if (!scratch_of_device[dev]) {
        // in host code the array's name is only a handle: the kernels need its device address
        void *p = nullptr;
        AI2B_CUDA(cudaGetSymbolAddress(&p, g_nep_static_scratch));
        scratch_of_device[dev] = p;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (B > 0 && npad >= 0) {
        if (int rc = nep_zero_outputs<float>(etot, (size_t)B, force, 3 * (size_t)B * (npad + nghost), virial,
                                             virial ? 9 * (size_t)B : 0, st)) return rc;
    }
    NepArgs<float> A{etot, force, virial, nullptr, nullptr, w0, b0, w1, bias, qs, binum, bilist, numneigh,
                     firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, n_r, n_a, l_max, nneu,
                     0, 0, rc_r, rc_a};
    return virial ? launch_nep<float, NEP_EFV>(A, coeffs, scratch_of_device[dev], NEP_STATIC_SCRATCH_BYTES, st)
                  : launch_nep<float, NEP_EF>(A, coeffs, scratch_of_device[dev], NEP_STATIC_SCRATCH_BYTES, st);
}
