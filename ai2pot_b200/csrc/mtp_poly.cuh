// Device building blocks shared by the linear-MTP kernels: radial functions, and evaluation of
// the per-mu moment polynomials with compile-time exponents.
//
// With u = r_vec / r, a basic moment (mu, ax, ay, az) of the reference
// (source/descriptor/mtpr/include/mtpBasis.h:472-519: coefficient * Q(r) * scaling * x^ax y^ay z^az / r^k)
// is  sum_j f_mu(r_j) * ux^ax uy^ay uz^az  with  f_mu(r) = scaling * sum_xi c[ti,tj,mu,xi] Q_xi(r).
// All monomials of degree <= kmu[mu] are enumerated in a fixed canonical order, so the moment
// sums (forward) and the adjoint-weighted polynomial and its gradient (force pass) are straight-
// line code over registers.
#pragma once
#include "mtp_program.cuh"

namespace ai2b {

template <typename T> struct Vec2;
template <> struct Vec2<double> { using type = double2; };
template <> struct Vec2<float> { using type = float2; };

// Q_xi = s(r) T_xi(u), Q'_xi = s' T_xi + s T'_xi  (source/descriptor/mtpr/include/basis.h:155-181,
// 352-380, 621-637), scaled by `scaling`. CSP >= chebyshev_size entries are produced; the ones
// past chebyshev_size meet zero coefficients (the coefficient rows are zero-padded to CSP).
// (inv = 1 / (rmax - rmin): the same for every pair of a call, so callers in a pair loop pass it in)
template <typename T, int CSP>
__device__ __forceinline__ void mtp_radial_basis(T r, T rmax, T rmin, T scaling, T (&q)[CSP], T (&dq)[CSP], T inv)
{
    const T w = (r - rmin) * inv;
    T s = T(0), ds = T(0);
    if (r >= rmin && r < rmax) {
        const T w2 = w * w;
        s = w2 * w * (T(-6) * w2 + T(15) * w - T(10)) + T(1);
        ds = inv * (T(-30) * w2 * w2 + T(60) * w2 * w - T(30) * w2);
    }
    s *= scaling; ds *= scaling;
    const T u = (T(2) * r - (rmax + rmin)) * inv;
    const T uc = T(2) * inv;
    T t0 = T(1), t1 = u, d0 = T(0), d1 = T(1);
#pragma unroll
    for (int xi = 0; xi < CSP; xi++) {
        T t, d;
        if (xi == 0) { t = T(1); d = T(0); }
        else if (xi == 1) { t = u; d = T(1); }
        else {
            t = T(2) * u * t1 - t0;
            d = T(2) * t1 + T(2) * u * d1 - d0;
            t0 = t1; t1 = t; d0 = d1; d1 = d;
        }
        q[xi] = s * t;
        dq[xi] = ds * t + s * (d * uc);
    }
}

template <typename T, int CSP>
__device__ __forceinline__ void mtp_radial_basis(T r, T rmax, T rmin, T scaling, T (&q)[CSP], T (&dq)[CSP])
{
    mtp_radial_basis<T, CSP>(r, rmax, rmin, scaling, q, dq, T(1) / (rmax - rmin));
}

template <typename T, int KD>
struct Powers {
    T x[KD + 1], y[KD + 1], z[KD + 1];
    // u^k = u^(k/2) * u^(k - k/2): the longest chain of dependent products has log2(KD) + 1 links instead of KD
    __device__ __forceinline__ void set(T ux, T uy, T uz)
    {
        x[0] = y[0] = z[0] = T(1);
        if constexpr (KD >= 1) { x[1] = ux; y[1] = uy; z[1] = uz; }
#pragma unroll
        for (int k = 2; k <= KD; k++) {
            x[k] = x[k / 2] * x[k - k / 2];
            y[k] = y[k / 2] * y[k - k / 2];
            z[k] = z[k / 2] * z[k - k / 2];
        }
    }
};

template <typename T, int KD, int D, int Q>
__device__ __forceinline__ T mono(const Powers<T, KD> &p)
{
    constexpr Exp3 e = deg_exp(D, Q);
    if constexpr (e.y == 0 && e.z == 0) return p.x[e.x];
    else if constexpr (e.x == 0 && e.z == 0) return p.y[e.y];
    else if constexpr (e.x == 0 && e.y == 0) return p.z[e.z];
    else if constexpr (e.z == 0) return p.x[e.x] * p.y[e.y];
    else if constexpr (e.y == 0) return p.x[e.x] * p.z[e.z];
    else if constexpr (e.x == 0) return p.y[e.y] * p.z[e.z];
    else return p.x[e.x] * p.y[e.y] * p.z[e.z];
}

// Forward: acc[q] += sum over lanes of f * mono_q for the ndeg(D) monomials of degree D.
// `acc` points at this degree's slice of the warp's dense moment array in shared memory.
template <typename T, int KD, int D>
__device__ __forceinline__ void fwd_degree(T f, const Powers<T, KD> &p, T *acc, int lane)
{
    constexpr int ND = ndeg(D);
    constexpr int GS = 16;   // values reduced together: 16 keeps the staging array at 32 registers (fp64)
    static_for<0, (ND + GS - 1) / GS>([&](auto g) {
        constexpr int G = decltype(g)::value;
        constexpr int CNT = (ND - GS * G) < GS ? (ND - GS * G) : GS;
        constexpr int N = pow2ceil(CNT);
        T v[N];
        static_for<0, N>([&](auto i) {
            constexpr int I = decltype(i)::value;
            if constexpr (I < CNT) v[I] = f * mono<T, KD, D, GS * G + I>(p);
            else v[I] = T(0);
        });
        const T r = warp_xreduce<T, N>(v, lane);
        constexpr int SH = 5 - ilog2(N);
        const int idx = lane >> SH;
        if ((lane & ((1 << SH) - 1)) == 0 && idx < CNT) acc[GS * G + idx] += r;
    });
}

template <typename T, int KD>
__device__ __forceinline__ void fwd_mu(int kmu, T f, const Powers<T, KD> &p, T *acc, int lane)
{
#define AI2B_FWD_DEG(D)                                                  \
    if constexpr (D <= KD) {                                             \
        if (kmu < D) return;                                             \
        fwd_degree<T, KD, D>(f, p, acc + ncan(D - 1), lane);             \
    }
    AI2B_FWD_DEG(0) AI2B_FWD_DEG(1) AI2B_FWD_DEG(2) AI2B_FWD_DEG(3) AI2B_FWD_DEG(4)
    AI2B_FWD_DEG(5) AI2B_FWD_DEG(6) AI2B_FWD_DEG(7) AI2B_FWD_DEG(8)
#undef AI2B_FWD_DEG
}

// Polynomial evaluation for one neighbour: with coefficient quadruples e4[q] = {e, cx, cy, cz}
// per monomial (cx = (ax+1) * e of the monomial with one more power of ux, ...):
//   P += sum e mono,  G{x,y,z} += sum c{x,y,z} mono   (G = gradient of the polynomial w.r.t. u)
// Every lane reads the same addresses (shared-memory broadcast). GRAD = false for the top
// degree of a mu, whose gradient coefficients are zero.
template <typename T, int KD, int D, bool GRAD>
__device__ __forceinline__ void eval_degree(const T *__restrict__ e4, const Powers<T, KD> &p, T &P, T &Gx, T &Gy, T &Gz)
{
    using V2 = typename Vec2<T>::type;
    static_for<0, ndeg(D)>([&](auto qq) {
        constexpr int Q = decltype(qq)::value;
        const T m = mono<T, KD, D, Q>(p);
        if constexpr (GRAD) {
            const V2 a = *reinterpret_cast<const V2 *>(e4 + 4 * Q);
            const V2 b = *reinterpret_cast<const V2 *>(e4 + 4 * Q + 2);
            P = fma(a.x, m, P);
            Gx = fma(a.y, m, Gx);
            Gy = fma(b.x, m, Gy);
            Gz = fma(b.y, m, Gz);
        } else {
            P = fma(e4[4 * Q], m, P);
        }
    });
}

template <typename T, int KD>
__device__ __forceinline__ void eval_mu(int kmu, const T *__restrict__ e4, const Powers<T, KD> &p, T &P, T &Gx, T &Gy, T &Gz)
{
#define AI2B_EVAL_DEG(D)                                                                         \
    if constexpr (D < KD) {                                                                      \
        if (kmu > D) eval_degree<T, KD, D, true>(e4 + 4 * ncan(D - 1), p, P, Gx, Gy, Gz);        \
        else { eval_degree<T, KD, D, false>(e4 + 4 * ncan(D - 1), p, P, Gx, Gy, Gz); return; }   \
    } else if constexpr (D == KD) {                                                              \
        eval_degree<T, KD, D, false>(e4 + 4 * ncan(D - 1), p, P, Gx, Gy, Gz);                    \
        return;                                                                                  \
    }
    AI2B_EVAL_DEG(0) AI2B_EVAL_DEG(1) AI2B_EVAL_DEG(2) AI2B_EVAL_DEG(3) AI2B_EVAL_DEG(4)
    AI2B_EVAL_DEG(5) AI2B_EVAL_DEG(6) AI2B_EVAL_DEG(7) AI2B_EVAL_DEG(8)
#undef AI2B_EVAL_DEG
}

}  // namespace ai2b
