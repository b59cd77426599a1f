// NEP loss gradient for models with at most NMAX radial / angular functions, chebyshev_size <= 8:
// eight lanes per atom (four atoms per warp), as in nep_fast_kernel, because only a fifth of the
// neighbours are inside the angular cutoff. Same mathematics as nep_loss_backward_kernel
// (nep_loss.cuh). Included by nep_kernels.cu after nep_fast.cuh and nep_loss.cuh.
//   1  lanes = neighbours: radial descriptors q_n and their directional derivative u_n along the
//      per-pair loss weight p, per-type sums of f_xi and f'_xi (r^.p) (the radial coefficient
//      gradient factorises into these and two per-atom vectors); angular neighbours compacted
//   2  angular sums S and DS as a staged matrix product (lane s owns lm = 3s..3s+2)
//   3  descriptors, network with the second-order terms (four neurons per lane, weights in shared
//      memory), adjoints of q and u, polynomial coefficients x, y per (lm, mu)
//   4  angular part of the coefficient gradient per compacted neighbour, summed per neighbour type
// Every atom leaves a small record in shared memory (scaled q and u, the neuron factors, the
// per-type sums); after each round of sixteen atoms the whole block adds the records into its
// gradient accumulators, every accumulator element owned by one thread: the first-layer gradient
// and the radial coefficient gradient are outer products of two record vectors, so no atomics
// are needed. One structure per blockIdx.y; the block accumulators reach global memory once: when
// the blocks of a structure form one thread-block cluster (CLUSTER), block r sums slice r of all
// blocks' accumulators through distributed shared memory and stores it (the outputs need no
// zeroing and see no atomics); otherwise every block adds its accumulators atomically.
#pragma once
#include <cooperative_groups.h>

namespace ai2b {

template <typename T> __device__ __forceinline__ T nep_mulz(T g, T p) { return g * p; }
template <typename T> __device__ __forceinline__ T nep_mulz(NepZero, T) { return T(0); }
// gradient (gx, gy, gz) of a harmonic polynomial, some components identically zero, dotted with p
template <typename T, typename GX, typename GY, typename GZ>
__device__ __forceinline__ T nep_dot3(GX gx, GY gy, GZ gz, T px, T py, T pz)
{
    return nep_mulz<T>(gx, px) + nep_mulz<T>(gy, py) + nep_mulz<T>(gz, pz);
}

// staging row of the angular sums: g[NMAX] | g' (r^.p) [NMAX] | B_lm[24] | grad B_lm . p_perp / r [24] | pad
// (15 chunks of 16 bytes for NMAX = 4: eight lanes storing eight rows meet no bank twice)
template <int NMAX> struct NepLossFastDims { static constexpr int RS = 2 * NMAX + 2 * NEP_NLM + 4; };
// neighbours staged per step of the angular sums: half a group, which keeps a block's shared memory small enough for four blocks per SM
constexpr int NEPL_STAGE = 4;

template <int NMAX>
__host__ __device__ inline int nepl_fast_atom_elems(int nneu, int ntypes)
{
    const int NDP = NepFastDims<NMAX>::NDP;
    const int NP = nep_r32(nneu);
    const int sea = 2 * NEP_NLM * NMAX + 2 * NP;                 // xc, yc, th, sp ...
    const int stage = NEPL_STAGE * NepLossFastDims<NMAX>::RS;     // ... share their space with the staging rows
    return 4 * NDP + (sea > stage ? sea : stage) + nep_r4(2 * ntypes * 8) + ntypes * NMAX * 8 + NP;
}

template <typename T, bool VIRIAL, int NMAX, int MINB, bool CLUSTER>
__global__ void __launch_bounds__(NEP_WARPS * 32, MINB) nep_loss_fast_kernel(const NepArgs<T> A, const T *__restrict__ coeffs,
                                                                          const NepLossArgs<T> L)
{
    constexpr int CSP = 8;
    constexpr int NDP = NepFastDims<NMAX>::NDP;
    constexpr int RS = NepLossFastDims<NMAX>::RS;
    constexpr int TROW = 2 * NMAX * CSP;
    extern __shared__ __align__(16) unsigned char nepl_smem[];
    __shared__ T iqs[NDP];
    __shared__ T c3w_s[NEP_NLM];
    __shared__ unsigned char pm_mu[NDP], pm_l[NDP];
    __shared__ unsigned tmask[2][16];   // per round parity and type: the block's atom slots of that type
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane & (NEP_GROUP - 1), grp = lane / NEP_GROUP;
    const int slot_in_block = warp * NEP_APW + grp;
    const unsigned gmask_shift = grp * NEP_GROUP;
    const unsigned gmask = 0xffu << gmask_shift;
    const int b = blockIdx.y;
    const int nfun = A.n_r + A.n_a, nd = A.nd, nneu = A.nneu;
    const int NP = nep_r32(nneu), nrow = A.ntypes * NP;
    const int nlm = A.l_max * A.l_max + 2 * A.l_max;
    const int nq_a = A.l_max > 0 ? A.n_a * A.l_max : 0;
    const int ntab = A.ntypes * A.ntypes * TROW;
    // block: gradient accumulators, then the padded tables
    const size_t nco = (size_t)A.ntypes * A.ntypes * nfun * A.cs, nw0 = (size_t)A.ntypes * nneu * nd, nb0 = (size_t)A.ntypes * nneu;
    T *g_co = reinterpret_cast<T *>(nepl_smem);
    T *g_w0 = g_co + nco, *g_b0 = g_w0 + nw0, *g_w1 = g_b0 + nb0, *g_bi = g_w1 + nb0;
    const size_t nacc = nepl_block_elems(A.ntypes, nfun, A.cs, nneu, nd);
    T *ctab_s = g_co + ((nacc + 3) & ~size_t(3));
    T *W0s = ctab_s + nep_r4(ntab);          // [ntypes * NP][NDP]
    T *B0s = W0s + (size_t)nrow * NDP, *W1s = B0s + nrow;
    T *atoms_s = W1s + nrow;
    const int per_atom = nepl_fast_atom_elems<NMAX>(nneu, A.ntypes);
    T *q = atoms_s + (size_t)slot_in_block * per_atom;   // [NDP] each: q, u, av, be
    T *u = q + NDP, *av = u + NDP, *be = av + NDP;
    T *S = be + NDP;                                     // region shared with the staging rows
    T *stage = S;
    T *xc = S;                                           // [24][NMAX]   (written after the sums left the staging rows)
    T *yc = xc + NEP_NLM * NMAX;                         // [24][NMAX]
    T *th = yc + NEP_NLM * NMAX;                         // [NP] W1 d1     (placed after x, y; S / DS themselves stay in registers)
    T *sp = th + NP;                                     // [NP] W1 s d2
    const int sea = 2 * NEP_NLM * NMAX + 2 * NP, stg = NEPL_STAGE * RS;
    T *Fs = S + (sea > stg ? sea : stg);                 // [ntypes][8] sum f_xi, then [ntypes][8] sum f'_xi (r^.p)
    T *Ga = Fs + nep_r4(2 * A.ntypes * 8);               // [ntypes][NMAX][8] angular coefficient gradient of this atom
    T *gw1s = Ga + A.ntypes * NMAX * 8;                  // [NP] d/d w1 of this atom (d/d b0 is lam th + sp)
    const int off_th = (int)(th - q), off_sp = (int)(sp - q), off_fs = (int)(Fs - q), off_ga = (int)(Ga - q), off_gw1 = (int)(gw1s - q);
    unsigned short *alist = reinterpret_cast<unsigned short *>(atoms_s + (size_t)NEP_APB * per_atom) + (size_t)slot_in_block * A.umax;
    const int ntot_n = nfun;

    for (size_t i = threadIdx.x; i < nacc; i += blockDim.x) g_co[i] = T(0);
    {   // tables: one batch of independent loads, then stores
        T qsv = T(1);
        if ((int)threadIdx.x < nd) qsv = A.qs[threadIdx.x];
        const int n0 = nep_r4(ntab), n1 = n0 + nrow * NDP, n2 = n1 + nrow, nall = n2 + nrow;
        auto load = [&](int i) -> T {
            if (i < n0) {
                if (i >= ntab) return T(0);
                const int k = i % CSP, n = (i / CSP) % (2 * NMAX), pair = i / TROW;
                const int row = n < NMAX ? (n < A.n_r ? n : -1) : (n - NMAX < A.n_a ? A.n_r + n - NMAX : -1);
                return (k < A.cs && row >= 0) ? coeffs[((size_t)pair * ntot_n + row) * A.cs + k] : T(0);
            }
            if (i < n1) {
                const int row = (i - n0) / NDP, k = (i - n0) % NDP, t = row / NP, pn = row % NP;
                return (k < nd && pn < nneu) ? A.w0[((size_t)t * nneu + pn) * nd + k] : T(0);
            }
            const int row = i < n2 ? i - n1 : i - n2, t = row / NP, pn = row % NP;
            if (pn >= nneu) return T(0);
            return i < n2 ? A.b0[t * nneu + pn] : A.w1[t * nneu + pn];
        };
        constexpr int U = 24;
        for (int i0 = threadIdx.x; i0 < nall; i0 += U * blockDim.x) {
            T v[U];
#pragma unroll
            for (int k = 0; k < U; k++) { const int i = i0 + k * blockDim.x; v[k] = i < nall ? load(i) : T(0); }
#pragma unroll
            for (int k = 0; k < U; k++) { const int i = i0 + k * blockDim.x; if (i < nall) ctab_s[i] = v[k]; }
        }
        if (threadIdx.x < NDP) iqs[threadIdx.x] = (int)threadIdx.x < nd ? T(1) / qsv : T(0);
    }
    if (threadIdx.x < NEP_NLM) {
        const int lm = threadIdx.x;
        const bool m0 = lm == 0 || lm == 3 || lm == 8 || lm == 15;
        c3w_s[lm] = (m0 ? T(1) : T(2)) * (T)c_C3B[lm];
    }
    for (int p = threadIdx.x; p < NDP; p += blockDim.x) {
        const bool in = p < nq_a;
        pm_mu[p] = (unsigned char)(in ? p / A.l_max : 0);
        pm_l[p] = (unsigned char)(in ? p % A.l_max + 1 : 0);
    }
    if (threadIdx.x < 32) tmask[threadIdx.x >> 4][threadIdx.x & 15] = 0u;
    for (int i = threadIdx.x; i < NEP_APB * 4 * NDP; i += blockDim.x) atoms_s[(size_t)(i / (4 * NDP)) * per_atom + i % (4 * NDP)] = T(0);
    __syncthreads();

    const int n = A.binum[b];
    const int *types = A.types + (size_t)b * A.npad;
    const T *fm = L.f_ml + (size_t)b * A.npad * 3, *fd = L.f_dft + (size_t)b * A.npad * 3;
    const T lam = T(2) * L.ew / T(n) * (L.e_ml[b] - L.e_dft[b]), cf = T(2) * L.fw / T(3 * n), cv = VIRIAL ? T(2) * L.vw / T(9 * n) : T(0);
    T dV[9];
#pragma unroll
    for (int k = 0; k < 9; k++) dV[k] = VIRIAL ? L.v_ml[9 * b + k] - L.v_dft[9 * b + k] : T(0);

    const int ngroups = gridDim.x * NEP_APB;
    const int rounds = (n + ngroups - 1) / ngroups;
    for (int it = 0; it < rounds; it++) {
        const int ii = it * ngroups + blockIdx.x * NEP_APB + slot_in_block;
        const bool valid = ii < n;
        if (valid) {
            const size_t slot = (size_t)b * A.npad + ii;
            const int ci = A.bilist[slot];
            const int nn = min(A.numneigh[slot], A.umax);
            const int ti = types[ci];
            const int *fn = A.firstneigh + slot * A.umax;
            const T *rc = A.rcs + slot * A.umax * 3;
            const T *ctab = ctab_s + (size_t)ti * A.ntypes * TROW;
            const T Pi0 = cf * (fm[3 * ci] - fd[3 * ci]), Pi1 = cf * (fm[3 * ci + 1] - fd[3 * ci + 1]), Pi2 = cf * (fm[3 * ci + 2] - fd[3 * ci + 2]);
            // pair weight p = P_i - P_j - Qm r, its radial part vp = r^ . p and perpendicular part over r
            auto pair_weight = [&](int nj, T x, T y, T z, T rinv, T &vp, T &px, T &py, T &pz) {
                const T p0 = Pi0 - cf * (fm[3 * nj] - fd[3 * nj]) - cv * (dV[0] * x + dV[1] * y + dV[2] * z);
                const T p1 = Pi1 - cf * (fm[3 * nj + 1] - fd[3 * nj + 1]) - cv * (dV[3] * x + dV[4] * y + dV[5] * z);
                const T p2 = Pi2 - cf * (fm[3 * nj + 2] - fd[3 * nj + 2]) - cv * (dV[6] * x + dV[7] * y + dV[8] * z);
                const T ux = x * rinv, uy = y * rinv, uz = z * rinv;
                vp = ux * p0 + uy * p1 + uz * p2;
                px = (p0 - vp * ux) * rinv; py = (p1 - vp * uy) * rinv; pz = (p2 - vp * uz) * rinv;
            };
            for (int i = sub; i < 2 * A.ntypes * 8; i += NEP_GROUP) Fs[i] = T(0);
            for (int i = sub; i < A.ntypes * NMAX * 8; i += NEP_GROUP) Ga[i] = T(0);
            if (sub == 0) atomicOr(&tmask[it & 1][ti], 1u << slot_in_block);
            __syncwarp(gmask);

            // ---- 1. radial pass --------------------------------------------------------------------------
            T qacc[NMAX], uacc[NMAX];
#pragma unroll
            for (int k = 0; k < NMAX; k++) qacc[k] = uacc[k] = T(0);
            int nang = 0;
            for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {
                const int j = j0 + sub;
                bool on = j < nn;
                T x = 0, y = 0, z = 0;
                int nj = 0;
                if (on) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j]; }
                const T r = gsqrt(x * x + y * y + z * z);
                on = on && r <= A.rc_r && r > T(0);
                const int tj = on ? types[nj] : 0;
                const T rinv = on ? T(1) / r : T(0);
                T vp, px, py, pz;
                pair_weight(nj, x, y, z, rinv, vp, px, py, pz);
                T f[CSP], df[CSP];
                nep_radial<T, CSP>(on ? r : A.rc_r, A.rc_r, f, df);
                const T *crow = ctab + (size_t)tj * TROW;
#pragma unroll
                for (int k = 0; k < NMAX; k++) {
                    T c[CSP];
                    load_vec<T, CSP>(crow + k * CSP, c);
                    T g = T(0), dg = T(0);
#pragma unroll
                    for (int xi = 0; xi < CSP; xi++) { g = fma(c[xi], f[xi], g); dg = fma(c[xi], df[xi], dg); }
                    if (on) { qacc[k] += g; uacc[k] += dg * vp; }
                }
                // per-type sums of f_xi and f'_xi (r^.p): lane xi of the group ends up with entry xi
                for (int t = 0; t < A.ntypes; t++) {
                    const bool mine = on && tj == t;
                    if (__ballot_sync(gmask, mine) & gmask) {
                        T v[CSP], w[CSP];
#pragma unroll
                        for (int xi = 0; xi < CSP; xi++) { v[xi] = mine ? f[xi] : T(0); w[xi] = mine ? df[xi] * vp : T(0); }
                        Fs[t * 8 + sub] += group_xreduce8(v, sub, gmask);
                        Fs[(A.ntypes + t) * 8 + sub] += group_xreduce8(w, sub, gmask);
                    }
                }
                const bool ang = on && r <= A.rc_a && A.l_max > 0;
                const unsigned bal = (__ballot_sync(gmask, ang) >> gmask_shift) & 0xffu;
                if (ang) alist[nang + __popc(bal & ((1u << sub) - 1u))] = (unsigned short)(j | (tj << 10));
                nang += __popc(bal);
            }
#pragma unroll
            for (int k = 0; k < NMAX; k++) {
                const T sq = group_sum(qacc[k], gmask), su = group_sum(uacc[k], gmask);
                if (sub == (k & (NEP_GROUP - 1)) && k < A.n_r) { q[k] = sq; u[k] = su; }
            }
            __syncwarp(gmask);

            // ---- 2. angular sums and their directional derivatives: lane owns lm = 3 sub .. 3 sub + 2 ----------
            T Sacc[NMAX][3], Dacc[NMAX][3];
#pragma unroll
            for (int mu = 0; mu < NMAX; mu++)
#pragma unroll
                for (int i = 0; i < 3; i++) Sacc[mu][i] = Dacc[mu][i] = T(0);
            for (int k0 = 0; k0 < nang; k0 += NEPL_STAGE) {
                const bool on = sub < NEPL_STAGE && k0 + sub < nang;
                if (sub < NEPL_STAGE) {   // the first lanes of the group stage one neighbour each
                    T x = 0, y = 0, z = 0, rinv = 0, r = A.rc_a;
                    int tj = 0, nj = 0;
                    if (on) {
                        const int ent = alist[k0 + sub], j = ent & 1023;
                        tj = ent >> 10;
                        x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j];
                        r = gsqrt(x * x + y * y + z * z);
                        rinv = T(1) / r;
                    }
                    T vp, px, py, pz;
                    pair_weight(nj, x, y, z, rinv, vp, px, py, pz);
                    T f[CSP], df[CSP], row[RS];
                    nep_radial<T, CSP>(r, A.rc_a, f, df);
                    const T *crow = ctab + (size_t)tj * TROW + NMAX * CSP;
#pragma unroll
                    for (int mu = 0; mu < NMAX; mu++) {
                        T c[CSP];
                        load_vec<T, CSP>(crow + mu * CSP, c);
                        T g = T(0), dg = T(0);
#pragma unroll
                        for (int xi = 0; xi < CSP; xi++) { g = fma(c[xi], f[xi], g); dg = fma(c[xi], df[xi], dg); }
                        row[mu] = on ? g : T(0);
                        row[NMAX + mu] = on ? dg * vp : T(0);
                    }
                    {
                        const T x_ = x * rinv, y_ = y * rinv, z_ = z * rinv;
                        NEP_POLY_COMMON(x_, y_, z_)
#define NEP_X(k, val, gx, gy, gz)                                                               \
    row[2 * NMAX + k] = (val);                                                                  \
    row[2 * NMAX + NEP_NLM + k] = nep_dot3<T>(gx, gy, gz, px, py, pz);
                        NEP_FOR_EACH_LM(NEP_X, x_, y_, z_)
#undef NEP_X
                    }
                    store_vec<T, RS>(stage + sub * RS, row);
                }
                __syncwarp(gmask);
                const int cnt = min(NEPL_STAGE, nang - k0);
                for (int jj = 0; jj < cnt; jj++) {
                    const T *rj = stage + jj * RS;
                    T gj[NMAX], gv[NMAX];
                    load_vec<T, NMAX>(rj, gj);
                    load_vec<T, NMAX>(rj + NMAX, gv);
#pragma unroll
                    for (int i = 0; i < 3; i++) {
                        const T bv = rj[2 * NMAX + 3 * sub + i], gp = rj[2 * NMAX + NEP_NLM + 3 * sub + i];
#pragma unroll
                        for (int mu = 0; mu < NMAX; mu++) {
                            Sacc[mu][i] = fma(gj[mu], bv, Sacc[mu][i]);
                            Dacc[mu][i] = fma(gv[mu], bv, fma(gj[mu], gp, Dacc[mu][i]));
                        }
                    }
                }
                __syncwarp(gmask);
            }
            // descriptors q_{mu,l} and u_{mu,l}: partial sums over this lane's lm, combined per (mu, l) through shared memory
            // (the staging rows are free now): tq[mu][lm], tu[mu][lm]
            {
                T *tq = stage, *tu = stage + NMAX * NEP_NLM;
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++)
#pragma unroll
                    for (int i = 0; i < 3; i++) {
                        const int lm = 3 * sub + i;
                        tq[mu * NEP_NLM + lm] = c3w_s[lm] * Sacc[mu][i] * Sacc[mu][i];
                        tu[mu * NEP_NLM + lm] = T(2) * c3w_s[lm] * Sacc[mu][i] * Dacc[mu][i];
                    }
                __syncwarp(gmask);
                for (int p = sub; p < nq_a; p += NEP_GROUP) {
                    const int mu = pm_mu[p], l = pm_l[p];
                    T aq = T(0), au = T(0);
                    for (int mp = 0; mp < 2 * l + 1; mp++) { aq += tq[mu * NEP_NLM + l * l - 1 + mp]; au += tu[mu * NEP_NLM + l * l - 1 + mp]; }
                    q[A.n_r + p] = aq; u[A.n_r + p] = au;
                }
                __syncwarp(gmask);
            }

            // ---- 3. network with second-order terms --------------------------------------------------------------
            // q, u become q / qs, u / qs (what the first layer sees and what its weight gradient needs)
            for (int k = sub; k < nd; k += NEP_GROUP) { q[k] *= iqs[k]; u[k] *= iqs[k]; }
            __syncwarp(gmask);
            const T *W0t = W0s + (size_t)ti * NP * NDP;
            for (int p0 = 0; p0 < NP; p0 += 4 * NEP_GROUP) {
                T h[4], sv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) h[i] = sv[i] = T(0);
#pragma unroll
                for (int c = 0; c < NDP / 4; c++) {
                    T eq[4], eu[4];
                    load_vec<T, 4>(q + 4 * c, eq);
                    load_vec<T, 4>(u + 4 * c, eu);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        T w[4];
                        load_vec<T, 4>(W0t + (size_t)(p0 + sub + NEP_GROUP * i) * NDP + 4 * c, w);
#pragma unroll
                        for (int k = 0; k < 4; k++) { h[i] = fma(w[k], eq[k], h[i]); sv[i] = fma(w[k], eu[k], sv[i]); }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int pn = p0 + sub + NEP_GROUP * i;
                    const T w1 = W1s[ti * NP + pn];
                    const T t = gtanh(h[i] + B0s[ti * NP + pn]), d1 = T(1) - t * t, d2 = T(-2) * t * d1;
                    th[pn] = w1 * d1;                                  // zero for the padding neurons (w1 = 0)
                    sp[pn] = w1 * sv[i] * d2;
                    gw1s[pn] = lam * t + d1 * sv[i];
                }
            }
            __syncwarp(gmask);
            // adjoints: av = dE/dq, be = coefficient of dq/dc  (overwrite the scaled copies)
            for (int c = sub; c < NDP / 4; c += NEP_GROUP) {
                const T *wcol = W0t + 4 * c;
                T a0[4] = {T(0), T(0), T(0), T(0)}, b0v[4] = {T(0), T(0), T(0), T(0)};
                for (int pn = 0; pn < NP; pn += 4) {
                    T xt[4], xs[4];
                    load_vec<T, 4>(th + pn, xt);
                    load_vec<T, 4>(sp + pn, xs);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        T w[4];
                        load_vec<T, 4>(wcol + (size_t)(pn + i) * NDP, w);
#pragma unroll
                        for (int k = 0; k < 4; k++) { a0[k] = fma(xt[i], w[k], a0[k]); b0v[k] = fma(xs[i], w[k], b0v[k]); }
                    }
                }
                T ra[4], rb[4];
#pragma unroll
                for (int k = 0; k < 4; k++) { ra[k] = a0[k] * iqs[4 * c + k]; rb[k] = lam * ra[k] + b0v[k] * iqs[4 * c + k]; }
                store_vec<T, 4>(av + 4 * c, ra);
                store_vec<T, 4>(be + 4 * c, rb);
            }
            __syncwarp(gmask);
            // polynomial coefficients per (lm, mu): x = w2c (be S + av DS), y = w2c av S
#pragma unroll
            for (int i = 0; i < 3; i++) {
                const int lm = 3 * sub + i;
                const int l = lm >= 15 ? 4 : lm >= 8 ? 3 : lm >= 3 ? 2 : 1;
                const T w2c = T(2) * c3w_s[lm];
                T xr[NMAX], yr[NMAX];
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++) {
                    const bool in = lm < nlm && mu < A.n_a;
                    const int k = A.n_r + mu * A.l_max + l - 1;
                    const T ak = in ? av[k] : T(0), bk = in ? be[k] : T(0);
                    xr[mu] = w2c * (bk * Sacc[mu][i] + ak * Dacc[mu][i]);
                    yr[mu] = w2c * ak * Sacc[mu][i];
                }
                store_vec<T, NMAX>(xc + lm * NMAX, xr);
                store_vec<T, NMAX>(yc + lm * NMAX, yr);
            }
            __syncwarp(gmask);

            // ---- 4. coefficient gradient, angular functions (the radial part is an outer product: see the round's end) ----
            for (int k0 = 0; k0 < nang; k0 += NEP_GROUP) {
                const bool on = k0 + sub < nang;
                int tj = 0;
                T vp = T(0), f[CSP], df[CSP];
                T X[NMAX], Y[NMAX], GY[NMAX];
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++) X[mu] = Y[mu] = GY[mu] = T(0);
                {
                    T x = 0, y = 0, z = 0, rinv = 0, r = A.rc_a;
                    int nj = 0;
                    if (on) {
                        const int ent = alist[k0 + sub], j = ent & 1023;
                        tj = ent >> 10;
                        x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j];
                        r = gsqrt(x * x + y * y + z * z);
                        rinv = T(1) / r;
                    }
                    T px, py, pz;
                    pair_weight(nj, x, y, z, rinv, vp, px, py, pz);
                    const T x_ = x * rinv, y_ = y * rinv, z_ = z * rinv;
                    NEP_POLY_COMMON(x_, y_, z_)
#define NEP_X(k, val, gx, gy, gz)                                                               \
    {                                                                                           \
        T xe[NMAX], ye[NMAX];                                                                   \
        load_vec<T, NMAX>(xc + (k) * NMAX, xe);                                                 \
        load_vec<T, NMAX>(yc + (k) * NMAX, ye);                                                 \
        const T bv = (val), gp = nep_dot3<T>(gx, gy, gz, px, py, pz);                           \
        nep_acc<T, NMAX>(xe, bv, X);                                                            \
        nep_acc<T, NMAX>(ye, bv, Y);                                                            \
        nep_acc<T, NMAX>(ye, gp, GY);                                                           \
    }
                    NEP_FOR_EACH_LM(NEP_X, x_, y_, z_)
#undef NEP_X
                    nep_radial<T, CSP>(r, A.rc_a, f, df);
                }
                // sum over the group's neighbours of each type; lane xi adds entry xi to the atom's record
                for (int t = 0; t < A.ntypes; t++) {
                    const bool mine = on && tj == t;
                    if (__ballot_sync(gmask, mine) & gmask) {
#pragma unroll
                        for (int mu = 0; mu < NMAX; mu++) {
                            const T wv = X[mu] + GY[mu], wd = Y[mu] * vp;
                            T v[CSP];
#pragma unroll
                            for (int xi = 0; xi < CSP; xi++) v[xi] = mine ? wv * f[xi] + wd * df[xi] : T(0);
                            const T tot = group_xreduce8(v, sub, gmask);
                            Ga[(t * NMAX + mu) * 8 + sub] += tot;
                        }
                    }
                }
            }
            __syncwarp(gmask);
        }
        // ---- end of the round: the block adds its atoms' records to the accumulators; one owner per element ----
        __syncthreads();
        const unsigned *tm = tmask[it & 1];
        constexpr int NC = NDP / 4;
        for (int x = threadIdx.x; x < A.ntypes * nneu * NC; x += blockDim.x) {   // first layer: gb0 (x) q + th (x) u
            const int kc = x % NC, pn = (x / NC) % nneu, t = x / (NC * nneu);
            T acc[4] = {T(0), T(0), T(0), T(0)};
            for (unsigned m = tm[t]; m; m &= m - 1) {
                const T *rec = atoms_s + (size_t)(__ffs(m) - 1) * per_atom;
                const T tw = rec[off_th + pn], gb = lam * tw + rec[off_sp + pn];   // d/d b0 of that atom
                T eq[4], eu[4];
                load_vec<T, 4>(rec + 4 * kc, eq);
                load_vec<T, 4>(rec + NDP + 4 * kc, eu);
#pragma unroll
                for (int k = 0; k < 4; k++) acc[k] = fma(gb, eq[k], fma(tw, eu[k], acc[k]));
            }
            T *gw = g_w0 + ((size_t)t * nneu + pn) * nd + 4 * kc;
#pragma unroll
            for (int k = 0; k < 4; k++) if (4 * kc + k < nd) gw[k] += acc[k];
        }
        for (int x = threadIdx.x; x < A.ntypes * nneu; x += blockDim.x) {
            const int pn = x % nneu, t = x / nneu;
            T a0 = T(0), a1 = T(0);
            for (unsigned m = tm[t]; m; m &= m - 1) {
                const T *rec = atoms_s + (size_t)(__ffs(m) - 1) * per_atom;
                a0 += lam * rec[off_th + pn] + rec[off_sp + pn]; a1 += rec[off_gw1 + pn];
            }
            g_b0[x] += a0; g_w1[x] += a1;
        }
        for (int x = threadIdx.x; x < A.ntypes * A.ntypes * nfun * A.cs; x += blockDim.x) {   // coefficients
            const int xi = x % A.cs, fidx = (x / A.cs) % nfun, tj = (x / (A.cs * nfun)) % A.ntypes, t = x / (A.cs * nfun * A.ntypes);
            T acc = T(0);
            if (fidx < A.n_r) {   // radial: be_n sum_j f_xi + av_n sum_j f'_xi (r^.p), sums per neighbour type
                for (unsigned m = tm[t]; m; m &= m - 1) {
                    const T *rec = atoms_s + (size_t)(__ffs(m) - 1) * per_atom;
                    acc = fma(rec[3 * NDP + fidx], rec[off_fs + tj * 8 + xi], fma(rec[2 * NDP + fidx], rec[off_fs + (A.ntypes + tj) * 8 + xi], acc));
                }
            } else {
                for (unsigned m = tm[t]; m; m &= m - 1)
                    acc += atoms_s[(size_t)(__ffs(m) - 1) * per_atom + off_ga + (tj * NMAX + fidx - A.n_r) * 8 + xi];
            }
            g_co[x] += acc;
        }
        if ((int)threadIdx.x < A.ntypes) g_bi[threadIdx.x] += lam * T(__popc(tm[threadIdx.x]));
        if (threadIdx.x < 16) tmask[(it + 1) & 1][threadIdx.x] = 0u;
        __syncthreads();
    }
    if constexpr (CLUSTER) {
        namespace cg = cooperative_groups;
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();   // every block of the structure has finished its accumulators
        const unsigned nblk = cl.num_blocks(), rank = cl.block_rank();
        const size_t per = (nacc + nblk - 1) / nblk, i0 = rank * per, i1 = i0 + per < nacc ? i0 + per : nacc;
        for (size_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
            T sum = T(0);
            for (unsigned c = 0; c < nblk; c++) sum += cl.map_shared_rank(g_co, c)[i];
            T *dst = i < nco ? L.dco + b * nco + i
                   : i < nco + nw0 ? L.dw0 + b * nw0 + (i - nco)
                   : i < nco + nw0 + nb0 ? L.db0 + b * nb0 + (i - nco - nw0)
                   : i < nco + nw0 + 2 * nb0 ? L.dw1 + b * nb0 + (i - nco - nw0 - nb0)
                   : L.dbi + (size_t)b * A.ntypes + (i - nco - nw0 - 2 * nb0);
            *dst = sum;
        }
        cl.sync();   // no block leaves while its shared memory is still being read
    } else {
        __syncthreads();
        for (size_t i = threadIdx.x; i < nco; i += blockDim.x) if (g_co[i] != T(0)) atomicAdd(L.dco + b * nco + i, g_co[i]);
        for (size_t i = threadIdx.x; i < nw0; i += blockDim.x) if (g_w0[i] != T(0)) atomicAdd(L.dw0 + b * nw0 + i, g_w0[i]);
        for (size_t i = threadIdx.x; i < nb0; i += blockDim.x) {
            if (g_b0[i] != T(0)) atomicAdd(L.db0 + b * nb0 + i, g_b0[i]);
            if (g_w1[i] != T(0)) atomicAdd(L.dw1 + b * nb0 + i, g_w1[i]);
        }
        for (int i = threadIdx.x; i < A.ntypes; i += blockDim.x) if (g_bi[i] != T(0)) atomicAdd(L.dbi + (size_t)b * A.ntypes + i, g_bi[i]);
    }
}

// *done = false: the model does not fit this kernel's plan (the general kernel then runs)
template <typename T, int NMAX>
static int launch_nep_loss_fast(const NepArgs<T> &A, const T *coeffs, const NepLossArgs<T> &L, cudaStream_t st, bool *done)
{
    *done = false;
    if (A.cs > 8 || A.n_r > NMAX || A.n_a > NMAX || A.ntypes > 16 || A.umax > 1024 || A.nneu > 256) return AI2B_OK;
    const int nfun = A.n_r + A.n_a;
    constexpr int NDP = NepFastDims<NMAX>::NDP;
    const int NP = nep_r32(A.nneu), nrow = A.ntypes * NP;
    const size_t nacc = (nepl_block_elems(A.ntypes, nfun, A.cs, A.nneu, A.nd) + 3) & ~size_t(3);
    const size_t elems = nacc + nep_r4(A.ntypes * A.ntypes * 2 * NMAX * 8) + (size_t)nrow * (NDP + 2) +
                         (size_t)NEP_APB * nepl_fast_atom_elems<NMAX>(A.nneu, A.ntypes);
    const size_t smem = elems * sizeof(T) + (size_t)NEP_APB * A.umax * sizeof(unsigned short) + 16;
    if (smem > 200 * 1024) return AI2B_OK;
    constexpr int MINB = sizeof(T) == 4 ? 4 : 2;
    const bool vir = L.v_ml != nullptr;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long bx = ((long)A.npad + NEP_APB - 1) / NEP_APB;
    const long cap = std::max(1L, (long)sms * std::min<long>(MINB, (long)(227 * 1024 / (smem + 1024))) / A.B);
    if (bx > cap) bx = cap;
    // portable cluster size 8: the blocks of a structure reduce among themselves; up to a third fewer blocks than
    // the occupancy asks for are traded for that
    if (bx > 8 && bx <= 12) bx = 8;
    const bool cluster = bx <= 8;
    bool use_cluster = false;
    auto run = [&](auto kern) -> int {
        AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)bx, (unsigned)A.B);
        cfg.blockDim = dim3(NEP_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)bx;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_cluster ? 1 : 0;
        AI2B_CUDA(cudaLaunchKernelEx(&cfg, kern, A, coeffs, L));
        return AI2B_OK;
    };
    // a cluster shape that the device cannot place falls back to the atomic path
    auto placeable = [&](auto kern) -> bool {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return false; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)bx, (unsigned)A.B);
        cfg.blockDim = dim3(NEP_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)bx;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int nclusters = 0;
        if (cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
        return nclusters > 0;
    };
    use_cluster = cluster && (vir ? placeable(nep_loss_fast_kernel<T, true, NMAX, MINB, true>)
                                             : placeable(nep_loss_fast_kernel<T, false, NMAX, MINB, true>));
    int rc;
    if (use_cluster) {
        rc = vir ? run(nep_loss_fast_kernel<T, true, NMAX, MINB, true>) : run(nep_loss_fast_kernel<T, false, NMAX, MINB, true>);
    } else {
        rc = nepl_zero_outputs(A, L, st);
        if (rc == AI2B_OK)
            rc = vir ? run(nep_loss_fast_kernel<T, true, NMAX, MINB, false>) : run(nep_loss_fast_kernel<T, false, NMAX, MINB, false>);
    }
    if (rc == AI2B_OK) *done = true;
    return rc;
}

}  // namespace ai2b
