// NEP energy / force / virial kernel specialised for models with at most NMAX radial and NMAX
// angular functions (NMAX = 4 covers the reference's defaults, ai2pot/models/nep/nep.py:36-40).
// Included by nep_kernels.cu after the shared helpers (NepArgs, nep_radial, NEP_FOR_EACH_LM).
//
// Same mapping as the general kernel (eight lanes per centre atom, lanes = neighbours) and the
// same math (nep.h:320-529), with the per-atom instruction count cut about in half:
//   * the coefficient table [ti][tj][2 NMAX][CSP] is zero-padded into shared memory by the block
//     itself (no separate padding launch) and read with 16-byte loads;
//   * radial pass: q_n accumulate in registers over the neighbour chunks, one group reduction at
//     the end; the contracted derivatives g'_n(r_j) are kept per neighbour in shared memory, so
//     the radial force pass does not rebuild the basis;
//   * angular sums S[mu][lm] = sum_j g_mu(j) B_lm(j): the lanes stage g and B_lm of their
//     neighbour in shared memory and lane s accumulates the 3 NMAX sums lm = 3s..3s+2 for every
//     mu (a small matrix product) instead of 3 NMAX eight-lane transpose-reductions;
//   * angular force pass: the harmonic polynomials and their gradients are consumed one lm at a
//     time against the adjoints of all mu (4 NMAX accumulators), never held as 96 registers;
//   * structures' atom offsets are read from the workspace only for batches of more than one
//     structure.
#pragma once

namespace ai2b {

template <typename T, int N>
__device__ __forceinline__ void load_vec(const T *__restrict__ p, T (&v)[N])
{
    constexpr int PER = 16 / (int)sizeof(T);
    static_assert(N % PER == 0, "row length must be a multiple of 16 bytes");
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < N / 4; i++) {
            const float4 t = reinterpret_cast<const float4 *>(p)[i];
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N / 2; i++) {
            const double2 t = reinterpret_cast<const double2 *>(p)[i];
            v[2 * i] = t.x; v[2 * i + 1] = t.y;
        }
    }
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T *__restrict__ p, const T (&v)[N])
{
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < N / 4; i++)
            reinterpret_cast<float4 *>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < N / 2; i++) reinterpret_cast<double2 *>(p)[i] = make_double2(v[2 * i], v[2 * i + 1]);
    }
}

// shared-memory elements (of T) per atom slot of the specialised kernel
template <int NMAX>
__host__ __device__ inline int nep_fast_atom_elems(int nd, int nneu, int umax, bool cache)
{
    auto r4 = [](int n) { return (n + 3) & ~3; };
    const int sea = 2 * NEP_NLM * NMAX + r4(nneu);            // S, ES, act ...
    const int stage = NEP_GROUP * (NMAX + NEP_NLM);           // ... share their space with the staging rows
    return 2 * r4(nd) + (sea > stage ? sea : stage) + (cache ? umax * NMAX : 0);
}

template <typename T, int CSP, int MODE, int NMAX, int MINB>
__global__ void __launch_bounds__(NEP_WARPS * 32, MINB) nep_fast_kernel(const NepArgs<T> A, const T *__restrict__ coeffs)
{
    constexpr int RS = NMAX + NEP_NLM;     // staging row: g[NMAX] | B_lm[24]
    constexpr int TROW = 2 * NMAX * CSP;   // coefficient rows of one (ti,tj) pair
    constexpr bool CACHE = MODE != NEP_DESC;
    extern __shared__ __align__(16) unsigned char nep_smem[];
    __shared__ T blk_acc[10];
    __shared__ int blk_b;
    __shared__ T iqs[96];
    __shared__ T fac_s[NEP_NLM];   // (2 - delta_m0) * 2 * C_lm
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane & (NEP_GROUP - 1), grp = lane / NEP_GROUP;
    const int slot_in_block = warp * NEP_APW + grp;
    const unsigned gmask_shift = grp * NEP_GROUP;
    const unsigned gmask = 0xffu << gmask_shift;
    auto r4 = [](int n) { return (n + 3) & ~3; };
    const int per_atom = nep_fast_atom_elems<NMAX>(A.nd, A.nneu, A.umax, CACHE);
    const int ntab = A.ntypes * A.ntypes * TROW;
    T *ctab_s = reinterpret_cast<T *>(nep_smem);
    T *q = ctab_s + r4(ntab) + (size_t)slot_in_block * per_atom;
    T *Eq = q + r4(A.nd);
    T *S = Eq + r4(A.nd);                  // [NMAX][24]
    T *ES = S + NEP_NLM * NMAX;            // [24][NMAX]
    T *act = ES + NEP_NLM * NMAX;
    T *stage = S;                          // staging rows of the angular sums (before S, ES, act are written)
    const int sea = 2 * NEP_NLM * NMAX + r4(A.nneu), stg = NEP_GROUP * RS;
    T *dcache = S + (sea > stg ? sea : stg);   // [umax][NMAX]: g'_n of every neighbour
    unsigned short *alist = reinterpret_cast<unsigned short *>(ctab_s + r4(ntab) + (size_t)NEP_APB * per_atom) +
                            (size_t)slot_in_block * A.umax;
    const int ntot_n = A.n_r + A.n_a;
    const int nlm = A.l_max * A.l_max + 2 * A.l_max;

    // block prologue: zero-padded coefficient table, 1/q_scaler, 3-body factors
    for (int i = threadIdx.x; i < ntab; i += blockDim.x) {
        const int k = i % CSP, n = (i / CSP) % (2 * NMAX), pair = i / TROW;
        T v = T(0);
        if (k < A.cs) {
            if (n < NMAX) {
                if (n < A.n_r) v = coeffs[((size_t)pair * ntot_n + n) * A.cs + k];
            } else if (n - NMAX < A.n_a) {
                v = coeffs[((size_t)pair * ntot_n + A.n_r + (n - NMAX)) * A.cs + k];
            }
        }
        ctab_s[i] = v;
    }
    if (threadIdx.x < NEP_NLM) {
        const int lm = threadIdx.x;
        const bool m0 = lm == 0 || lm == 3 || lm == 8 || lm == 15;
        fac_s[lm] = (m0 ? T(1) : T(2)) * T(2) * (T)c_C3B[lm];
    }
    if (MODE != NEP_DESC)
        for (int k = threadIdx.x; k < A.nd; k += blockDim.x) iqs[k] = T(1) / A.qs[k];
    __syncthreads();

    const int ntot = A.B == 1 ? A.binum[0] : A.prefix[A.B];
    const int ngroups = gridDim.x * NEP_APB;
    const int gidx = blockIdx.x * NEP_APB + slot_in_block;
    const int rounds = (ntot + ngroups - 1) / ngroups;

    for (int it = 0; it < rounds; it++) {
        const int t = it * ngroups + gidx;
        const bool valid = t < ntot;
        int b = 0;
        if (valid && A.B > 1) {
            int lo = 0, hi = A.B;
            while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (A.prefix[mid] <= t) lo = mid; else hi = mid; }
            b = lo;
        }
        const int ii = valid ? (A.B > 1 ? t - A.prefix[b] : t) : 0;
        const size_t slot = (size_t)b * A.npad + ii;
        const int ci = valid ? A.bilist[slot] : 0;
        const int nn = valid ? min(A.numneigh[slot], A.umax) : 0;
        const int *types = A.types + (size_t)b * (A.npad + (MODE == NEP_DESC ? 0 : A.nghost));
        const int ti = valid ? types[ci] : 0;
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;
        const T *ctab = ctab_s + (size_t)ti * A.ntypes * TROW;

        if (MODE != NEP_DESC) {
            if (threadIdx.x == 0) blk_b = valid ? b : -1;
            if (threadIdx.x < 10) blk_acc[threadIdx.x] = T(0);
            __syncthreads();
        }

        // ---- 1. radial pass: q_n, cached g'_n, compaction of the angular neighbours ----------------
        T qacc[NMAX];
#pragma unroll
        for (int n = 0; n < NMAX; n++) qacc[n] = T(0);
        int nang = 0;
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {
            const int j = j0 + sub;
            bool on = j < nn;
            T x = 0, y = 0, z = 0;
            int tj = 0;
            if (on) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; tj = types[fn[j]]; }
            const T r = gsqrt(x * x + y * y + z * z);
            on = on && r <= A.rc_r && r > T(0);
            T f[CSP], df[CSP];
            nep_radial<T, CSP>(on ? r : A.rc_r, A.rc_r, f, df);
            const T *crow = ctab + (size_t)tj * TROW;
            T dgv[NMAX];
#pragma unroll
            for (int n = 0; n < NMAX; n++) {
                T c[CSP];
                load_vec<T, CSP>(crow + n * CSP, c);
                T g = T(0), dg = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k++) {
                    g = fma(c[k], f[k], g);
                    if (CACHE) dg = fma(c[k], df[k], dg);
                }
                qacc[n] += on ? g : T(0);
                dgv[n] = on ? dg : T(0);
            }
            if (CACHE && j < A.umax) store_vec<T, NMAX>(dcache + (size_t)j * NMAX, dgv);
            const bool ang = on && r <= A.rc_a && A.l_max > 0;
            const unsigned bal = (__ballot_sync(gmask, ang) >> gmask_shift) & 0xffu;
            if (ang) alist[nang + __popc(bal & ((1u << sub) - 1u))] = (unsigned short)j;
            nang += __popc(bal);
        }
#pragma unroll
        for (int n = 0; n < NMAX; n++) {
            const T s = group_sum(qacc[n], gmask);
            if (sub == (n & (NEP_GROUP - 1)) && n < A.n_r) q[n] = s;
        }
        __syncwarp(gmask);

        // ---- 2. angular sums: lane `sub` ends with S[mu][3 sub .. 3 sub + 2] ------------------------
        T Sacc[NMAX][3];
#pragma unroll
        for (int mu = 0; mu < NMAX; mu++) Sacc[mu][0] = Sacc[mu][1] = Sacc[mu][2] = T(0);
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
            {
                T f[CSP], df[CSP], row[RS];
                nep_radial<T, CSP>(r, A.rc_a, f, df);
                const T *crow = ctab + (size_t)tj * TROW + NMAX * CSP;
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++) {
                    T c[CSP];
                    load_vec<T, CSP>(crow + mu * CSP, c);
                    T g = T(0);
#pragma unroll
                    for (int k = 0; k < CSP; k++) g = fma(c[k], f[k], g);
                    row[mu] = on ? g : T(0);
                }
                const T ux = x * rinv, uy = y * rinv, uz = z * rinv;
                {
                    const T x_ = ux, y_ = uy, z_ = uz;
                    NEP_POLY_COMMON(x_, y_, z_)
#define NEP_X(k, val, gx, gy, gz) row[NMAX + k] = (val);
                    NEP_FOR_EACH_LM(NEP_X, x_, y_, z_)
#undef NEP_X
                }
                store_vec<T, RS>(stage + sub * RS, row);
            }
            __syncwarp(gmask);
            const int cnt = min(NEP_GROUP, nang - k0);
            for (int jj = 0; jj < cnt; jj++) {
                const T *rj = stage + jj * RS;
                T gj[NMAX];
                load_vec<T, NMAX>(rj, gj);
                const T b0 = rj[NMAX + 3 * sub], b1 = rj[NMAX + 3 * sub + 1], b2 = rj[NMAX + 3 * sub + 2];
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++) {
                    Sacc[mu][0] = fma(gj[mu], b0, Sacc[mu][0]);
                    Sacc[mu][1] = fma(gj[mu], b1, Sacc[mu][1]);
                    Sacc[mu][2] = fma(gj[mu], b2, Sacc[mu][2]);
                }
            }
            __syncwarp(gmask);
        }
#pragma unroll
        for (int mu = 0; mu < NMAX; mu++) {
            S[mu * NEP_NLM + 3 * sub] = Sacc[mu][0];
            S[mu * NEP_NLM + 3 * sub + 1] = Sacc[mu][1];
            S[mu * NEP_NLM + 3 * sub + 2] = Sacc[mu][2];
        }
        __syncwarp(gmask);

        // ---- 3. angular descriptors, network ------------------------------------------------------------
        for (int p = sub; p < A.n_a * A.l_max; p += NEP_GROUP) {
            const int mu = p / A.l_max, l = p % A.l_max + 1;
            T acc = T(0);
            for (int mp = 0; mp < 2 * l + 1; mp++) {
                const int lm = l * l - 1 + mp;
                const T s = S[mu * NEP_NLM + lm];
                acc += (mp == 0 ? T(1) : T(2)) * (T)c_C3B[lm] * s * s;
            }
            q[A.n_r + p] = acc;
        }
        __syncwarp(gmask);
        if (MODE == NEP_DESC) {
            if (valid)
                for (int k = sub; k < A.nd; k += NEP_GROUP) A.desc[slot * A.nd + k] = q[k];
            __syncwarp(gmask);
            continue;
        }
        const T *W0 = A.w0 + (size_t)ti * A.nneu * A.nd, *B0 = A.b0 + (size_t)ti * A.nneu, *W1 = A.w1 + (size_t)ti * A.nneu;
        for (int k = sub; k < A.nd; k += NEP_GROUP) Eq[k] = q[k] * iqs[k];
        __syncwarp(gmask);
        T es = T(0);
        for (int p = sub; p < A.nneu; p += NEP_GROUP) {
            const T *wrow = W0 + p * A.nd;
            T h0 = T(0), h1 = T(0), h2 = T(0), h3 = T(0);
            int k = 0;
            for (; k + 3 < A.nd; k += 4) {
                h0 = fma(wrow[k], Eq[k], h0);
                h1 = fma(wrow[k + 1], Eq[k + 1], h1);
                h2 = fma(wrow[k + 2], Eq[k + 2], h2);
                h3 = fma(wrow[k + 3], Eq[k + 3], h3);
            }
            for (; k < A.nd; k++) h0 = fma(wrow[k], Eq[k], h0);
            const T th = gtanh((h0 + h1) + (h2 + h3) + B0[p]);
            es += W1[p] * th;
            act[p] = W1[p] * (T(1) - th * th);
        }
        es = group_sum(es, gmask);
        __syncwarp(gmask);
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
        __syncwarp(gmask);
        // adjoints of the sums, layout [lm][NMAX] for 16-byte broadcast loads in the force pass
#pragma unroll
        for (int i = 0; i < 3; i++) {
            const int lm = 3 * sub + i;
            const int l = lm >= 15 ? 4 : lm >= 8 ? 3 : lm >= 3 ? 2 : 1;
            T e[NMAX];
#pragma unroll
            for (int mu = 0; mu < NMAX; mu++)
                e[mu] = (lm < nlm && mu < A.n_a) ? fac_s[lm] * Eq[A.n_r + mu * A.l_max + l - 1] * Sacc[mu][i] : T(0);
            store_vec<T, NMAX>(ES + lm * NMAX, e);
        }
        T eqr[NMAX];
#pragma unroll
        for (int n = 0; n < NMAX; n++) eqr[n] = n < A.n_r ? Eq[n] : T(0);
        __syncwarp(gmask);

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
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {     // radial part from the cached g'_n
            const int j = j0 + sub;
            bool on = j < nn;
            T x = 0, y = 0, z = 0;
            int nj = 0;
            T dgv[NMAX];
#pragma unroll
            for (int n = 0; n < NMAX; n++) dgv[n] = T(0);
            if (on) {
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j];
                load_vec<T, NMAX>(dcache + (size_t)j * NMAX, dgv);
            }
            const T r = gsqrt(x * x + y * y + z * z);
            on = on && r <= A.rc_r && r > T(0);
            T gr = T(0);
#pragma unroll
            for (int n = 0; n < NMAX; n++) gr = fma(eqr[n], dgv[n], gr);
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
            T g[NMAX], dg[NMAX];
            {
                T f[CSP], df[CSP];
                nep_radial<T, CSP>(r, A.rc_a, f, df);
                const T *crow = ctab + (size_t)tj * TROW + NMAX * CSP;
#pragma unroll
                for (int mu = 0; mu < NMAX; mu++) {
                    T c[CSP];
                    load_vec<T, CSP>(crow + mu * CSP, c);
                    T a = T(0), d = T(0);
#pragma unroll
                    for (int k = 0; k < CSP; k++) {
                        a = fma(c[k], f[k], a);
                        d = fma(c[k], df[k], d);
                    }
                    g[mu] = a; dg[mu] = d;
                }
            }
            T Pv[NMAX], Gx[NMAX], Gy[NMAX], Gz[NMAX];
#pragma unroll
            for (int mu = 0; mu < NMAX; mu++) Pv[mu] = Gx[mu] = Gy[mu] = Gz[mu] = T(0);
            {
                NEP_POLY_COMMON(ux, uy, uz)
#define NEP_X(k, val, gx_, gy_, gz_)                                      \
    {                                                                     \
        T e[NMAX];                                                        \
        load_vec<T, NMAX>(ES + (k) * NMAX, e);                            \
        nep_acc<T, NMAX>(e, (val), Pv);                                   \
        nep_acc<T, NMAX>(e, (gx_), Gx);                                   \
        nep_acc<T, NMAX>(e, (gy_), Gy);                                   \
        nep_acc<T, NMAX>(e, (gz_), Gz);                                   \
    }
                NEP_FOR_EACH_LM(NEP_X, ux, uy, uz)
#undef NEP_X
            }
            T gx = 0, gy = 0, gz = 0;
#pragma unroll
            for (int mu = 0; mu < NMAX; mu++) {
                const T ug = ux * Gx[mu] + uy * Gy[mu] + uz * Gz[mu];
                const T c = g[mu] * rinv, a = dg[mu] * Pv[mu] - c * ug;
                gx += a * ux + c * Gx[mu];
                gy += a * uy + c * Gy[mu];
                gz += a * uz + c * Gz[mu];
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
        __syncwarp();   // blk_b is rewritten by thread 0 at the top of the next round
    }
}

}  // namespace ai2b
