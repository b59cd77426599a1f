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
//   * the network weights of all types sit in shared memory as zero-padded rows (16-byte loads,
//     compile-time trip counts);
//   * energy and virial accumulate per lane over all atoms a group visits and are reduced once
//     per block at the end of the kernel (or when the structure index changes), so the loop over
//     atoms has no block-wide barrier;
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

// padded descriptor count: rows of the network's first layer are 16-byte aligned and an odd
// number of 16-byte chunks long (conflict-free when eight lanes read eight rows)
template <int NMAX>
struct NepFastDims {
    static constexpr int ND = 5 * NMAX;                                   // >= n_r + n_a * l_max
    static constexpr int NDP = ((ND / 4) & 1) ? ND : ND + 4;
};
__host__ __device__ inline int nep_r4(int n) { return (n + 3) & ~3; }
__host__ __device__ inline int nep_r32(int n) { return (n + 31) & ~31; }   // neurons per type, padded
// shared-memory elements (of T) per atom slot of the specialised kernel
template <int NMAX>
__host__ __device__ inline int nep_fast_atom_elems(int nneu, int umax, bool cache)
{
    const int sea = 2 * NEP_NLM * NMAX + nep_r32(nneu);       // S, ES, act ...
    const int stage = NEP_GROUP * (NMAX + NEP_NLM);           // ... share their space with the staging rows
    return 2 * NepFastDims<NMAX>::NDP + (sea > stage ? sea : stage) + (cache ? umax * NMAX : 0);
}
// elements (of T) of the block-wide tables: coefficients, then (unless descriptors only) W0, b0, w1
template <int NMAX, int CSP>
__host__ __device__ inline int nep_fast_table_elems(int ntypes, int nneu, bool net)
{
    int n = nep_r4(ntypes * ntypes * 2 * NMAX * CSP);
    if (net) n += ntypes * nep_r32(nneu) * (NepFastDims<NMAX>::NDP + 2);
    return n;
}

template <typename T, int CSP, int MODE, int NMAX, int MINB>
__global__ void __launch_bounds__(NEP_WARPS * 32, MINB) nep_fast_kernel(const NepArgs<T> A, const T *__restrict__ coeffs)
{
    constexpr int RS = NMAX + NEP_NLM;     // staging row: g[NMAX] | B_lm[24]
    constexpr int TROW = 2 * NMAX * CSP;   // coefficient rows of one (ti,tj) pair
    constexpr bool CACHE = MODE != NEP_DESC;
    extern __shared__ __align__(16) unsigned char nep_smem[];
    constexpr int NDP = NepFastDims<NMAX>::NDP;
    constexpr bool NET = MODE != NEP_DESC;
    __shared__ T blk_acc[10];
    __shared__ int blk_b;
    __shared__ T iqs[NDP];           // 1 / q_scaler, zero beyond the descriptor count
    __shared__ T fac_s[NEP_NLM];     // (2 - delta_m0) * 2 * C_lm
    __shared__ T c3w_s[NEP_NLM];     // (2 - delta_m0) * C_lm
    __shared__ unsigned char pm_mu[NDP], pm_l[NDP];   // angular descriptor p -> (mu, l)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    chain_release();
    const int sub = lane & (NEP_GROUP - 1), grp = lane / NEP_GROUP;
    const int slot_in_block = warp * NEP_APW + grp;
    const unsigned gmask_shift = grp * NEP_GROUP;
    const unsigned gmask = 0xffu << gmask_shift;
    const int per_atom = nep_fast_atom_elems<NMAX>(A.nneu, A.umax, CACHE);
    const int ntab = A.ntypes * A.ntypes * TROW;
    const int NP = nep_r32(A.nneu), nrow = A.ntypes * NP;   // zero rows pad every type to NP neurons
    T *ctab_s = reinterpret_cast<T *>(nep_smem);
    T *W0s = ctab_s + nep_r4(ntab);              // [ntypes * nneu][NDP], zero-padded rows
    T *B0s = W0s + (NET ? nrow * NDP : 0);
    T *W1s = B0s + (NET ? nrow : 0);
    T *atoms_s = ctab_s + nep_fast_table_elems<NMAX, CSP>(A.ntypes, A.nneu, NET);
    T *q = atoms_s + (size_t)slot_in_block * per_atom;   // [NDP]
    T *Eq = q + NDP;                       // [NDP]
    T *S = Eq + NDP;                       // [NMAX][24]
    T *ES = S + NEP_NLM * NMAX;            // [24][NMAX]
    T *act = ES + NEP_NLM * NMAX;
    T *stage = S;                          // staging rows of the angular sums (before S, ES, act are written)
    const int sea = 2 * NEP_NLM * NMAX + NP, stg = NEP_GROUP * RS;
    T *dcache = S + (sea > stg ? sea : stg);   // [umax][NMAX]: g'_n of every neighbour
    unsigned short *alist = reinterpret_cast<unsigned short *>(atoms_s + (size_t)NEP_APB * per_atom) + (size_t)slot_in_block * A.umax;
    const int ntot_n = A.n_r + A.n_a;
    const int nlm = A.l_max * A.l_max + 2 * A.l_max;
    const int nq_a = A.l_max > 0 ? A.n_a * A.l_max : 0;

    // block prologue: zero-padded tables, 1/q_scaler, 3-body factors, descriptor index map.
    // The tables [coefficients | W0 rows | b0 | w1] are one contiguous run of shared memory; every
    // thread first issues all of its (independent) global loads of the coefficients, then stores.
    {
        T qsv = T(1);
        if (NET && (int)threadIdx.x < A.nd) qsv = A.qs[threadIdx.x];
        const int n0 = nep_r4(ntab), n1 = n0 + (NET ? nrow * NDP : 0), n2 = n1 + (NET ? nrow : 0);
        const int nall = n2 + (NET ? nrow : 0);
        // neurons per type are padded to a multiple of 32: a power of two for the usual sizes, so the row -> (type,
        // neuron) split is a shift instead of an integer division per staged element
        const int np_shift = (NP & (NP - 1)) == 0 ? __ffs(NP) - 1 : -1;
        auto split = [&](int row, int &t, int &pn) {
            if (np_shift >= 0) { t = row >> np_shift; pn = row & (NP - 1); }
            else { t = row / NP; pn = row % NP; }
        };
        auto load = [&](int i) -> T {
            if (i < n0) {
                if (i >= ntab) return T(0);
                const int k = i % CSP, n = (i / CSP) % (2 * NMAX), pair = i / TROW;
                const int row = n < NMAX ? (n < A.n_r ? n : -1) : (n - NMAX < A.n_a ? A.n_r + n - NMAX : -1);
                return (k < A.cs && row >= 0) ? coeffs[((size_t)pair * ntot_n + row) * A.cs + k] : T(0);
            }
            if (i < n1) {
                const int row = (i - n0) / NDP, k = (i - n0) % NDP;
                int t, pn;
                split(row, t, pn);
                return (k < A.nd && pn < A.nneu) ? A.w0[((size_t)t * A.nneu + pn) * A.nd + k] : T(0);
            }
            const int row = i < n2 ? i - n1 : i - n2;
            int t, pn;
            split(row, t, pn);
            if (pn >= A.nneu) return T(0);
            return i < n2 ? A.b0[t * A.nneu + pn] : A.w1[t * A.nneu + pn];
        };
        // coefficients: through registers (the radial pass of the first atom needs them at once)
        constexpr int U = 8;
        for (int i0 = threadIdx.x; i0 < n0; i0 += U * blockDim.x) {
            T v[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < n0 ? load(i) : T(0);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = i0 + u * blockDim.x;
                if (i < n0) ctab_s[i] = v[u];
            }
        }
        // network tables: asynchronous copies straight into shared memory, awaited before the first atom's network
        // (they travel during its radial and angular passes); padding entries are plain zero stores
        for (int i = n0 + threadIdx.x; i < nall; i += blockDim.x) {
            const T *src = nullptr;
            if (i < n1) {
                const int row = (i - n0) / NDP, k = (i - n0) % NDP;
                int t, pn;
                split(row, t, pn);
                if (k < A.nd && pn < A.nneu) src = A.w0 + ((size_t)t * A.nneu + pn) * A.nd + k;
            } else {
                const int row = i < n2 ? i - n1 : i - n2;
                int t, pn;
                split(row, t, pn);
                if (pn < A.nneu) src = (i < n2 ? A.b0 : A.w1) + t * A.nneu + pn;
            }
            if (src) __pipeline_memcpy_async(ctab_s + i, src, sizeof(T));
            else ctab_s[i] = T(0);
        }
        __pipeline_commit();
        if (NET && threadIdx.x < NDP) iqs[threadIdx.x] = (int)threadIdx.x < A.nd ? T(1) / qsv : T(0);
    }
    if (threadIdx.x < NEP_NLM) {
        const int lm = threadIdx.x;
        const bool m0 = lm == 0 || lm == 3 || lm == 8 || lm == 15;
        c3w_s[lm] = (m0 ? T(1) : T(2)) * (T)c_C3B[lm];
        fac_s[lm] = (m0 ? T(1) : T(2)) * T(2) * (T)c_C3B[lm];
    }
    for (int p = threadIdx.x; p < NDP; p += blockDim.x) {
        const bool in = p < nq_a;
        pm_mu[p] = (unsigned char)(in ? p / A.l_max : 0);
        pm_l[p] = (unsigned char)(in ? p % A.l_max + 1 : 0);
    }
    // descriptors and their adjoints are read as NDP-long vectors: the padding stays zero
    for (int i = threadIdx.x; i < NEP_APB * 2 * NDP; i += blockDim.x) atoms_s[(size_t)(i / (2 * NDP)) * per_atom + i % (2 * NDP)] = T(0);
    __syncthreads();
    chain_wait();        // the prologue read the model only: it ran while the kernels before this one drained

    const int ntot = A.B == 1 ? A.binum[0] : A.prefix[A.B];
    const int ngroups = gridDim.x * NEP_APB;
    const int gidx = blockIdx.x * NEP_APB + slot_in_block;
    const int rounds = (ntot + ngroups - 1) / ngroups;

    // energy / virial of the atoms this lane has worked on, all of structure `bcur`
    T e_acc = T(0), vir[9];
#pragma unroll
    for (int k = 0; k < 9; k++) vir[k] = T(0);
    int bcur = -1;
    auto flush_group = [&]() {   // called by all lanes of a group together
        e_acc = group_sum(e_acc, gmask);
        if (sub == 0) atomicAdd(A.etot + bcur, e_acc);
        e_acc = T(0);
        if (MODE == NEP_EFV) {
#pragma unroll
            for (int k = 0; k < 9; k++) {
                const T v = group_sum(vir[k], gmask);
                if (sub == 0) atomicAdd(A.virial + 9 * bcur + k, v);
                vir[k] = T(0);
            }
        }
    };

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

        if (NET && valid && b != bcur) {
            if (bcur >= 0) flush_group();
            bcur = b;
        }

        // ---- 1. radial pass: q_n, cached g'_n, compaction of the angular neighbours ----------------
        T qacc[NMAX];
#pragma unroll
        for (int n = 0; n < NMAX; n++) qacc[n] = T(0);
        int nang = 0;
        // the next chunk's positions and indices are requested before this chunk is worked on
        T xn = 0, yn = 0, zn = 0;
        int njn = 0;
        if (sub < nn) { xn = rc[3 * sub]; yn = rc[3 * sub + 1]; zn = rc[3 * sub + 2]; njn = fn[sub]; }
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {
            const int j = j0 + sub;
            bool on = j < nn;
            const T x = xn, y = yn, z = zn;
            const int tj = on ? types[njn] : 0;
            {
                const int jn = j + NEP_GROUP;
                xn = yn = zn = T(0);
                if (jn < nn) { xn = rc[3 * jn]; yn = rc[3 * jn + 1]; zn = rc[3 * jn + 2]; njn = fn[jn]; }
            }
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
            // list entry: neighbour slot (10 bits) | neighbour type (4 bits)
            if (ang) alist[nang + __popc(bal & ((1u << sub) - 1u))] = (unsigned short)(j | (tj << 10));
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
                const int ent = alist[k0 + sub], j = ent & 1023;
                tj = ent >> 10;
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
                r = gsqrt(x * x + y * y + z * z);
                rinv = T(1) / r;
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
        for (int p = sub; p < nq_a; p += NEP_GROUP) {
            const int mu = pm_mu[p], l = pm_l[p];
            const T *Srow = S + mu * NEP_NLM + l * l - 1;
            const T *cw = c3w_s + l * l - 1;
            T acc = T(0);
            for (int mp = 0; mp < 2 * l + 1; mp++) acc += cw[mp] * Srow[mp] * Srow[mp];
            q[A.n_r + p] = acc;
        }
        __syncwarp(gmask);
        if constexpr (MODE == NEP_DESC) {
            if (valid)
                for (int k = sub; k < A.nd; k += NEP_GROUP) A.desc[slot * A.nd + k] = q[k];
            __syncwarp(gmask);
        } else {
        // network on the scaled descriptors; rows and vectors are zero-padded to NDP
        if (it == 0) {      // the network tables requested in the prologue have to be there now
            __pipeline_wait_prior(0);
            __syncthreads();
        }
        for (int k = sub; k < A.nd; k += NEP_GROUP) Eq[k] = q[k] * iqs[k];
        __syncwarp(gmask);
        T es = T(0);
        const T *W0t = W0s + (size_t)ti * NP * NDP;
        for (int p0 = 0; p0 < NP; p0 += 4 * NEP_GROUP) {   // four neurons per lane at a time
            T h[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) h[i][0] = h[i][1] = h[i][2] = h[i][3] = T(0);
#pragma unroll
            for (int c = 0; c < NDP / 4; c++) {
                T e[4];
                load_vec<T, 4>(Eq + 4 * c, e);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    T w[4];
                    load_vec<T, 4>(W0t + (size_t)(p0 + sub + NEP_GROUP * i) * NDP + 4 * c, w);
#pragma unroll
                    for (int k = 0; k < 4; k++) h[i][k] = fma(w[k], e[k], h[i][k]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int p = p0 + sub + NEP_GROUP * i;
                const T th = gtanh((h[i][0] + h[i][1]) + (h[i][2] + h[i][3]) + B0s[ti * NP + p]);
                const T w1 = W1s[ti * NP + p];   // zero for padding neurons
                es += w1 * th;
                act[p] = w1 * (T(1) - th * th);
            }
        }
        if (valid) e_acc += es + (sub == 0 ? A.bias[ti] : T(0));
        __syncwarp(gmask);
        for (int c = sub; c < NDP / 4; c += NEP_GROUP) {   // lane c: descriptors 4c .. 4c+3
            const T *wcol = W0t + 4 * c;
            T a[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i][0] = a[i][1] = a[i][2] = a[i][3] = T(0);
            for (int p = 0; p < NP; p += 4) {
                T x[4];
                load_vec<T, 4>(act + p, x);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    T w[4];
                    load_vec<T, 4>(wcol + (size_t)(p + i) * NDP, w);
#pragma unroll
                    for (int k = 0; k < 4; k++) a[i][k] = fma(x[i], w[k], a[i][k]);
                }
            }
            T r[4];
#pragma unroll
            for (int k = 0; k < 4; k++) r[k] = ((a[0][k] + a[1][k]) + (a[2][k] + a[3][k])) * iqs[4 * c + k];
            store_vec<T, 4>(Eq + 4 * c, r);
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
        T fcx = 0, fcy = 0, fcz = 0;
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
        xn = yn = zn = T(0);
        if (sub < nn) { xn = rc[3 * sub]; yn = rc[3 * sub + 1]; zn = rc[3 * sub + 2]; njn = fn[sub]; }
        for (int j0 = 0; j0 < nn; j0 += NEP_GROUP) {     // radial part from the cached g'_n
            const int j = j0 + sub;
            bool on = j < nn;
            const T x = xn, y = yn, z = zn;
            const int nj = njn;
            {
                const int jn = j + NEP_GROUP;
                xn = yn = zn = T(0);
                if (jn < nn) { xn = rc[3 * jn]; yn = rc[3 * jn + 1]; zn = rc[3 * jn + 2]; njn = fn[jn]; }
            }
            T dgv[NMAX];
#pragma unroll
            for (int n = 0; n < NMAX; n++) dgv[n] = T(0);
            if (on) load_vec<T, NMAX>(dcache + (size_t)j * NMAX, dgv);
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
                const int ent = alist[k0 + sub], j = ent & 1023;
                tj = ent >> 10;
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
                nj = fn[j];
                r = gsqrt(x * x + y * y + z * z);
                rinv = T(1) / r;
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
        if (sub == 0 && valid) {
            atomicAdd(frc + 3 * ci + 0, fcx);
            atomicAdd(frc + 3 * ci + 1, fcy);
            atomicAdd(frc + 3 * ci + 2, fcz);
        }
        }   // MODE != NEP_DESC
    }

    // energy / virial: groups whose atoms belong to the structure of the block's first group
    // combine in shared memory, the others add to the outputs directly
    if (NET) {
        if (threadIdx.x == 0) blk_b = bcur;
        if (threadIdx.x < 10) blk_acc[threadIdx.x] = T(0);
        __syncthreads();
        if (bcur >= 0) {
            const bool local = bcur == blk_b;
            e_acc = group_sum(e_acc, gmask);
            if (sub == 0) atomicAdd(local ? &blk_acc[0] : A.etot + bcur, e_acc);
            if (MODE == NEP_EFV) {
#pragma unroll
                for (int k = 0; k < 9; k++) {
                    const T v = group_sum(vir[k], gmask);
                    if (sub == 0) atomicAdd(local ? &blk_acc[1 + k] : A.virial + 9 * bcur + k, v);
                }
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
