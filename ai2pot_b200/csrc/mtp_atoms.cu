// Linear MTP, forward (basic moments) and force kernels with lanes = atoms.
//
// The reference evaluates one atom at a time: for every neighbour it raises the distance vector to all
// powers, multiplies by the radial functions and adds into the basic moments (mtpBasis.h:472-519), and on
// the way back multiplies every basic moment's adjoint by the derivative of that product
// (linearMtp.h:297-320). Here a block owns a tile of 32 atoms and every lane owns ONE atom, so a moment
// sum or a polynomial value never leaves the registers of its thread:
//  * forward: the four warps of the block share the tile; each owns the monomial degrees of one group
//    (groups balanced by accumulator count) and keeps those moments of its atom in registers while it
//    walks over the atom's neighbours. The radial functions and unit vectors of 16 neighbour slots at a
//    time are computed once (each warp a quarter of them) and handed over through shared memory.
//  * force: each warp takes every fourth neighbour slot. The adjoints of the tile's basic moments sit in
//    shared memory as [dense moment][atom], so a coefficient is one conflict-free load at a compile-time
//    offset; the polynomial of a radial function and its gradient are evaluated by nested sums over the
//    z, y and x exponents (two FMAs per coefficient instead of four).
// The basic moments and their adjoints travel between the kernels as [tile][basic row][32 atoms], which
// all three kernels read and write in full 256-byte rows.
// The kernels are compiled per "signature" = the highest monomial degree of every radial function
// (non-increasing, at most four functions); other tables take the warp-per-atom kernels.
#include <cuda_pipeline.h>
#include "mtp_device.cuh"
#include "tile_rows.cuh"

namespace ai2b {

constexpr int AT_WARPS = 4;       // warps per block; a block works on one tile of MTP_TILE atoms at a time
constexpr int AT_CH = 16;         // neighbour slots staged per round of the forward kernel
constexpr size_t AT_CF_BYTES = 16 * 1024;   // largest radial-coefficient table kept in shared memory

template <int K0, int K1, int K2, int K3>
struct KSig {
    static constexpr int KD = K0;
    static constexpr int NMUS = (K0 >= 0) + (K1 >= 0) + (K2 >= 0) + (K3 >= 0);
    __host__ __device__ static constexpr int k(int mu) { return mu == 0 ? K0 : mu == 1 ? K1 : mu == 2 ? K2 : K3; }
    // number of radial functions whose moments reach degree D: they are mu = 0 .. cnt(D) - 1
    __host__ __device__ static constexpr int cnt(int D) { return (K0 >= D) + (K1 >= D) + (K2 >= D) + (K3 >= D); }
    __host__ __device__ static constexpr int doff(int mu)
    {
        int o = 0;
        for (int m = 0; m < mu; m++) o += ncan(k(m));
        return o;
    }
    static constexpr int NDENSE = doff(NMUS);
    // warp that accumulates the monomials of degree D: degrees are dealt by decreasing accumulator count to
    // the least loaded warp
    __host__ __device__ static constexpr int group(int D)
    {
        int load[AT_WARPS] = {0, 0, 0, 0};
        int grp[KD + 1] = {};
        bool done[KD + 1] = {};
        for (int it = 0; it <= KD; it++) {
            int best = -1, bw = -1;
            for (int d = 0; d <= KD; d++) {
                const int w = ndeg(d) * cnt(d);
                if (!done[d] && w > bw) { bw = w; best = d; }
            }
            int g = 0;
            for (int i = 1; i < AT_WARPS; i++)
                if (load[i] < load[g]) g = i;
            grp[best] = g;
            load[g] += bw;
            done[best] = true;
        }
        return grp[D];
    }
    __host__ __device__ static constexpr int acc_off(int D)
    {
        int o = 0;
        for (int d = 0; d < D; d++)
            if (group(d) == group(D)) o += ndeg(d) * cnt(d);
        return o;
    }
    __host__ __device__ static constexpr int acc_count(int G)
    {
        int o = 0;
        for (int d = 0; d <= KD; d++)
            if (group(d) == G) o += ndeg(d) * cnt(d);
        return o;
    }
};

// Row stride of the radial-coefficient table in shared memory: lanes of a warp read the rows of different type
// pairs at the same offset, so consecutive rows are shifted by 16 bytes (4 banks) against one another.
template <typename SIG, int CSP>
__host__ __device__ constexpr int cf_stride() { return SIG::NMUS * CSP + 2; }
// elements of the whole table, rounded so that what follows it in shared memory starts on a 16-byte boundary
template <typename SIG, int CSP>
__host__ __device__ constexpr int cf_elems(int ntypes) { return (ntypes * ntypes * cf_stride<SIG, CSP>() + 3) & ~3; }

// One neighbour of this lane's atom: geometry and the radial functions of every mu (registers). The three steps
// are separate so that the loads of several neighbours can be in flight together.
template <typename T, typename SIG, int CSP>
struct PairEval {
    T x, y, z, ux, uy, uz, rinv;
    T f[SIG::NMUS], fd[SIG::NMUS];
    int nj, tj;
    bool act;
    __device__ __forceinline__ void load(const MtpArgs<T> &A, size_t row, int j, int nn)
    {
        act = j < nn;
        x = y = z = T(0);
        nj = 0;
        if (act) {
            const T *rc = A.rcs + (row + j) * 3;
            x = rc[0]; y = rc[1]; z = rc[2];
            nj = A.firstneigh[row + j];
        }
    }
    __device__ __forceinline__ void lookup(const int *types_b) { tj = act ? types_b[nj] : 0; }
    // slot j of this lane's atom: from the staged rows, or from global memory beyond them
    __device__ __forceinline__ void fetch(const MtpArgs<T> &A, const TileRows<T> &tr, const int *types_b, size_t row, int lane, int j, int nn)
    {
        if (j < TR_SLOTS) {
            act = j < nn;
            const T *p = tr.pos + lane * TR_RS + 3 * j;
            const int w = tr.idx[lane * TR_IS + j];
            x = act ? p[0] : T(0); y = act ? p[1] : T(0); z = act ? p[2] : T(0);
            nj = w & TR_INDEX_MASK;
            tj = w >> TR_TYPE_SHIFT;
        } else {
            load(A, row, j, nn);
            lookup(types_b);
        }
    }
    // inv_range = 1 / (rmax - rmin), computed once per thread
    template <bool DERIV>
    __device__ __forceinline__ void compute(const MtpArgs<T> &A, const T *cf, int ti, T inv_range)
    {
        using V2 = typename Vec2<T>::type;
        // 1 / r from the reciprocal square root (one special-function sequence instead of a square root and a division)
        const T r2 = x * x + y * y + z * z;
        const T ri = r2 > T(0) ? grsqrt(r2) : T(0);
        const T r = r2 * ri;
        act = act && (r <= A.rmax) && (r > T(0));
        rinv = act ? ri : T(0);
        ux = x * rinv; uy = y * rinv; uz = z * rinv;
        T q[CSP], dq[CSP];
        mtp_radial_basis<T, CSP>(act ? r : A.rmax, A.rmax, A.rmin, A.scaling, q, dq, inv_range);
        const T *crow = cf + (size_t)(ti * A.ntypes + (act ? tj : 0)) * cf_stride<SIG, CSP>();
        static_for<0, SIG::NMUS>([&](auto mm) {
            constexpr int m = decltype(mm)::value;
            T s = T(0), sd = T(0);
#pragma unroll
            for (int k = 0; k < CSP; k += 2) {
                const V2 c2 = *reinterpret_cast<const V2 *>(crow + m * CSP + k);
                s = fma(c2.x, q[k], s);
                s = fma(c2.y, q[k + 1], s);
                if (DERIV) { sd = fma(c2.x, dq[k], sd); sd = fma(c2.y, dq[k + 1], sd); }
            }
            f[m] = act ? s : T(0);
            fd[m] = act ? sd : T(0);
        });
    }
};

// radial coefficients [ntypes^2][NMUS][CSP] -> shared-memory rows of cf_stride elements
template <typename T, typename SIG, int CSP>
__device__ __forceinline__ void stage_coefficients(const MtpArgs<T> &A, T *cf)
{
    constexpr int RL = SIG::NMUS * CSP, RS = cf_stride<SIG, CSP>();
    const int n = A.ntypes * A.ntypes * RL;
    for (int i = threadIdx.x; i < n; i += blockDim.x) cf[(i / RL) * RS + (i % RL)] = A.coeffs_pad[i];
}

// per-lane bookkeeping of a tile
template <typename T>
struct TileAtom {
    bool valid;
    int b, ci, nn, ti;
    size_t slot;
    const int *types_b;
    __device__ __forceinline__ void set(const MtpArgs<T> &A, int t, int ntot)
    {
        valid = t < ntot;
        b = 0; ci = 0; nn = 0; ti = 0; slot = 0;
        types_b = A.types;
        if (valid) {
            if (A.B > 1) {      // one structure: atom t is slot t, no look-ups
                b = find_structure(A.prefix, A.B, t);
                slot = (size_t)b * A.npad + (t - A.prefix[b]);
            } else {
                slot = (size_t)t;
            }
            types_b = A.types + (size_t)b * (A.npad + A.nghost);
            ci = A.bilist[slot];
            nn = min(A.numneigh[slot], A.umax);
            ti = types_b[ci];
        }
    }
};

__device__ __forceinline__ int warp_max_int(int v)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = max(v, __shfl_xor_sync(FULL_MASK, v, o));
    return v;
}

// ---- forward --------------------------------------------------------------------------------------
// DERIV = false: basic moments M -> A.Mb. DERIV = true (loss gradient, linearMtpLoss.h:331-389): their directional
// derivatives D = sum_j p_ij . dM/dr_j along the pair weights p of the loss -> L.Db; per neighbour and monomial m
// that is a_mu m + f_mu (q . grad m) with a_mu = f'_mu (p . u), q = (p - (p . u) u) / r.
// shared memory: radial coefficients [ntypes^2][NMUS][CSP] (rows shifted), staging [AT_CH][NV][32], tile rows
template <typename T, typename SIG, int CSP, bool DERIV>
__global__ void __launch_bounds__(AT_WARPS * 32, DERIV ? 2 : 3) mtp_fwd_atoms_kernel(const MtpProgramDev P, const MtpArgs<T> A, const LossArgs<T> L)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NV = 3 + SIG::NMUS + (DERIV ? SIG::NMUS + 3 : 0);   // u, f [, a, q]
    constexpr int KD = SIG::KD;
    T *cf = reinterpret_cast<T *>(smem_raw);
    T *st = cf + cf_elems<SIG, CSP>(A.ntypes);
    TileRows<T> tr;
    tr.bind(reinterpret_cast<unsigned char *>(st + (size_t)AT_CH * NV * 32));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    chain_release();
    stage_coefficients<T, SIG, CSP>(A, cf);   // model constants: staged while the kernel before this one drains
    chain_wait();
    if (!DERIV && A.zero_outputs == 2) {      // no set-up launch: this first kernel of the call zeroes the outputs
        const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
        const size_t nf = 3 * (size_t)A.B * (A.npad + A.nghost);
        for (size_t i = i0; i < nf; i += step) A.force[i] = T(0);
        if (i0 < (size_t)A.B) A.etot[i0] = T(0);
        if (A.virial && i0 < 9 * (size_t)A.B) A.virial[i0] = T(0);
    }
    const int ntot = total_atoms(A);
    const int ntiles = (ntot + MTP_TILE - 1) / MTP_TILE;

    const bool single = A.B == 1;      // one structure: a tile's rows are known from its index alone
    const T inv_range = T(1) / (A.rmax - A.rmin);
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        if (single) {
            if (tile != (int)blockIdx.x) __syncthreads();     // the previous tile's rows are no longer read
            tr.template request<AT_WARPS * 32>(A.rcs, A.firstneigh, A.umax, (size_t)tile * MTP_TILE, (size_t)A.npad);
        }
        TileAtom<T> at;
        at.set(A, tile * MTP_TILE + lane, ntot);
        const int nmax = warp_max_int(at.nn);      // the same in every warp of the block
        const size_t row = at.slot * A.umax;
        const int nstruct = at.valid ? A.binum[at.b] : 1;
        T *out = (DERIV ? L.Db : A.Mb) + (size_t)tile * A.nbp * MTP_TILE + lane;
        if (single) {
            __pipeline_wait_prior(0);
            __syncthreads();     // every thread's copies have arrived
            tr.template complete<AT_WARPS * 32>(A.types, A.npad + A.nghost);
        } else {
            __syncthreads();     // the previous tile's rows are no longer read
            if (warp == 0) tr.describe(lane, row, (size_t)(at.types_b - A.types), at.nn);
            __syncthreads();
            tr.template stage<AT_WARPS * 32>(A.rcs, A.firstneigh, A.types, A.umax);
        }

        auto body = [&](auto gg) {
            constexpr int G = decltype(gg)::value;
            constexpr int NACC = SIG::acc_count(G);
            T acc[NACC > 0 ? NACC : 1];
#pragma unroll
            for (int i = 0; i < (NACC > 0 ? NACC : 1); i++) acc[i] = T(0);
            for (int j0 = 0; j0 < nmax; j0 += AT_CH) {
                const int cnt = min(AT_CH, nmax - j0);
                __syncthreads();     // rows and coefficients staged / the previous round's slots consumed
                for (int jj = warp; jj < cnt; jj += AT_WARPS) {   // this warp's slots of the round
                    PairEval<T, SIG, CSP> pe;
                    pe.fetch(A, tr, at.types_b, row, lane, j0 + jj, at.nn);
                    pe.template compute<DERIV>(A, cf, at.ti, inv_range);
                    T *s = st + (size_t)jj * NV * 32 + lane;
                    s[0] = pe.ux; s[32] = pe.uy; s[64] = pe.uz;
                    static_for<0, SIG::NMUS>([&](auto mm) { s[(3 + decltype(mm)::value) * 32] = pe.f[decltype(mm)::value]; });
                    if constexpr (DERIV) {
                        T px = T(0), py = T(0), pz = T(0);
                        if (pe.act) pair_weight(A, L, at.b, nstruct, at.ci, pe.nj, pe.x, pe.y, pe.z, px, py, pz);
                        const T ppar = px * pe.ux + py * pe.uy + pz * pe.uz;
                        static_for<0, SIG::NMUS>([&](auto mm) {
                            s[(3 + SIG::NMUS + decltype(mm)::value) * 32] = pe.fd[decltype(mm)::value] * ppar;
                        });
                        s[(3 + 2 * SIG::NMUS) * 32] = (px - ppar * pe.ux) * pe.rinv;
                        s[(4 + 2 * SIG::NMUS) * 32] = (py - ppar * pe.uy) * pe.rinv;
                        s[(5 + 2 * SIG::NMUS) * 32] = (pz - ppar * pe.uz) * pe.rinv;
                    }
                }
                __syncthreads();
                if constexpr (NACC > 0) {
#pragma unroll 2
                    for (int jj = 0; jj < cnt; jj++) {
                        const T *s = st + (size_t)jj * NV * 32 + lane;
                        Powers<T, KD> pw;
                        pw.set(s[0], s[32], s[64]);
                        T f[SIG::NMUS], a[SIG::NMUS], qx = T(0), qy = T(0), qz = T(0);
                        static_for<0, SIG::NMUS>([&](auto mm) { f[decltype(mm)::value] = s[(3 + decltype(mm)::value) * 32]; });
                        if constexpr (DERIV) {
                            static_for<0, SIG::NMUS>([&](auto mm) { a[decltype(mm)::value] = s[(3 + SIG::NMUS + decltype(mm)::value) * 32]; });
                            qx = s[(3 + 2 * SIG::NMUS) * 32]; qy = s[(4 + 2 * SIG::NMUS) * 32]; qz = s[(5 + 2 * SIG::NMUS) * 32];
                        }
                        static_for<0, KD + 1>([&](auto dd) {
                            constexpr int D = decltype(dd)::value;
                            if constexpr (SIG::group(D) == G) {
                                static_for<0, ndeg(D)>([&](auto qq) {
                                    constexpr int Q = decltype(qq)::value;
                                    const T m = mono<T, KD, D, Q>(pw);
                                    T dm = T(0);
                                    if constexpr (DERIV) {   // q . grad of the monomial
                                        constexpr Exp3 e = deg_exp(D, Q);
                                        if constexpr (e.x > 0) dm = fma(qx * T(e.x), pw.x[e.x - 1] * pw.y[e.y] * pw.z[e.z], dm);
                                        if constexpr (e.y > 0) dm = fma(qy * T(e.y), pw.x[e.x] * pw.y[e.y - 1] * pw.z[e.z], dm);
                                        if constexpr (e.z > 0) dm = fma(qz * T(e.z), pw.x[e.x] * pw.y[e.y] * pw.z[e.z - 1], dm);
                                    }
                                    static_for<0, SIG::cnt(D)>([&](auto mm) {
                                        constexpr int mu = decltype(mm)::value;
                                        constexpr int I = SIG::acc_off(D) + Q * SIG::cnt(D) + mu;
                                        if constexpr (DERIV) acc[I] = fma(a[mu], m, fma(f[mu], dm, acc[I]));
                                        else acc[I] = fma(f[mu], m, acc[I]);
                                    });
                                });
                            }
                        });
                    }
                }
            }
            // this warp's moments of the tile: one 256-byte row per moment
            static_for<0, KD + 1>([&](auto dd) {
                constexpr int D = decltype(dd)::value;
                if constexpr (SIG::group(D) == G) {
                    static_for<0, ndeg(D)>([&](auto qq) {
                        constexpr int Q = decltype(qq)::value;
                        static_for<0, SIG::cnt(D)>([&](auto mm) {
                            constexpr int mu = decltype(mm)::value;
                            const int r = P.dense_basic[SIG::doff(mu) + ncan(D - 1) + Q];
                            if (r >= 0) out[(size_t)r * MTP_TILE] = acc[SIG::acc_off(D) + Q * SIG::cnt(D) + mu];
                        });
                    });
                }
            });
        };
        switch (warp) {
            case 0: body(std::integral_constant<int, 0>{}); break;
            case 1: body(std::integral_constant<int, 1>{}); break;
            case 2: body(std::integral_constant<int, 2>{}); break;
            default: body(std::integral_constant<int, 3>{}); break;
        }
    }
}

// ---- force and virial -----------------------------------------------------------------------------
// shared memory: radial coefficients, adjoints [NDENSE][32]
template <typename T, int MODE, typename SIG, int CSP>
__global__ void __launch_bounds__(AT_WARPS * 32, 3) mtp_force_atoms_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KD = SIG::KD;
    T *cf = reinterpret_cast<T *>(smem_raw);
    T *Es = cf + cf_elems<SIG, CSP>(A.ntypes);
    TileRows<T> tr;
    tr.bind(reinterpret_cast<unsigned char *>(Es + (size_t)SIG::NDENSE * 32));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    chain_release();
    stage_coefficients<T, SIG, CSP>(A, cf);   // model constants: staged while the contraction drains
    chain_wait();
    const int ntot = total_atoms(A);
    const int ntiles = (ntot + MTP_TILE - 1) / MTP_TILE;
    const bool single = A.B == 1;      // one structure: a tile's rows are known from its index alone
    const T inv_range = T(1) / (A.rmax - A.rmin);

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        if (tile != (int)blockIdx.x) __syncthreads();     // the previous tile's adjoints and rows are no longer read
        {   // The contraction leaves the adjoints of a tile in dense monomial order, [dense][32 atoms] in one piece: they are
            // requested here with asynchronous 16-byte copies and awaited only before the neighbour loop.
            const T *ein = A.Eb + (size_t)tile * A.ndp * MTP_TILE;
            constexpr int CH = 16 / (int)sizeof(T);
            for (int c = threadIdx.x; c < SIG::NDENSE * 32 / CH; c += AT_WARPS * 32) __pipeline_memcpy_async(Es + c * CH, ein + c * CH, 16);
            __pipeline_commit();
        }
        if (single) tr.template request<AT_WARPS * 32>(A.rcs, A.firstneigh, A.umax, (size_t)tile * MTP_TILE, (size_t)A.npad);
        TileAtom<T> at;
        at.set(A, tile * MTP_TILE + lane, ntot);
        const int nmax = warp_max_int(at.nn);
        const size_t row = at.slot * A.umax;
        T *frc = A.force + (size_t)at.b * (A.npad + A.nghost) * 3;
        if (single) {
            __pipeline_wait_prior(0);     // the adjoints and the rows requested at the top of the tile
            __syncthreads();
            tr.template complete<AT_WARPS * 32>(A.types, A.npad + A.nghost);
        } else {
            __syncthreads();     // the previous tile's rows are no longer read
            if (warp == 0) tr.describe(lane, row, (size_t)(at.types_b - A.types), at.nn);
            __syncthreads();
            tr.template stage<AT_WARPS * 32>(A.rcs, A.firstneigh, A.types, A.umax);
            __pipeline_wait_prior(0);     // the adjoints requested at the top of the tile
        }
        __syncthreads();

        T fcx = T(0), fcy = T(0), fcz = T(0);
        T vir[9];
#pragma unroll
        for (int k = 0; k < 9; k++) vir[k] = T(0);
        const T *el = Es + lane;
        for (int j = warp; j < nmax; j += AT_WARPS) {
            PairEval<T, SIG, CSP> pe;
            pe.fetch(A, tr, at.types_b, row, lane, j, at.nn);
            pe.template compute<true>(A, cf, at.ti, inv_range);
            // powers of the unit vector and their derivatives k u^(k-1)
            T X[KD + 1], Y[KD + 1], Z[KD + 1], dX[KD + 1], dY[KD + 1], dZ[KD + 1];
            X[0] = Y[0] = Z[0] = T(1);
            dX[0] = dY[0] = dZ[0] = T(0);
            if constexpr (KD >= 1) { X[1] = pe.ux; Y[1] = pe.uy; Z[1] = pe.uz; }
#pragma unroll
            for (int k = 2; k <= KD; k++) {      // u^k = u^(k/2) u^(k - k/2): short chains of dependent products
                X[k] = X[k / 2] * X[k - k / 2]; Y[k] = Y[k / 2] * Y[k - k / 2]; Z[k] = Z[k / 2] * Z[k - k / 2];
            }
#pragma unroll
            for (int k = 1; k <= KD; k++) { dX[k] = T(k) * X[k - 1]; dY[k] = T(k) * Y[k - 1]; dZ[k] = T(k) * Z[k - 1]; }
            T gx = T(0), gy = T(0), gz = T(0);
            static_for<0, SIG::NMUS>([&](auto mm) {
                constexpr int mu = decltype(mm)::value;
                constexpr int K = SIG::k(mu);
                constexpr int base = SIG::doff(mu);
                // polynomial of this radial function in (ux, uy, uz) and its gradient, by nested sums
                T Pv = T(0), Gx = T(0), Gy = T(0), Gz = T(0);
                static_for<0, K + 1>([&](auto aa) {
                    constexpr int a = decltype(aa)::value;
                    T S = T(0), Sy = T(0), Sz = T(0);
                    static_for<0, K - a + 1>([&](auto bb) {
                        constexpr int b = decltype(bb)::value;
                        T R = T(0), Rz = T(0);
                        static_for<0, K - a - b + 1>([&](auto cc) {
                            constexpr int c = decltype(cc)::value;
                            const T e = el[(base + canon_index(a, b, c)) * 32];
                            if constexpr (c == 0) R = e; else R = fma(e, Z[c], R);
                            if constexpr (c == 1) Rz = e; else if constexpr (c > 1) Rz = fma(e, dZ[c], Rz);
                        });
                        if constexpr (b == 0) S = R; else S = fma(Y[b], R, S);
                        if constexpr (b == 1) Sy = R; else if constexpr (b > 1) Sy = fma(dY[b], R, Sy);
                        if constexpr (K - a - b >= 1) { if constexpr (b == 0) Sz = Rz; else Sz = fma(Y[b], Rz, Sz); }
                    });
                    if constexpr (a == 0) Pv = S; else Pv = fma(X[a], S, Pv);
                    if constexpr (a == 1) Gx = S; else if constexpr (a > 1) Gx = fma(dX[a], S, Gx);
                    if constexpr (K - a >= 1) {
                        if constexpr (a == 0) { Gy = Sy; Gz = Sz; }
                        else { Gy = fma(X[a], Sy, Gy); Gz = fma(X[a], Sz, Gz); }
                    }
                });
                const T ug = pe.ux * Gx + pe.uy * Gy + pe.uz * Gz;
                const T cc = pe.f[mu] * pe.rinv;
                const T aa = pe.fd[mu] * Pv - cc * ug;
                gx += aa * pe.ux + cc * Gx;
                gy += aa * pe.uy + cc * Gy;
                gz += aa * pe.uz + cc * Gz;
            });
            if (pe.act) {
                fcx += gx; fcy += gy; fcz += gz;
                atomicAdd(frc + 3 * pe.nj + 0, -gx);
                atomicAdd(frc + 3 * pe.nj + 1, -gy);
                atomicAdd(frc + 3 * pe.nj + 2, -gz);
                if (MODE == MODE_EFV) {
                    vir[0] -= gx * pe.x; vir[1] -= gx * pe.y; vir[2] -= gx * pe.z;
                    vir[3] -= gy * pe.x; vir[4] -= gy * pe.y; vir[5] -= gy * pe.z;
                    vir[6] -= gz * pe.x; vir[7] -= gz * pe.y; vir[8] -= gz * pe.z;
                }
            }
        }
        if (at.valid && warp < at.nn) {      // this warp saw at least one slot of the atom
            atomicAdd(frc + 3 * at.ci + 0, fcx);
            atomicAdd(frc + 3 * at.ci + 1, fcy);
            atomicAdd(frc + 3 * at.ci + 2, fcz);
        }
        if (MODE == MODE_EFV) {
            // one atomic per component when the 32 atoms belong to one structure, else one per atom
            const int b0 = __shfl_sync(FULL_MASK, at.b, 0);
            const bool uniform = __all_sync(FULL_MASK, !at.valid || at.b == b0);
            if (uniform) {      // (the same decision in every warp of the block: they share the tile's atoms)
                // the block's four partial sums are combined first: a quarter of the atomics on these nine addresses
                __shared__ T vred[AT_WARPS][9];
#pragma unroll
                for (int k = 0; k < 9; k++) {
                    const T s = warp_sum(vir[k]);
                    if (lane == 0) vred[warp][k] = s;
                }
                __syncthreads();
                if (threadIdx.x < 9) {
                    T s = T(0);
#pragma unroll
                    for (int w = 0; w < AT_WARPS; w++) s += vred[w][threadIdx.x];
                    atomicAdd(A.virial + 9 * b0 + threadIdx.x, s);
                }
            } else if (at.valid && warp < at.nn) {
#pragma unroll
                for (int k = 0; k < 9; k++) atomicAdd(A.virial + 9 * at.b + k, vir[k]);
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------
template <typename SIG>
static bool sig_matches(const MtpProgramDev &P)
{
    if (P.nmus != SIG::NMUS || P.ndense != SIG::NDENSE) return false;
    for (int m = 0; m < SIG::NMUS; m++)
        if (P.kmu[m] != SIG::k(m) || P.doff[m] != SIG::doff(m)) return false;
    return true;
}

// the template levels 6 to 16 of the reference's MTP_templates
using Sig16 = KSig<6, 4, 2, 0>;
using Sig14 = KSig<5, 3, 1, 0>;
using Sig12 = KSig<4, 2, 0, -1>;
using Sig10 = KSig<3, 1, 0, -1>;
using Sig08 = KSig<2, 0, -1, -1>;
using Sig06 = KSig<1, 0, -1, -1>;

#define AI2B_FOR_SIG(P, CALL)                \
    if (sig_matches<Sig16>(P)) { CALL(Sig16) } \
    if (sig_matches<Sig14>(P)) { CALL(Sig14) } \
    if (sig_matches<Sig12>(P)) { CALL(Sig12) } \
    if (sig_matches<Sig10>(P)) { CALL(Sig10) } \
    if (sig_matches<Sig08>(P)) { CALL(Sig08) } \
    if (sig_matches<Sig06>(P)) { CALL(Sig06) }

constexpr int AT_CSP = 8;

bool mtp_atoms_supported(const MtpProgramDev &P, int ntypes, int cs, size_t elem, long atom_ids)
{
    if (cs > AT_CSP || P.nmus > 4) return false;
    if (ntypes > 32 || atom_ids > TR_INDEX_MASK) return false;   // index | type << 26 in the staged rows
    if ((size_t)ntypes * ntypes * (P.nmus * AT_CSP + 2) * elem > AT_CF_BYTES) return false;
#define AI2B_SIG_YES(S) return true;
    AI2B_FOR_SIG(P, AI2B_SIG_YES)
#undef AI2B_SIG_YES
    return false;
}

template <typename T, typename SIG, bool DERIV>
static int launch_fwd_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, const LossArgs<T> &L, cudaStream_t st)
{
    const size_t ncf = (size_t)cf_elems<SIG, AT_CSP>(A.ntypes);
    const size_t smem = sizeof(T) * (ncf + (size_t)AT_CH * (3 + SIG::NMUS + (DERIV ? SIG::NMUS + 3 : 0)) * 32) + tile_rows_bytes<T>();
    auto kern = mtp_fwd_atoms_kernel<T, SIG, AT_CSP, DERIV>;
    static KernelSetup setup;
    int per_sm = 1;
    if (int rc = kernel_setup(setup, kern, smem, AT_WARPS * 32, &per_sm)) return rc;
    long tiles = ((long)A.B * A.npad + MTP_TILE - 1) / MTP_TILE;
    long blocks = (long)sm_count() * per_sm;
    if (blocks > tiles) blocks = tiles;
    AI2B_CUDA(launch_chained(kern, (unsigned)blocks, AT_WARPS * 32, smem, st, P, A, L));
    return AI2B_OK;
}

template <typename T, int MODE, typename SIG>
static int launch_force_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, cudaStream_t st)
{
    const size_t ncf = (size_t)cf_elems<SIG, AT_CSP>(A.ntypes);
    const size_t smem = sizeof(T) * (ncf + (size_t)SIG::NDENSE * 32) + tile_rows_bytes<T>();
    auto kern = mtp_force_atoms_kernel<T, MODE, SIG, AT_CSP>;
    static KernelSetup setup;
    int per_sm = 1;
    if (int rc = kernel_setup(setup, kern, smem, AT_WARPS * 32, &per_sm)) return rc;
    long tiles = ((long)A.B * A.npad + MTP_TILE - 1) / MTP_TILE;
    long blocks = (long)sm_count() * per_sm;
    if (blocks > tiles) blocks = tiles;
    AI2B_CUDA(launch_chained(kern, (unsigned)blocks, AT_WARPS * 32, smem, st, P, A));
    return AI2B_OK;
}

template <typename T>
int mtp_fwd_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, cudaStream_t st)
{
#define AI2B_SIG_FWD(S) return launch_fwd_atoms<T, S, false>(P, A, LossArgs<T>{}, st);
    AI2B_FOR_SIG(P, AI2B_SIG_FWD)
#undef AI2B_SIG_FWD
    set_error("no lanes-as-atoms MTP kernel for these tables");
    return AI2B_ERR_UNSUPPORTED;
}

template <typename T>
int mtp_dfwd_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, const LossArgs<T> &L, cudaStream_t st)
{
#define AI2B_SIG_DFWD(S) return launch_fwd_atoms<T, S, true>(P, A, L, st);
    AI2B_FOR_SIG(P, AI2B_SIG_DFWD)
#undef AI2B_SIG_DFWD
    set_error("no lanes-as-atoms MTP kernel for these tables");
    return AI2B_ERR_UNSUPPORTED;
}

template <typename T, int MODE>
int mtp_force_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, cudaStream_t st)
{
#define AI2B_SIG_FORCE(S) return launch_force_atoms<T, MODE, S>(P, A, st);
    AI2B_FOR_SIG(P, AI2B_SIG_FORCE)
#undef AI2B_SIG_FORCE
    set_error("no lanes-as-atoms MTP kernel for these tables");
    return AI2B_ERR_UNSUPPORTED;
}

template int mtp_fwd_atoms<float>(const MtpProgramDev &, const MtpArgs<float> &, cudaStream_t);
template int mtp_fwd_atoms<double>(const MtpProgramDev &, const MtpArgs<double> &, cudaStream_t);
template int mtp_dfwd_atoms<float>(const MtpProgramDev &, const MtpArgs<float> &, const LossArgs<float> &, cudaStream_t);
template int mtp_dfwd_atoms<double>(const MtpProgramDev &, const MtpArgs<double> &, const LossArgs<double> &, cudaStream_t);
template int mtp_force_atoms<float, MODE_EFV>(const MtpProgramDev &, const MtpArgs<float> &, cudaStream_t);
template int mtp_force_atoms<float, MODE_EF>(const MtpProgramDev &, const MtpArgs<float> &, cudaStream_t);
template int mtp_force_atoms<double, MODE_EFV>(const MtpProgramDev &, const MtpArgs<double> &, cudaStream_t);
template int mtp_force_atoms<double, MODE_EF>(const MtpProgramDev &, const MtpArgs<double> &, cudaStream_t);

}  // namespace ai2b
