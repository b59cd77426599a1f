// Linear MTP: energy, force, virial and descriptors on sm_100a, as three kernels per call.
//
// Tables of the reference's template levels 6 to 16 (monomial degree <= 6, four radial functions at most):
//   mtp_fwd_atoms_kernel    (mtp_atoms.cu) lanes = atoms, basic moments in registers -> Mb[tile][basic row][32 atoms]
//   mtp_contract_seg_kernel lanes = atoms, one tile of 32 atoms per block at a time: the product rows and the adjoint
//                           sweep run out of shared memory, every moment owned by one warp; site energies; adjoints
//                           of the basic moments -> Eb[tile][dense monomial][32 atoms] (or the descriptors)
//   mtp_force_atoms_kernel  (mtp_atoms.cu) lanes = atoms: polynomial of every radial function and its gradient per
//                           neighbour; pair force g = f' P u + f/r (G - (u.G) u); F_i += g, F_j -= g, V -= g (x) r
// Other tables (levels 18 and 20, or more than 32 atom types) take the warp-per-atom kernels of this file with rows per
// atom in the workspace: mtp_fwd_lanes_kernel / mtp_fwd_kernel, mtp_contract_kernel (flat row streams), mtp_force_kernel.
//
// The three lanes-as-atoms kernels are launched as a chain (launch_chained() in common.cuh): each stages its model
// tables while the kernel before it drains, then waits for it.
//
// Reference semantics: source/descriptor/mtpr/include/mtpBasis.h:400-534, linearMtp.h:190-352.
#include "mtp_device.cuh"
#include <cuda_pipeline.h>

namespace ai2b {

// ---- kernel A: dense basic-moment sums ---------------------------------------------------------
template <typename T, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 4) mtp_fwd_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T *Md = reinterpret_cast<T *>(smem_raw) + (size_t)warp * (A.ndp + MTP_MAX_MU * 32);
    T *fr = Md + A.ndp;
    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS;
    for (int t = blockIdx.x * MTP_WARPS + warp; t < ntot; t += nw) {
        const int b = find_structure(A.prefix, A.B, t);
        const size_t slot = (size_t)b * A.npad + (t - A.prefix[b]);
        const int ci = A.bilist[slot];
        const int nn = min(A.numneigh[slot], A.umax);
        // descriptor launches index types with row stride Np (linearMtp_cpu_launcher.h:284-345)
        const int *types = A.types + (size_t)b * (A.npad + (A.desc ? 0 : A.nghost));
        const int ti = types[ci];
        for (int i = lane; i < A.ndp; i += 32) Md[i] = T(0);
        __syncwarp();
        for (int j0 = 0; j0 < nn; j0 += 32) {
            PairState<T, CSP, false> ps;
            ps.setup(P, A, A.rcs + slot * A.umax * 3, A.firstneigh + slot * A.umax, types, ti, nn, j0 + lane, lane, fr, nullptr);
            Powers<T, KD> pw;
            pw.set(ps.ux, ps.uy, ps.uz);
            for (int m = 0; m < P.nmus; m++) fwd_mu<T, KD>(P.kmu[m], fr[m * 32 + lane], pw, Md + P.doff[m], lane);
        }
        __syncwarp();
        T *out = A.Mb + (size_t)t * A.nbp;
        for (int i = lane; i < A.nbp; i += 32) out[i] = i < P.nb ? Md[P.basic_dense[i]] : T(0);
        __syncwarp();
    }
}

// ---- kernel A, second form: lanes = neighbours, then lanes = monomials -------------------------------
// The sums above cost one warp transpose-reduction per moment. Here the lanes first write their
// neighbour's monomials (all of degree <= KD) to a shared-memory tile mono[neighbour][monomial]
// and its radial values f_mu to a row fr[neighbour][mu]; then they switch roles: lane l owns the
// monomials l, l + 32, ... and walks over the neighbours. In canonical order the monomials a mu
// uses are the first ncan(kmu[mu]) ones, so one monomial load serves every mu, and the f row is a
// broadcast load. No cross-lane reduction is left. Needs nmus <= NMU and kmu non-increasing.
//  * The tile holds 16 neighbours: the two half-warps store in turn (the monomials are rebuilt
//    from the 3 (KD + 1) powers, which is cheaper than a 32-neighbour tile that halves the number
//    of resident warps).
//  * The next atom's row (positions, neighbour indices, centre index, count) is requested before
//    the summation loop of the current atom, and the type look-ups that depend on it are issued
//    ahead of the radial basis, so little global-memory latency is left exposed.
// acc[r][m] += sum_jj f[jj][m] * mono[jj][q_r] for the first C_r radial functions of lane-round r
// (C_0 = NMU); the counts are template parameters so the loop body is branch- and select-free.
template <typename T, int NMU, int MS, int C1, int C2>
__device__ __forceinline__ void fwd_accumulate(const T *__restrict__ mono_s, const T *__restrict__ fh, int cnt, const int (&qidx)[3],
                                               T (&acc)[3][NMU])
{
    using V2 = typename Vec2<T>::type;
#pragma unroll 2
    for (int jj = 0; jj < cnt; jj++) {
        const T *mj = mono_s + jj * MS;
        T f[NMU];
#pragma unroll
        for (int m = 0; m < NMU; m += 2) {
            const V2 v = *reinterpret_cast<const V2 *>(fh + jj * NMU + m);
            f[m] = v.x; f[m + 1] = v.y;
        }
        const T m0 = mj[qidx[0]];
#pragma unroll
        for (int m = 0; m < NMU; m++) acc[0][m] = fma(f[m], m0, acc[0][m]);
        if constexpr (C1 > 0) {
            const T m1 = mj[qidx[1]];
#pragma unroll
            for (int m = 0; m < C1; m++) acc[1][m] = fma(f[m], m1, acc[1][m]);
        }
        if constexpr (C2 > 0) {
            const T m2 = mj[qidx[2]];
#pragma unroll
            for (int m = 0; m < C2; m++) acc[2][m] = fma(f[m], m2, acc[2][m]);
        }
    }
}

template <typename T, int KD, int CSP, int NMU>
__global__ void __launch_bounds__(MTP_WARPS * 32, 4) mtp_fwd_lanes_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    using V2 = typename Vec2<T>::type;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    constexpr int NC = ncan(KD);
    constexpr int RQ = (NC + 31) / 32;   // monomials per lane
    constexpr int MS = NC | 1;           // odd row stride: the 16 lanes' stores to one column hit distinct banks
    constexpr int TJ = 16;               // neighbours per tile
    static_assert(NMU % 2 == 0, "f rows are read as pairs");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T *mono_s = reinterpret_cast<T *>(smem_raw) + (size_t)warp * (TJ * MS + 32 * NMU);
    T *fr = mono_s + TJ * MS;            // [32 neighbours][NMU]
    static_assert(RQ == 3 && NMU == 4, "the accumulation loop is specialised for three monomials per lane");
    int qidx[RQ];
    int c1 = 0, c2 = 0;                  // radial functions that reach into the 2nd / 3rd group of 32 monomials
#pragma unroll
    for (int r = 0; r < RQ; r++) qidx[r] = min(32 * r + lane, NC - 1);
    for (int m = 0; m < P.nmus; m++) {
        c1 += ncan(P.kmu[m]) > 32 ? 1 : 0;
        c2 += ncan(P.kmu[m]) > 64 ? 1 : 0;
    }
    const int shape = c1 * 8 + c2;
    // basic-moment row of (monomial of round r, mu), -1 for none: one table per lane
    int *orow = reinterpret_cast<int *>(reinterpret_cast<T *>(smem_raw) + (size_t)MTP_WARPS * (TJ * MS + 32 * NMU)) + warp * (RQ * NMU * 32) + lane;
#pragma unroll
    for (int r = 0; r < RQ; r++)
#pragma unroll
        for (int m = 0; m < NMU; m++) {
            const int q = 32 * r + lane;
            orow[(r * NMU + m) * 32] = (m < P.nmus && q < ncan(P.kmu[m])) ? P.dense_basic[P.doff[m] + q] : -1;
        }
    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS;

    // row of an atom: what the first chunk needs, loaded without waiting for the neighbour count
    // (rows are padded to umax entries, index -1 marks padding)
    struct Row { size_t slot; int b, ci, nn, nj; T x, y, z; };
    auto fetch = [&](int t) {
        Row w;
        w.b = find_structure(A.prefix, A.B, t);
        w.slot = (size_t)w.b * A.npad + (t - A.prefix[w.b]);
        w.ci = A.bilist[w.slot];
        w.nn = A.numneigh[w.slot];
        w.nj = -1; w.x = w.y = w.z = T(0);
        if (lane < A.umax) {
            const T *rc = A.rcs + (w.slot * A.umax + lane) * 3;
            w.x = rc[0]; w.y = rc[1]; w.z = rc[2];
            w.nj = A.firstneigh[w.slot * A.umax + lane];
        }
        return w;
    };
    int t = blockIdx.x * MTP_WARPS + warp;
    // the types of the next atom and of its first 32 neighbours depend on that row: they are looked up
    // once the row has arrived (after the summation loop), one atom ahead of their use
    auto row_types = [&](const Row &w, int &ti_out, int &tj_out) {
        const int *ty = A.types + (size_t)w.b * (A.npad + (A.desc ? 0 : A.nghost));
        ti_out = ty[w.ci];
        tj_out = (lane < min(w.nn, A.umax) && w.nj >= 0) ? ty[w.nj] : 0;
    };
    Row nx;
    int nx_ti = 0, nx_tj = 0;
    if (t < ntot) { nx = fetch(t); row_types(nx, nx_ti, nx_tj); }
    for (; t < ntot; t += nw) {
        const Row cur = nx;
        const int nn = min(cur.nn, A.umax);
        const int *types = A.types + (size_t)cur.b * (A.npad + (A.desc ? 0 : A.nghost));
        const int ti = nx_ti, tj_first = nx_tj;
        T acc[RQ][NMU];
#pragma unroll
        for (int r = 0; r < RQ; r++)
#pragma unroll
            for (int m = 0; m < NMU; m++) acc[r][m] = T(0);
        for (int j0 = 0; j0 < nn; j0 += 32) {
            const int j = j0 + lane;
            T x = cur.x, y = cur.y, z = cur.z;
            int nj = cur.nj;
            if (j0 > 0) {
                x = y = z = T(0); nj = -1;
                if (j < nn) {
                    const T *rc = A.rcs + (cur.slot * A.umax + j) * 3;
                    x = rc[0]; y = rc[1]; z = rc[2];
                    nj = A.firstneigh[cur.slot * A.umax + j];
                }
            }
            bool act = j < nn && nj >= 0;
            const int tj = j0 == 0 ? tj_first : (act ? types[nj] : 0);
            const T r = gsqrt(x * x + y * y + z * z);
            act = act && (r <= A.rmax) && (r > T(0));
            const T rinv = act ? T(1) / r : T(0);
            {
                T q[CSP], dq[CSP], fv[NMU];
                mtp_radial_basis<T, CSP>(act ? r : A.rmax, A.rmax, A.rmin, A.scaling, q, dq);
                const T *crow = A.coeffs_pad + (size_t)(ti * A.ntypes + tj) * P.nmus * CSP;
#pragma unroll
                for (int m = 0; m < NMU; m++) {
                    T f = T(0);
                    if (m < P.nmus) {
#pragma unroll
                        for (int k = 0; k < CSP; k += 2) {
                            const V2 c2 = *reinterpret_cast<const V2 *>(crow + m * CSP + k);
                            f = fma(c2.x, q[k], f);
                            f = fma(c2.y, q[k + 1], f);
                        }
                    }
                    fv[m] = act ? f : T(0);
                }
#pragma unroll
                for (int m = 0; m < NMU; m += 2) {
                    V2 v; v.x = fv[m]; v.y = fv[m + 1];
                    *reinterpret_cast<V2 *>(fr + lane * NMU + m) = v;
                }
            }
            Powers<T, KD> pw;
            pw.set(x * rinv, y * rinv, z * rinv);
            const int left = nn - j0;   // neighbours in this chunk (may exceed 32)
#pragma unroll 1
            for (int h = 0; h < 2; h++) {
                if (h * TJ >= left) break;
                if ((lane >> 4) == h) {
                    T *mrow = mono_s + (lane & 15) * MS;
                    static_for<0, KD + 1>([&](auto dd) {
                        constexpr int D = decltype(dd)::value;
                        static_for<0, ndeg(D)>([&](auto qq) {
                            constexpr int Q = decltype(qq)::value;
                            mrow[ncan(D - 1) + Q] = mono<T, KD, D, Q>(pw);
                        });
                    });
                }
                __syncwarp();
                if (h == 0 && j0 == 0 && t + nw < ntot) nx = fetch(t + nw);   // lands during the loop below
                const int cnt = min(TJ, left - h * TJ);
                const T *fh = fr + h * TJ * NMU;
                switch (shape) {   // kmu is non-increasing, so c2 <= c1
#define AI2B_ACC(C1, C2) case C1 * 8 + C2: fwd_accumulate<T, NMU, MS, C1, C2>(mono_s, fh, cnt, qidx, acc); break;
                    AI2B_ACC(0, 0)
                    AI2B_ACC(1, 0) AI2B_ACC(1, 1)
                    AI2B_ACC(2, 0) AI2B_ACC(2, 1) AI2B_ACC(2, 2)
                    AI2B_ACC(3, 0) AI2B_ACC(3, 1) AI2B_ACC(3, 2) AI2B_ACC(3, 3)
                    AI2B_ACC(4, 0) AI2B_ACC(4, 1) AI2B_ACC(4, 2) AI2B_ACC(4, 3) AI2B_ACC(4, 4)
#undef AI2B_ACC
                    default: break;
                }
                __syncwarp();
            }
        }
        if (nn <= 0 && t + nw < ntot) nx = fetch(t + nw);
        if (t + nw < ntot) row_types(nx, nx_ti, nx_tj);
        T *out = A.Mb + (size_t)t * A.nbp;
#pragma unroll
        for (int r = 0; r < RQ; r++)
#pragma unroll
            for (int m = 0; m < NMU; m++) {
                const int row = orow[(r * NMU + m) * 32];
                if (row >= 0) out[row] = acc[r][m];
            }
        for (int i = P.nb + lane; i < A.nbp; i += 32) out[i] = T(0);
    }
}

// ---- kernel B: products and adjoint sweep, lanes = atoms ----------------------------------------
// TA atoms per tile (32, 16 or 8); with TA < 32 the 32/TA lane groups of a warp work on different
// rows. Shared memory: M[nm][TA+1] and (unless DESC) E[nm][TA+1], then the row tables.
// Persistent: one block per SM walks over tiles; the row tables are staged once, and the next
// tile's moment rows are fetched into registers while the current tile is being processed, so
// no global-memory latency sits between two tiles.
constexpr int MTP_PREF = 8;   // prefetch registers per thread: basic moments <= 32 * MTP_PREF

template <typename T, int TA, int MODE, bool SMEMTAB>
__global__ void __launch_bounds__(MTP_CWARPS * 32, 1) mtp_contract_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    extern __shared__ __align__(32) unsigned char smem_raw[];
    constexpr int LD = TA + 1;
    constexpr int G = 32 / TA;
    constexpr int NWORK = MTP_CWARPS * G;
    __shared__ T esum[NWORK][TA];
    T *M = reinterpret_cast<T *>(smem_raw);
    T *E = M + (size_t)P.nm * LD;
    const size_t arr_bytes = (sizeof(T) * (size_t)P.nm * LD * (MODE == MODE_DESC ? 1 : 2) + 15) & ~size_t(15);
    int2 *s_fwd = reinterpret_cast<int2 *>(smem_raw + arr_bytes);
    int2 *s_rev = s_fwd + P.nt;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int a = lane % TA, wid = warp * G + lane / TA;
    const T *Ma = M + a, *Ea = E + a;
    const int ntot = A.prefix[A.B];
    const int ntiles = (ntot + TA - 1) / TA;
    const int nthreads = MTP_CWARPS * 32;
    if ((int)blockIdx.x >= ntiles) return;

    // row tables, staged once, with the moment indices already scaled to element offsets (index * LD fits 16 bits)
    auto scale = [](int2 r) {
        return make_int2(((r.x & 0xffff) * LD) | (((r.x >> 16) & 0xffff) * LD) << 16, (r.y & 0xffff) | (((r.y >> 16) & 0xffff) * LD) << 16);
    };
    if (SMEMTAB) {
#pragma unroll 4
        for (int i = threadIdx.x; i < P.nt; i += nthreads) s_fwd[i] = scale(P.fwd_flat[i]);
        if (MODE != MODE_DESC)
#pragma unroll 4
            for (int i = threadIdx.x; i < 2 * P.nt; i += nthreads) s_rev[i] = scale(P.rev_flat[i]);
    }
    // large tables (template levels above 16) stay in global memory
    auto frow = [&](int r) { return SMEMTAB ? s_fwd[r] : scale(P.fwd_flat[r]); };
    auto rrow = [&](int r) { return SMEMTAB ? s_rev[r] : scale(P.rev_flat[r]); };

    // moment rows of a tile: warp w fetches atom w (and w + nwarps, ..), lanes run over the row
    const bool can_prefetch = P.nb <= 32 * MTP_PREF && TA <= MTP_CWARPS;
    T pre[MTP_PREF];
    auto fetch = [&](int tile) {
#pragma unroll
        for (int k = 0; k < MTP_PREF; k++) {
            const int i = lane + 32 * k, t = tile * TA + warp;
            pre[k] = (warp < TA && t < ntot && i < P.nb) ? A.Mb[(size_t)t * A.nbp + i] : T(0);
        }
    };
    if (can_prefetch) fetch(blockIdx.x);

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int t0 = tile * TA;
        for (int i = threadIdx.x; i < P.nm * LD; i += nthreads) {
            M[i] = T(0);
            if (MODE != MODE_DESC) E[i] = T(0);
        }
        __syncthreads();
        if (can_prefetch) {
            if (warp < TA) {
#pragma unroll
                for (int k = 0; k < MTP_PREF; k++) {
                    const int i = lane + 32 * k;
                    if (i < P.nb) M[i * LD + warp] = pre[k];
                }
            }
            if (tile + (int)gridDim.x < ntiles) fetch(tile + gridDim.x);   // in flight during this tile
        } else {
            for (int at = warp; at < TA && t0 + at < ntot; at += MTP_CWARPS) {
                const T *src = A.Mb + (size_t)(t0 + at) * A.nbp;
                for (int i = lane; i < P.nb; i += 32) M[i * LD + at] = src[i];
            }
        }
        __syncthreads();

        // product rows: every depth's rows are one contiguous stream; each worker takes an equal share
        // of it and adds a destination's partial sum when the stream leaves that destination
        // (shared-memory atomic add: a destination may straddle two workers)
        for (int lev = 0; lev < P.nlev; lev++) {
            const int R0 = P.fwd_lev_row[lev], len = P.fwd_lev_row[lev + 1] - R0;
            const int rb = R0 + (int)((long)len * wid / NWORK), re = R0 + (int)((long)len * (wid + 1) / NWORK);
            T acc = T(0);
#pragma unroll 4
            for (int r = rb; r < re; r++) {
                const int2 row = frow(r);
                acc = fma(T(row.y & 0xff) * Ma[row.x & 0xffff], Ma[(unsigned)row.x >> 16], acc);
                if ((row.y & 0x100) || r == re - 1) {
                    atomicAdd(M + ((unsigned)row.y >> 16) + a, acc);
                    acc = T(0);
                }
            }
            __syncthreads();
        }

        // per-atom bookkeeping (all lanes of a column agree)
        const int t = t0 + a;
        const bool valid = t < ntot;
        int b = 0;
        size_t slot = 0;
        if (valid) {
            b = find_structure(A.prefix, A.B, t);
            slot = (size_t)b * A.npad + (t - A.prefix[b]);
        }

        if (MODE == MODE_DESC) {
            if (valid)
                for (int s = wid; s < P.ns; s += NWORK) A.desc[slot * P.ns + s] = M[P.map[s] * LD + a];
            __syncthreads();
            continue;
        }

        // site energy and adjoint seeds (linearMtp.h:281-295)
        T es = T(0);
#pragma unroll 4
        for (int s = wid; s < P.ns; s += NWORK) {
            const int m = P.map[s];
            const T w = A.lin[s] / A.qs[s];
            es = fma(w, M[m * LD + a], es);
            E[m * LD + a] = w;
        }
        esum[wid][a] = es;
        __syncthreads();
        if (wid == 0) {
            T e = T(0);
#pragma unroll
            for (int k = 0; k < NWORK; k++) e += esum[k][a];
            if (valid) {
                const int *types = A.types + (size_t)b * (A.npad + A.nghost);
                e += A.bias[types[A.bilist[slot]]];
            } else {
                e = T(0);
            }
            // one atomic per structure present in these TA atoms. Every lane of the group walks all TA
            // lanes (a fixed trip count: the shuffles must be executed by the whole group together)
            const unsigned grp = (TA == 32) ? FULL_MASK : (((1u << TA) - 1u) << (lane / TA * TA));
            const int base = lane / TA * TA;
            const int key = valid ? b : -1;
            T tot = T(0);
            int leader = TA;
            for (int k = 0; k < TA; k++) {
                const T ek = __shfl_sync(grp, e, base + k);
                const int bk = __shfl_sync(grp, key, base + k);
                if (bk == key) { tot += ek; leader = min(leader, k); }
            }
            if (valid && a == leader) atomicAdd(A.etot + b, tot);
        }

        // adjoint sweep, deepest sources first: E[source] += sum mult E[dst] M[other]
        for (int k = 0; k < P.nlev; k++) {
            const int R0 = P.rev_lev_row[k], len = P.rev_lev_row[k + 1] - R0;
            const int rb = R0 + (int)((long)len * wid / NWORK), re = R0 + (int)((long)len * (wid + 1) / NWORK);
            T acc = T(0);
#pragma unroll 4
            for (int r = rb; r < re; r++) {
                const int2 row = rrow(r);
                acc = fma(T(row.y & 0xff) * Ea[(unsigned)row.x >> 16], Ma[row.x & 0xffff], acc);
                if ((row.y & 0x100) || r == re - 1) {
                    atomicAdd(E + ((unsigned)row.y >> 16) + a, acc);
                    acc = T(0);
                }
            }
            __syncthreads();
        }

        // adjoints of the basic moments, back to per-atom rows
        for (int at = warp; at < TA && t0 + at < ntot; at += MTP_CWARPS) {
            T *dstp = A.Eb + (size_t)(t0 + at) * A.nbp;
            for (int i = lane; i < A.nbp; i += 32) dstp[i] = i < P.nb ? E[i * LD + at] : T(0);
        }
        __syncthreads();
    }
}


// ---- kernel B, segment form: lanes = atoms, one worker (warp) owns a moment ------------------------
// The flat-stream kernel above spends ~30 instructions around the two FP64 instructions of a product row
// (offset unpacking, multiplier conversion, flag test, shared-memory atomic flush). Here the tables are
// compiled into segments (mtp_program.cuh): a header {moment, row count, multiplier} followed by rows of
// two element offsets, every moment owned by one warp, so a row is one 8-byte broadcast load, two address
// adds, two operand loads and one FMA, and a moment is finished with a plain store. Tiles of 32 atoms;
// the workspace holds them tile by tile ([tile][row][32 atoms]; per-atom rows from the warp-per-atom forward
// kernels are transposed on the way in and out, row stride 33 keeps those accesses spread over the banks),
// the next tile's rows travelling in registers while the current tile is processed.
// Shared memory: M[nm][33], E[nm][33] (not for descriptors), headers, rows, seeds, worker tables.
constexpr int MTP_SEG_EWARPS = 8;   // warps that sum the site energies of a tile
template <typename T>
struct SegSmem {
    T *M, *E, *seed, *wsc;     // wsc[s] = lin[s] / q[s]; seed[m] = sum of wsc over the scalars mapped to moment m
    int *mapo;                 // element offset of the moment of scalar s
    T *ep;                     // [MTP_SEG_EWARPS][33] partial site energies
    int *db;                   // [ndense] element offset of the basic moment of dense index d (-1: none)
    int4 *hdr;
    int2 *row;
    int *wseg, *wrow;
};
template <typename T, int MODE>
__host__ __device__ inline size_t seg_smem_layout(const MtpProgramDev &P, unsigned char *base, SegSmem<T> *out)
{
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t r = o; o += (bytes + 15) & ~size_t(15); return r; };
    const size_t oM = take(sizeof(T) * (size_t)P.nm * MTP_SEG_LD);
    const size_t oE = MODE == MODE_DESC ? oM : take(sizeof(T) * (size_t)P.nm * MTP_SEG_LD);
    const size_t oh = take(sizeof(int4) * (size_t)P.nseg);
    const size_t orow = take(sizeof(int2) * (size_t)P.nseg_rows);
    const size_t os = take(sizeof(T) * (size_t)P.nm);
    const size_t osc = take(sizeof(T) * (size_t)P.ns);
    const size_t omo = take(sizeof(int) * (size_t)P.ns);
    const size_t oep = take(MODE == MODE_DESC ? 0 : sizeof(T) * MTP_SEG_EWARPS * MTP_SEG_LD);
    const size_t odb = take(MODE == MODE_DESC ? 0 : sizeof(int) * (size_t)P.ndense);
    const size_t ow = take(sizeof(int) * (size_t)(2 * P.nlev) * (MTP_SEG_WORKERS + 1));
    const size_t owr = take(sizeof(int) * (size_t)(2 * P.nlev) * MTP_SEG_WORKERS);
    if (out) {
        out->M = reinterpret_cast<T *>(base + oM); out->E = reinterpret_cast<T *>(base + oE);
        out->hdr = reinterpret_cast<int4 *>(base + oh); out->row = reinterpret_cast<int2 *>(base + orow);
        out->seed = reinterpret_cast<T *>(base + os); out->wsc = reinterpret_cast<T *>(base + osc);
        out->wseg = reinterpret_cast<int *>(base + ow); out->wrow = reinterpret_cast<int *>(base + owr);
        out->mapo = reinterpret_cast<int *>(base + omo);
        out->ep = reinterpret_cast<T *>(base + oep);
        out->db = reinterpret_cast<int *>(base + odb);
    }
    return o;
}

// Shared-memory accesses of the row loop, by 32-bit shared-window address (explicit ld.shared / st.shared: the
// loop is bound by instruction issue and shared-memory bandwidth, so it must not fall back to generic addressing).
__device__ __forceinline__ int2 lds_int2(unsigned a)
{
    int2 v;
    asm volatile("ld.shared.v2.s32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ int4 lds_int4(unsigned a)
{
    int4 v;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ double lds_val(unsigned a, double)
{
    double v;
    asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_val(unsigned a, float)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_val(unsigned a, double v) { asm volatile("st.shared.f64 [%0], %1;" ::"r"(a), "d"(v) : "memory"); }
__device__ __forceinline__ void sts_val(unsigned a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }

// one phase for one worker. xl, yl = shared addresses of this lane's column of the arrays a row's first / second
// offset refers to, dl = of the destination array; hdr, row, seed = shared addresses of the tables
template <typename T, bool SEEDED>
__device__ __forceinline__ void seg_phase(int h, int hend, unsigned hdr, unsigned rp, unsigned seed, unsigned xl, unsigned yl, unsigned dl)
{
    constexpr unsigned ES = (unsigned)sizeof(T);
    T dsum = T(0);
    for (; h < hend; h++) {
        // a worker's rows follow one another across its segments, so the first two row records are requested together
        // with the header (they are simply not used if the segment is shorter), and inside a segment the next pair is
        // requested before the current pair's products are formed
        const int4 hd = lds_int4(hdr + 16u * (unsigned)h);
        int2 r0 = lds_int2(rp), r1 = lds_int2(rp + 8u);
        const int n = hd.y & 0x3fffffff;
        T acc0 = T(0), acc1 = T(0);
        const unsigned rend = rp + 8u * (unsigned)n;
#pragma unroll 1
        while (rp + 8u < rend) {
            const T x0 = lds_val(xl + (unsigned)r0.x * ES, T()), y0 = lds_val(yl + (unsigned)r0.y * ES, T());
            const T x1 = lds_val(xl + (unsigned)r1.x * ES, T()), y1 = lds_val(yl + (unsigned)r1.y * ES, T());
            rp += 16u;
            r0 = lds_int2(rp); r1 = lds_int2(rp + 8u);
            acc0 = fma(x0, y0, acc0);
            acc1 = fma(x1, y1, acc1);
        }
        if (rp < rend) {
            acc0 = fma(lds_val(xl + (unsigned)r0.x * ES, T()), lds_val(yl + (unsigned)r0.y * ES, T()), acc0);
            rp += 8u;
        }
        const T mult = (T)__hiloint2double(hd.w, hd.z);
        const T acc = acc0 + acc1;
        dsum = (hd.y & (1 << 30)) ? mult * acc : fma(mult, acc, dsum);
        if (hd.y < 0) {                                  // bit 31: last segment of the moment
            T out = dsum;
            if (SEEDED) out += lds_val(seed + (unsigned)(hd.x / MTP_SEG_LD) * ES, T());
            sts_val(dl + (unsigned)hd.x * ES, out);
        }
    }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(MTP_SEG_WORKERS * 32, 1) mtp_contract_seg_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NT = MTP_SEG_WORKERS * 32;
    SegSmem<T> S;
    seg_smem_layout<T, MODE>(P, smem_raw, &S);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    chain_release();
    const int ntot = total_atoms(A);
    const int ntiles = (ntot + MTP_TILE - 1) / MTP_TILE;
    if ((int)blockIdx.x >= ntiles) {
        chain_wait();        // every block waits, so that this kernel never completes before the one it follows
        return;
    }

    // tables, staged once per block
    for (int i = threadIdx.x; i < P.nseg; i += NT) S.hdr[i] = P.seg_hdr[i];
    for (int i = threadIdx.x; i < P.nseg_rows; i += NT) S.row[i] = P.seg_row[i];
    for (int i = threadIdx.x; i < 2 * P.nlev * (MTP_SEG_WORKERS + 1); i += NT) S.wseg[i] = P.seg_wseg[i];
    for (int i = threadIdx.x; i < 2 * P.nlev * MTP_SEG_WORKERS; i += NT) S.wrow[i] = P.seg_wrow[i];
    if (MODE != MODE_DESC) {
        for (int i = threadIdx.x; i < P.nm; i += NT) S.seed[i] = T(0);
        __syncthreads();
        // adjoint seeds lin[s] / q[s] (linearMtp.h:292-295); a moment may serve several scalars
        for (int s = threadIdx.x; s < P.ns; s += NT) {
            const T w = A.lin[s] / A.qs[s];
            const int m = P.map[s];
            S.wsc[s] = w;
            S.mapo[s] = m * MTP_SEG_LD;
            atomicAdd(S.seed + m, w);
        }
        for (int d = threadIdx.x; d < P.ndense; d += NT) {
            const int r = P.dense_basic[d];
            S.db[d] = r >= 0 ? r * MTP_SEG_LD : -1;
        }
    } else {
        for (int s = threadIdx.x; s < P.ns; s += NT) S.mapo[s] = P.map[s] * MTP_SEG_LD;
    }

    // basic-moment rows of a tile: warp w fetches atom w, lanes run over the row; fetched one tile ahead
    const bool can_prefetch = P.nb <= 32 * MTP_PREF;
    T pre[MTP_PREF];
    // (tiled workspace: warp w fetches the rows w, w + 32, ... of the tile, lanes run over its atoms)
    auto fetch = [&](int tile) {
#pragma unroll
        for (int k = 0; k < MTP_PREF; k++) {
            if (A.tiled) {
                const int i = warp + 32 * k;
                pre[k] = i < P.nb ? A.Mb[((size_t)tile * A.nbp + i) * MTP_TILE + lane] : T(0);
            } else {
                const int i = lane + 32 * k, t = tile * MTP_TILE + warp;
                pre[k] = (t < ntot && i < P.nb) ? A.Mb[(size_t)t * A.nbp + i] : T(0);
            }
        }
    };
    chain_wait();        // everything above reads the program's tables and the model only
    if (can_prefetch) fetch(blockIdx.x);
    // shared-window addresses of this lane's columns and of the tables
    const unsigned ml = (unsigned)__cvta_generic_to_shared(S.M + lane), el = (unsigned)__cvta_generic_to_shared(S.E + lane);
    const unsigned a_hdr = (unsigned)__cvta_generic_to_shared(S.hdr), a_row = (unsigned)__cvta_generic_to_shared(S.row),
                   a_seed = (unsigned)__cvta_generic_to_shared(S.seed);
    auto run_phase = [&](int p, auto seeded, unsigned xl, unsigned yl, unsigned dl) {
        const int h = S.wseg[p * (MTP_SEG_WORKERS + 1) + warp], hend = S.wseg[p * (MTP_SEG_WORKERS + 1) + warp + 1];
        seg_phase<T, decltype(seeded)::value>(h, hend, a_hdr, a_row + 8u * (unsigned)S.wrow[p * MTP_SEG_WORKERS + warp], a_seed, xl, yl, dl);
    };

    __syncthreads();         // tables staged
    if (MODE != MODE_DESC) {
        // moments no product reads: their adjoint is their seed for every atom of every tile, written once
        for (int i = warp; i < P.nseg_init; i += MTP_SEG_WORKERS) {
            const int m = P.seg_init[i];
            S.E[m * MTP_SEG_LD + lane] = S.seed[m];
        }
    }
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        // (no barrier here: the last adjoint phase ended with one, after which the moments are no longer read, and the
        // adjoint array is not written again before the barrier that follows the product phases)
        if (can_prefetch) {
#pragma unroll
            for (int k = 0; k < MTP_PREF; k++) {
                const int i = (A.tiled ? warp : lane) + 32 * k;
                if (i < P.nb) S.M[i * MTP_SEG_LD + (A.tiled ? lane : warp)] = pre[k];
            }
            if (tile + (int)gridDim.x < ntiles) fetch(tile + gridDim.x);   // in flight during this tile
        } else if (A.tiled) {
            const T *src = A.Mb + (size_t)tile * A.nbp * MTP_TILE + lane;
            for (int i = warp; i < P.nb; i += MTP_SEG_WORKERS) S.M[i * MTP_SEG_LD + lane] = src[(size_t)i * MTP_TILE];
        } else {
            const int t = tile * MTP_TILE + warp;
            const T *src = A.Mb + (size_t)t * A.nbp;
            for (int i = lane; i < P.nb; i += 32) S.M[i * MTP_SEG_LD + warp] = t < ntot ? src[i] : T(0);
        }
        __syncthreads();

        // per-atom bookkeeping (lane = atom of the tile): its loads are in flight during the product phases
        const int t = tile * MTP_TILE + lane;
        const bool valid = t < ntot;
        int b = 0;
        size_t slot = 0;
        T ebias = T(0);
        if (valid) {
            if (A.B > 1) {
                b = find_structure(A.prefix, A.B, t);
                slot = (size_t)b * A.npad + (t - A.prefix[b]);
            } else {
                slot = (size_t)t;
            }
            if (MODE != MODE_DESC && warp == 0) {
                const int *types = A.types + (size_t)b * (A.npad + A.nghost);
                ebias = A.bias[types[A.bilist[slot]]];
            }
        }

        for (int p = 0; p < P.nlev; p++) {
            run_phase(p, std::false_type{}, ml, ml, ml);
            // The sources of the deepest adjoint level feed only products of the last level, whose adjoints are their
            // seeds: that level reads nothing the last product level writes and follows it without a barrier.
            if (MODE != MODE_DESC && p == P.nlev - 1) run_phase(P.nlev, std::true_type{}, el, ml, el);
            __syncthreads();
        }

        if (MODE == MODE_DESC) {
            if (valid)
                for (int s = warp; s < P.ns; s += MTP_SEG_WORKERS) A.desc[slot * P.ns + s] = S.M[S.mapo[s] + lane];
            __syncthreads();     // the moments are overwritten by the next tile
            continue;
        }

        // site energies (linearMtp.h:281-289) by the first MTP_SEG_EWARPS warps, which meet at a barrier of their own;
        // the other warps go on to the adjoints (they read the moments and write the adjoint array only)
        if (warp < MTP_SEG_EWARPS) {
            T es = T(0);
            for (int s = warp; s < P.ns; s += MTP_SEG_EWARPS) es = fma(S.wsc[s], S.M[S.mapo[s] + lane], es);
            S.ep[warp * MTP_SEG_LD + lane] = es;
            asm volatile("bar.sync 1, %0;" ::"n"(MTP_SEG_EWARPS * 32) : "memory");
            if (warp == 0) {
                T e = ebias;
#pragma unroll
                for (int k = 0; k < MTP_SEG_EWARPS; k++) e += S.ep[k * MTP_SEG_LD + lane];
                if (!valid) e = T(0);
                // one atomic per structure present in these 32 atoms
                const int key = valid ? b : -1;
                const int key0 = __shfl_sync(FULL_MASK, key, 0);
                if (__all_sync(FULL_MASK, key == key0 || key < 0)) {      // one structure: a plain warp sum
                    const T tot = warp_sum(e);
                    if (lane == 0 && key0 >= 0) atomicAdd(A.etot + key0, tot);
                } else {
                    T tot = T(0);
                    int leader = MTP_TILE;
                    for (int k = 0; k < MTP_TILE; k++) {
                        const T ek = __shfl_sync(FULL_MASK, e, k);
                        const int bk = __shfl_sync(FULL_MASK, key, k);
                        if (bk == key) { tot += ek; leader = min(leader, k); }
                    }
                    if (valid && lane == leader) atomicAdd(A.etot + b, tot);
                }
            }
        }
        // the other adjoint levels, deepest sources first: E[src] = seed + sum mult E[dst] M[other]
        for (int p = P.nlev + 1; p < 2 * P.nlev; p++) {
            run_phase(p, std::true_type{}, el, ml, el);
            __syncthreads();
        }
        if (P.nlev < 2) __syncthreads();     // the energy warps still read the moments the next tile overwrites
        // adjoints of the basic moments: whole rows of the tile, or back to per-atom rows (warp w writes atom w)
        if (A.tiled) {      // in dense monomial order, the order the force kernel evaluates its polynomials in
            T *dstp = A.Eb + (size_t)tile * A.ndp * MTP_TILE + lane;
            for (int d = warp; d < P.ndense; d += MTP_SEG_WORKERS) {
                const int o = S.db[d];
                dstp[(size_t)d * MTP_TILE] = o >= 0 ? S.E[o + lane] : T(0);
            }
        } else {
            const int t = tile * MTP_TILE + warp;
            if (t < ntot) {
                T *dstp = A.Eb + (size_t)t * A.nbp;
                for (int i = lane; i < A.nbp; i += 32) dstp[i] = i < P.nb ? S.E[i * MTP_SEG_LD + warp] : T(0);
            }
        }
    }
}

// ---- kernel C: force and virial -----------------------------------------------------------------
// shared-memory elements (of T) per warp: E4[4 ndp] Ed[nbp + 4] fr, fd[2 nmus 32] row buffer [96 + 36 ints]
template <typename T>
__host__ __device__ inline size_t force_warp_elems(int ndp, int nbp, int nmus)
{
    return (size_t)4 * ndp + nbp + 4 + 2 * nmus * 32 + 96 + 36 * sizeof(int) / sizeof(T);
}

template <typename T, int MODE, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 3) mtp_force_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    using V2 = typename Vec2<T>::type;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // block: gather table of the coefficient quadruples, s_g[ndp] (basic rows of {value, d/dx, d/dy,
    // d/dz}; "none" points at a zero slot) and s_m[ndp][4] (their multipliers, already of type T)
    // per warp: see force_warp_elems
    int4 *s_g = reinterpret_cast<int4 *>(smem_raw);
    T *s_m = reinterpret_cast<T *>(smem_raw + sizeof(int4) * A.ndp);
    T *E4 = s_m + 4 * A.ndp + (size_t)warp * force_warp_elems<T>(A.ndp, A.nbp, P.nmus);
    T *Ed = E4 + 4 * A.ndp;
    T *fr = Ed + A.nbp + 4;
    T *fdv = fr + P.nmus * 32;
    T *rb_rc = fdv + P.nmus * 32;                           // [32][3] positions of the first 32 neighbours
    int *rb_fn = reinterpret_cast<int *>(rb_rc + 96);       // [32] their indices, then centre index and count
    for (int c = threadIdx.x; c < P.ndense; c += blockDim.x) {
        int4 g = P.e4g[c];
        const int mu = P.e4m[c];
        g.x = g.x >= 0 ? g.x : A.nbp; g.y = g.y >= 0 ? g.y : A.nbp;
        g.z = g.z >= 0 ? g.z : A.nbp; g.w = g.w >= 0 ? g.w : A.nbp;
        s_g[c] = g;
        s_m[4 * c] = T(1); s_m[4 * c + 1] = T(mu & 255); s_m[4 * c + 2] = T((mu >> 8) & 255); s_m[4 * c + 3] = T((mu >> 16) & 255);
    }
    if (lane < 4) Ed[A.nbp + lane] = T(0);
    __syncthreads();

    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS, gw = blockIdx.x * MTP_WARPS + warp;
    const int chunk = (ntot + nw - 1) / nw;
    const int t0 = gw * chunk, t1 = min(ntot, t0 + chunk);

    int cur_b = -1;
    T vir[9];
#pragma unroll
    for (int k = 0; k < 9; k++) vir[k] = T(0);
    auto flush = [&]() {
        if (cur_b < 0 || MODE != MODE_EFV) return;
#pragma unroll
        for (int k = 0; k < 9; k++) {
            T s = warp_sum(vir[k]);
            if (lane == 0) atomicAdd(A.virial + 9 * cur_b + k, s);
            vir[k] = T(0);
        }
    };

    // The row of the next atom (positions and indices of its first 32 neighbours, centre index,
    // count) and its adjoints are copied into shared memory asynchronously while the current atom
    // is evaluated: no registers are held, and the copies need not wait for the count because rows
    // are padded to umax entries.
    int fb = -1, fb_end = 0, row_b = 0;
    size_t row_slot = 0;
    auto request = [&](int t) {
        if (t >= fb_end || fb < 0) { fb = find_structure(A.prefix, A.B, t); fb_end = A.prefix[fb + 1]; }
        row_b = fb;
        row_slot = (size_t)fb * A.npad + (t - A.prefix[fb]);
        if (lane < A.umax) {
            const T *src = A.rcs + (row_slot * A.umax + lane) * 3;
#pragma unroll
            for (int k = 0; k < 3; k++) __pipeline_memcpy_async(rb_rc + 3 * lane + k, src + k, sizeof(T));
            __pipeline_memcpy_async(rb_fn + lane, A.firstneigh + row_slot * A.umax + lane, sizeof(int));
        }
        if (lane == 0) __pipeline_memcpy_async(rb_fn + 32, A.bilist + row_slot, sizeof(int));
        if (lane == 1) __pipeline_memcpy_async(rb_fn + 33, A.numneigh + row_slot, sizeof(int));
        const T *ein = A.Eb + (size_t)t * A.nbp;
        for (int i = lane; i < A.nbp; i += 32) __pipeline_memcpy_async(Ed + i, ein + i, sizeof(T));
        __pipeline_commit();
    };
    // types of the next atom and of its first 32 neighbours: looked up from the arrived row one atom ahead
    int nx_ti = 0, nx_tj = 0;
    auto row_types = [&]() {
        __pipeline_wait_prior(0);
        __syncwarp();
        const int *ty = A.types + (size_t)row_b * (A.npad + A.nghost);
        nx_ti = ty[rb_fn[32]];
        nx_tj = lane < min(rb_fn[33], A.umax) ? ty[rb_fn[lane]] : 0;
    };
    if (t0 < t1) { request(t0); row_types(); }

    for (int t = t0; t < t1; t++) {
        if (row_b != cur_b) {
            flush();
            cur_b = row_b;
        }
        const int b = cur_b;
        const size_t slot = row_slot;
        const int ci = rb_fn[32];
        const int nn = min(rb_fn[33], A.umax);
        const int *types = A.types + (size_t)b * (A.npad + A.nghost);
        const int ti = nx_ti;
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;

        PairState<T, CSP, true> ps;
        ps.act = lane < nn;
        ps.x = ps.y = ps.z = T(0); ps.nj = 0;
        if (ps.act) { ps.x = rb_rc[3 * lane]; ps.y = rb_rc[3 * lane + 1]; ps.z = rb_rc[3 * lane + 2]; ps.nj = rb_fn[lane]; }
        ps.compute(P, A, types, ti, lane, fr, fdv, 32, ps.act ? nx_tj : 0);

        // adjoints -> coefficient quadruples {e, (ax+1) e[+x], (ay+1) e[+y], (az+1) e[+z]}
        for (int c = lane; c < P.ndense; c += 32) {
            const int4 g = s_g[c];
            const V2 m01 = *reinterpret_cast<const V2 *>(s_m + 4 * c), m23 = *reinterpret_cast<const V2 *>(s_m + 4 * c + 2);
            V2 lo, hi;
            lo.x = Ed[g.x];
            lo.y = m01.y * Ed[g.y];
            hi.x = m23.x * Ed[g.z];
            hi.y = m23.y * Ed[g.w];
            *reinterpret_cast<V2 *>(E4 + 4 * c) = lo;
            *reinterpret_cast<V2 *>(E4 + 4 * c + 2) = hi;
        }
        __syncwarp();
        if (t + 1 < t1) request(t + 1);   // lands while this atom is evaluated

        T *frc = A.force + (size_t)b * (A.npad + A.nghost) * 3;
        T fcx = T(0), fcy = T(0), fcz = T(0);
        for (int j0 = 0; j0 < nn; j0 += 32) {
            if (j0 > 0) ps.setup(P, A, rc, fn, types, ti, nn, j0 + lane, lane, fr, fdv);
            Powers<T, KD> pw;
            pw.set(ps.ux, ps.uy, ps.uz);
            T gx = T(0), gy = T(0), gz = T(0);
            for (int m = 0; m < P.nmus; m++) {
                T Pv = T(0), Gx = T(0), Gy = T(0), Gz = T(0);
                eval_mu<T, KD>(P.kmu[m], E4 + 4 * P.doff[m], pw, Pv, Gx, Gy, Gz);
                const T f = fr[m * 32 + lane], fd = fdv[m * 32 + lane];
                const T ug = ps.ux * Gx + ps.uy * Gy + ps.uz * Gz;
                const T aa = fd * Pv - f * ps.rinv * ug, cc = f * ps.rinv;
                gx += aa * ps.ux + cc * Gx;
                gy += aa * ps.uy + cc * Gy;
                gz += aa * ps.uz + cc * Gz;
            }
            if (ps.act) {
                fcx += gx; fcy += gy; fcz += gz;
                atomicAdd(frc + 3 * ps.nj + 0, -gx);
                atomicAdd(frc + 3 * ps.nj + 1, -gy);
                atomicAdd(frc + 3 * ps.nj + 2, -gz);
                if (MODE == MODE_EFV) {
                    vir[0] -= gx * ps.x; vir[1] -= gx * ps.y; vir[2] -= gx * ps.z;
                    vir[3] -= gy * ps.x; vir[4] -= gy * ps.y; vir[5] -= gy * ps.z;
                    vir[6] -= gz * ps.x; vir[7] -= gz * ps.y; vir[8] -= gz * ps.z;
                }
            }
        }
        if (t + 1 < t1) row_types();   // the next row has arrived during the evaluation
        fcx = warp_sum(fcx); fcy = warp_sum(fcy); fcz = warp_sum(fcz);
        if (lane == 0) {
            atomicAdd(frc + 3 * ci + 0, fcx);
            atomicAdd(frc + 3 * ci + 1, fcy);
            atomicAdd(frc + 3 * ci + 2, fcz);
        }
        __syncwarp();
    }
    flush();
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <typename T, int MODE>
static size_t contract_smem(const MtpProgramDev &P, int ta, bool tables)
{
    const size_t arrays = sizeof(T) * (size_t)P.nm * (ta + 1) * (MODE == MODE_DESC ? 1 : 2);
    const size_t tab = tables ? sizeof(int2) * (size_t)P.nt * (MODE == MODE_DESC ? 1 : 3) : 0;
    return ((arrays + 15) & ~size_t(15)) + tab + 16;
}

template <typename T, int TA, int MODE, bool SMEMTAB>
static int launch_contract(const MtpProgramDev &P, const MtpArgs<T> &A, long atoms_upper, cudaStream_t st)
{
    const size_t smem = contract_smem<T, MODE>(P, TA, SMEMTAB);
    auto kern = mtp_contract_kernel<T, TA, MODE, SMEMTAB>;
    static KernelSetup setup;
    if (int rc = kernel_setup(setup, kern, smem)) return rc;
    long tiles = (atoms_upper + TA - 1) / TA;
    if (tiles > sm_count()) tiles = sm_count();      // persistent: one block per SM walks over the tiles
    kern<<<(unsigned)tiles, MTP_CWARPS * 32, smem, st>>>(P, A);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

// largest tile (and shared-memory row tables if they fit too) within the 227 KiB opt-in limit;
// moment offsets are packed as index * (TA + 1) in 16 bits
template <typename T, int MODE>
static int dispatch_contract(const MtpProgramDev &P, const MtpArgs<T> &A, long atoms_upper, cudaStream_t st)
{
    const size_t cap = 222 * 1024;
    {   // segment form: whole tables and a tile of 32 atoms in shared memory
        const size_t smem = seg_smem_layout<T, MODE>(P, nullptr, nullptr);
        if (smem <= 226 * 1024 && P.nseg > 0) {
            auto kern = mtp_contract_seg_kernel<T, MODE>;
            static KernelSetup setup;
            if (int rc = kernel_setup(setup, kern, smem)) return rc;
            long tiles = (atoms_upper + MTP_TILE - 1) / MTP_TILE;
            if (tiles > sm_count()) tiles = sm_count();      // persistent: one block per SM walks over the tiles
            AI2B_CUDA(launch_chained(kern, (unsigned)tiles, MTP_SEG_WORKERS * 32, smem, st, P, A));
            return AI2B_OK;
        }
    }
#define AI2B_TRY(TA_)                                                                                       \
    if ((long)P.nm * (TA_ + 1) <= 65535) {                                                                  \
        if (contract_smem<T, MODE>(P, TA_, true) <= cap) return launch_contract<T, TA_, MODE, true>(P, A, atoms_upper, st);   \
        if (contract_smem<T, MODE>(P, TA_, false) <= cap) return launch_contract<T, TA_, MODE, false>(P, A, atoms_upper, st); \
    }
    AI2B_TRY(32) AI2B_TRY(16) AI2B_TRY(8)
#undef AI2B_TRY
    set_error("MTP tables with %d moments do not fit the contraction kernel's shared memory", P.nm);
    return AI2B_ERR_UNSUPPORTED;
}

template <typename T, int MODE, int KD, int CSP>
static int launch_mtp_v(const ai2b_mtp_program *prog, MtpArgs<T> A, void *ws, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    const MtpWs L = mtp_ws_layout(P, A.B, A.npad, A.ntypes, sizeof(T));
    unsigned char *w = reinterpret_cast<unsigned char *>(ws);
    int *prefix = reinterpret_cast<int *>(w + L.prefix);
    T *cpad = reinterpret_cast<T *>(w + L.cpad);
    A.prefix = prefix;
    A.coeffs_pad = cpad;
    A.Mb = reinterpret_cast<T *>(w + L.mb);
    A.Eb = reinterpret_cast<T *>(w + L.eb);
    A.ndp = ndense_pad(P);
    A.nbp = nbasic_pad(P);
    MtpZero<T> Z;
    if (A.zero_outputs) {
        Z.p[0] = A.etot; Z.n[0] = (size_t)A.B;
        Z.p[1] = A.force; Z.n[1] = 3 * (size_t)A.B * (A.npad + A.nghost);
        if (A.virial) { Z.p[2] = A.virial; Z.n[2] = 9 * (size_t)A.B; }
    }
    // lanes-as-atoms forward and force kernels around the segment contraction, where all three apply
    bool atoms_path = false;
    if constexpr (KD <= 6 && CSP == 8)
        atoms_path = mtp_atoms_supported(P, A.ntypes, A.cs, sizeof(T), (long)A.npad + A.nghost) && P.nseg > 0 &&
                     seg_smem_layout<T, MODE>(P, nullptr, nullptr) <= 226 * 1024;
    const bool need_pad = A.cs != CSP || (reinterpret_cast<size_t>(A.coeffs) % (2 * sizeof(T))) != 0;
    if (atoms_path && A.B == 1 && !need_pad) {
        // one structure, coefficient rows usable as they are: no set-up launch; the forward kernel zeroes the outputs
        A.coeffs_pad = A.coeffs;
        if (A.zero_outputs) A.zero_outputs = 2;
    } else {
        A.coeffs_pad = mtp_prepare<T>(A.binum, A.B, prefix, A.coeffs, cpad, A.ntypes * A.ntypes * P.nmus, A.cs, CSP, st, Z);
        AI2B_CUDA(cudaGetLastError());
    }

    const long atoms_upper = (long)A.B * A.npad;
    const long need = (atoms_upper + MTP_WARPS - 1) / MTP_WARPS;
    bool fwd_done = false;
    if (atoms_path) {
        A.tiled = 1;
        if (int rc = mtp_fwd_atoms<T>(P, A, st)) return rc;
        fwd_done = true;
    }
    if constexpr (KD <= 6) if (!fwd_done) {   // A: forward with lanes = monomials in the summation
        constexpr int NMU = 4;
        bool ok = P.nmus <= NMU;
        for (int m = 1; m < P.nmus; m++) ok = ok && P.kmu[m] <= P.kmu[m - 1];
        if (ok) {
            const size_t smem = (sizeof(T) * (size_t)(16 * (ncan(KD) | 1) + 32 * NMU) + sizeof(int) * 3 * NMU * 32) * MTP_WARPS;
            auto kern = mtp_fwd_lanes_kernel<T, KD, CSP, NMU>;
            static KernelSetup setup;
            int per_sm = 1;
            if (int rc = kernel_setup(setup, kern, smem, MTP_WARPS * 32, &per_sm)) return rc;
            long blocks = (long)sm_count() * per_sm;
            if (blocks > need) blocks = need;
            kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
            AI2B_CUDA(cudaGetLastError());
            fwd_done = true;
        }
    }
    if (!fwd_done) {   // A: forward with warp reductions (levels 18, 20)
        const size_t smem = sizeof(T) * (size_t)(A.ndp + MTP_MAX_MU * 32) * MTP_WARPS;
        auto kern = mtp_fwd_kernel<T, KD, CSP>;
        static KernelSetup setup;
        int per_sm = 1;
        if (int rc = kernel_setup(setup, kern, smem, MTP_WARPS * 32, &per_sm)) return rc;
        long blocks = (long)sm_count() * per_sm;
        if (blocks > need) blocks = need;
        kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
        AI2B_CUDA(cudaGetLastError());
    }
    {   // B: products / adjoints with lanes = atoms; tile size by shared-memory footprint
        int rc = dispatch_contract<T, MODE>(P, A, atoms_upper, st);
        if (rc) return rc;
    }
    if constexpr (MODE != MODE_DESC) {
        if (atoms_path) return mtp_force_atoms<T, MODE>(P, A, st);
    }
    if (MODE != MODE_DESC) {   // C: forces / virial
        const size_t smem = sizeof(int4) * A.ndp + sizeof(T) * 4 * A.ndp +
                            sizeof(T) * force_warp_elems<T>(A.ndp, A.nbp, P.nmus) * MTP_WARPS;
        auto kern = mtp_force_kernel<T, MODE, KD, CSP>;
        static KernelSetup setup;
        int per_sm = 1;
        if (int rc = kernel_setup(setup, kern, smem, MTP_WARPS * 32, &per_sm)) return rc;
        long blocks = (long)sm_count() * per_sm;
        if (blocks > need) blocks = need;
        kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
        AI2B_CUDA(cudaGetLastError());
    }
    return AI2B_OK;
}

template <typename T, int MODE>
static int launch_mtp(const ai2b_mtp_program *prog, MtpArgs<T> A, void *ws, size_t ws_bytes, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    AI2B_REQUIRE(A.cs >= 1 && A.cs <= 16, AI2B_ERR_UNSUPPORTED, "chebyshev_size %d outside 1..16", A.cs);
    AI2B_REQUIRE(A.B >= 0 && A.npad >= 0 && A.umax >= 0 && A.ntypes >= 1 && A.nghost >= 0, AI2B_ERR_INVALID, "negative size");
    if (A.B == 0 || A.npad == 0) return AI2B_OK;
    const size_t need = mtp_ws_layout(P, A.B, A.npad, A.ntypes, sizeof(T)).total;
    AI2B_REQUIRE(ws && ws_bytes >= need, AI2B_ERR_WORKSPACE, "MTP workspace too small: %zu < %zu bytes", ws_bytes, need);
    // fast variant: monomial degree <= 6 (template level <= 16) and <= 8 radial basis functions
    if (P.kmax <= 6 && A.cs <= 8) return launch_mtp_v<T, MODE, 6, 8>(prog, A, ws, st);
    return launch_mtp_v<T, MODE, 8, 16>(prog, A, ws, st);
}

}  // namespace ai2b

using namespace ai2b;

extern "C" size_t ai2b_mtp_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int natoms_pad, int ntypes)
{
    if (!prog) return 0;
    return mtp_ws_layout(prog->dev, batch_size, natoms_pad, ntypes > 0 ? ntypes : 1, sizeof(double)).total;
}

#define AI2B_DEF_MTP(SUF, T)                                                                                   \
    extern "C" int ai2b_mtp_efv_##SUF(const ai2b_mtp_program *prog, T *etot, T *force, T *virial, int cs,      \
                                      T scaling, const T *coeffs, const T *lin, const T *bias, int B, int npad, \
                                      const int *binum, const int *bilist, const int *numneigh,                \
                                      const int *firstneigh, const T *rcs, const int *types, int ntypes,       \
                                      int umax, int nghost, T rmax, T rmin, const T *qs, void *ws,             \
                                      size_t ws_bytes, void *stream)                                           \
    {                                                                                                          \
        AI2B_REQUIRE(prog && etot && force && coeffs && lin && bias && qs && binum && bilist && numneigh &&    \
                         firstneigh && rcs && types, AI2B_ERR_INVALID, "ai2b_mtp_efv: NULL argument");         \
        cudaStream_t st = (cudaStream_t)stream;                                                                \
        if (B > 0 && npad == 0) {   /* no atoms: the kernels are not launched */                               \
            AI2B_CUDA(cudaMemsetAsync(etot, 0, sizeof(T) * B, st));                                            \
            AI2B_CUDA(cudaMemsetAsync(force, 0, sizeof(T) * 3 * (size_t)B * (npad + nghost), st));             \
            if (virial) AI2B_CUDA(cudaMemsetAsync(virial, 0, sizeof(T) * 9 * B, st));                          \
        }                                                                                                      \
        MtpArgs<T> A{etot, force, virial, nullptr, coeffs, lin, bias, qs, nullptr, binum, bilist, numneigh,    \
                     firstneigh, types, rcs, nullptr, nullptr, nullptr, B, npad, ntypes, umax, nghost, cs, 0, 0, \
                     scaling, rmax, rmin};                                                                     \
        A.zero_outputs = 1;                                                                                    \
        return virial ? launch_mtp<T, MODE_EFV>(prog, A, ws, ws_bytes, st)                                     \
                      : launch_mtp<T, MODE_EF>(prog, A, ws, ws_bytes, st);                                     \
    }                                                                                                          \
    extern "C" int ai2b_mtp_descriptors_##SUF(const ai2b_mtp_program *prog, T *desc, int cs, T scaling,        \
                                              const T *coeffs, int B, int npad, const int *binum,              \
                                              const int *bilist, const int *numneigh, const int *firstneigh,   \
                                              const T *rcs, const int *types, int ntypes, int umax,            \
                                              int nghost, T rmax, T rmin, void *ws, size_t ws_bytes,           \
                                              void *stream)                                                    \
    {                                                                                                          \
        AI2B_REQUIRE(prog && desc && coeffs && binum && bilist && numneigh && firstneigh && rcs && types,      \
                     AI2B_ERR_INVALID, "ai2b_mtp_descriptors: NULL argument");                                 \
        cudaStream_t st = (cudaStream_t)stream;                                                                \
        if (B > 0 && npad > 0)                                                                                 \
            AI2B_CUDA(cudaMemsetAsync(desc, 0, sizeof(T) * (size_t)B * npad * prog->dev.ns, st));              \
        MtpArgs<T> A{nullptr, nullptr, nullptr, desc, coeffs, nullptr, nullptr, nullptr, nullptr, binum,       \
                     bilist, numneigh, firstneigh, types, rcs, nullptr, nullptr, nullptr, B, npad, ntypes,     \
                     umax, nghost, cs, 0, 0, scaling, rmax, rmin};                                             \
        return launch_mtp<T, MODE_DESC>(prog, A, ws, ws_bytes, st);                                            \
    }

AI2B_DEF_MTP(f64, double)
AI2B_DEF_MTP(f32, float)
