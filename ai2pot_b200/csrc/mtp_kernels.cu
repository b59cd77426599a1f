// Linear MTP: energy, force, virial and descriptors on sm_100a, as three kernels per call.
//
//   mtp_fwd_kernel      one warp per atom, lanes = neighbours: r, unit vector, radial functions
//                       f_mu, dense basic-moment sums per mu (compile-time monomials + warp
//                       transpose-reduce) -> Mb[atom][dense] in the workspace
//   mtp_contract_kernel one block per tile of atoms, LANES = ATOMS: the product rows and the
//                       adjoint sweep run out of shared memory with the row tables uniform across
//                       the warp (no divergence, no per-lane table loads); site energies;
//                       adjoints of the basic moments -> Eb[atom][dense] (or the descriptors)
//   mtp_force_kernel    one warp per atom, lanes = neighbours: adjoints -> polynomial coefficient
//                       quadruples in shared memory, evaluated per neighbour with their gradient;
//                       pair force g = f' P u + f/r (G - (u.G) u); F_i += g, F_j -= g, V -= g (x) r
//
// Reference semantics: source/descriptor/mtpr/include/mtpBasis.h:400-534, linearMtp.h:190-352.
#include "mtp_device.cuh"

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

// ---- kernel C: force and virial -----------------------------------------------------------------
template <typename T, int MODE, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 4) mtp_force_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // per warp: E4[4*ndp] Ed[nbp] fr, fd[2 * MU * 32]
    T *E4 = reinterpret_cast<T *>(smem_raw) + (size_t)warp * (4 * A.ndp + A.nbp + 2 * MTP_MAX_MU * 32);
    T *Ed = E4 + 4 * A.ndp;
    T *fr = Ed + A.nbp;
    T *fdv = fr + MTP_MAX_MU * 32;

    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS, gw = blockIdx.x * MTP_WARPS + warp;
    const int chunk = (ntot + nw - 1) / nw;
    const int t0 = gw * chunk, t1 = min(ntot, t0 + chunk);

    int cur_b = -1, b_end = 0;
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

    for (int t = t0; t < t1; t++) {
        if (t >= b_end || cur_b < 0) {
            flush();
            cur_b = find_structure(A.prefix, A.B, t);
            b_end = A.prefix[cur_b + 1];
        }
        const int b = cur_b;
        const size_t slot = (size_t)b * A.npad + (t - A.prefix[b]);
        const int ci = A.bilist[slot];
        const int nn = min(A.numneigh[slot], A.umax);
        const int *types = A.types + (size_t)b * (A.npad + A.nghost);
        const int ti = types[ci];
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;

        // the first chunk of neighbours is set up before the coefficient quadruples are built: its
        // global loads (neighbour row, types, radial coefficients) overlap the loads of the adjoint row
        PairState<T, CSP, true> ps;
        ps.setup(P, A, rc, fn, types, ti, nn, lane, lane, fr, fdv);

        // adjoints of this atom -> coefficient quadruples {e, (ax+1) e[+x], (ay+1) e[+y], (az+1) e[+z]}
        const T *ein = A.Eb + (size_t)t * A.nbp;
        for (int i = lane; i < A.nbp; i += 32) Ed[i] = ein[i];
        __syncwarp();
        for (int c = lane; c < P.ndense; c += 32) {
            using V2 = typename Vec2<T>::type;
            const int4 g = P.e4g[c];
            const int mu = P.e4m[c];
            V2 lo, hi;
            lo.x = g.x >= 0 ? Ed[g.x] : T(0);
            lo.y = g.y >= 0 ? T(mu & 255) * Ed[g.y] : T(0);
            hi.x = g.z >= 0 ? T((mu >> 8) & 255) * Ed[g.z] : T(0);
            hi.y = g.w >= 0 ? T((mu >> 16) & 255) * Ed[g.w] : T(0);
            *reinterpret_cast<V2 *>(E4 + 4 * c) = lo;
            *reinterpret_cast<V2 *>(E4 + 4 * c + 2) = hi;
        }
        __syncwarp();

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
    static size_t configured = 0;
    if (int rc = set_smem(kern, smem, &configured)) return rc;
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
    A.coeffs_pad = mtp_prepare<T>(A.binum, A.B, prefix, A.coeffs, cpad, A.ntypes * A.ntypes * P.nmus, A.cs, CSP, st);
    AI2B_CUDA(cudaGetLastError());

    const long atoms_upper = (long)A.B * A.npad;
    const long need = (atoms_upper + MTP_WARPS - 1) / MTP_WARPS;
    {   // A: forward
        const size_t smem = sizeof(T) * (size_t)(A.ndp + MTP_MAX_MU * 32) * MTP_WARPS;
        auto kern = mtp_fwd_kernel<T, KD, CSP>;
        static size_t configured = 0;
        static int per_sm = 0;
        if (smem > configured || per_sm == 0) {
            if (int rc = set_smem(kern, smem, &configured)) return rc;
            AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MTP_WARPS * 32, smem));
            if (per_sm < 1) per_sm = 1;
        }
        long blocks = (long)sm_count() * per_sm;
        if (blocks > need) blocks = need;
        kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
        AI2B_CUDA(cudaGetLastError());
    }
    {   // B: products / adjoints with lanes = atoms; tile size by shared-memory footprint
        int rc = dispatch_contract<T, MODE>(P, A, atoms_upper, st);
        if (rc) return rc;
    }
    if (MODE != MODE_DESC) {   // C: forces / virial
        const size_t smem = sizeof(T) * (size_t)(4 * A.ndp + A.nbp + 2 * MTP_MAX_MU * 32) * MTP_WARPS;
        auto kern = mtp_force_kernel<T, MODE, KD, CSP>;
        static size_t configured = 0;
        static int per_sm = 0;
        if (smem > configured || per_sm == 0) {
            if (int rc = set_smem(kern, smem, &configured)) return rc;
            AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MTP_WARPS * 32, smem));
            if (per_sm < 1) per_sm = 1;
        }
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
        if (B > 0 && npad >= 0) {                                                                              \
            AI2B_CUDA(cudaMemsetAsync(etot, 0, sizeof(T) * B, st));                                            \
            AI2B_CUDA(cudaMemsetAsync(force, 0, sizeof(T) * 3 * (size_t)B * (npad + nghost), st));             \
            if (virial) AI2B_CUDA(cudaMemsetAsync(virial, 0, sizeof(T) * 9 * B, st));                          \
        }                                                                                                      \
        MtpArgs<T> A{etot, force, virial, nullptr, coeffs, lin, bias, qs, nullptr, binum, bilist, numneigh,    \
                     firstneigh, types, rcs, nullptr, nullptr, nullptr, B, npad, ntypes, umax, nghost, cs, 0, 0, \
                     scaling, rmax, rmin};                                                                     \
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
