// Linear MTP training path: per-structure loss and its analytic gradient w.r.t. the radial
// coefficients, the linear coefficients and the type bias.
//
// Reference: source/descriptor/mtpr/include/linearMtpLoss.h:138-210 (loss), :212-569 (gradient),
// batch loops linearMtpLoss_cpu_launcher.h:152-533, RMSEs src/linearMtpOp.cc:885-911.
//
// With dF = F_ml - F_dft, dV = V_ml - V_dft, dE = E_ml - E_dft of the atom's structure (n atoms):
//   p(i,j)   = 2 f_w/(3n) (dF_i - dF_j) - 2 v_w/(9n) dV r_ij            (one vector per pair)
//   D_m      = sum_j p . dM_m/dr_j           directional derivative of every moment (forward mode)
//   E_m      = dE_site/dM_m                  adjoint, as in the force path
//   G_m      = second-order adjoint: sum over product rows of E_dst D_other, pushed back through
//              the product rows
//   dL/dc[ti,tj,mu,xi] += sum_pairs Q_xi (X_mu(u) + p_perp . grad Ebar_mu(u) / r) + Q'_xi (p.u) Ebar_mu(u)
//              with the polynomials Ebar_mu = sum_a E_a u^a, X_mu = sum_a (2 e_w/n dE E_a + G_a) u^a
//   dL/dlin[s]  += (2 e_w/n dE M_map(s) + D_map(s)) / q[s],     dL/dbias[ti] += 2 e_w/n dE
// Three kernels, as in the force path: per-atom forward (lanes = neighbours) producing the basic
// moments and their directional derivatives, a tile kernel with lanes = atoms for all product-row
// sweeps, and a per-atom kernel that evaluates the two polynomials per neighbour and reduces the
// coefficient gradient over the lanes of each neighbour type.
#include "mtp_device.cuh"

namespace ai2b {

// ---- loss and squared-error sums ---------------------------------------------------------------
// one block per structure; se[0..2] accumulate sum dE^2 (of the energy per atom if e_per_atom: the NEP ops'
// definition, nepLoss_cpu_launcher.h:300-345), sum dF^2, sum dV^2, se[3] the atom count
template <typename T>
__global__ void mtp_loss_kernel(T *__restrict__ loss, T *__restrict__ se, int e_per_atom, int npad, int nghost, const int *__restrict__ binum,
                                const int *__restrict__ bilist, T ew, T fw, T vw, const T *__restrict__ e_ml,
                                const T *__restrict__ e_dft, const T *__restrict__ f_ml, const T *__restrict__ f_dft,
                                const T *__restrict__ v_ml, const T *__restrict__ v_dft)
{
    __shared__ T sh[32];
    const int b = blockIdx.x, n = binum[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T fs = T(0);
    for (int k = threadIdx.x; k < 3 * n; k += blockDim.x) {
        const int ii = k / 3, a = k - 3 * ii;
        const int ci = bilist[(size_t)b * npad + ii];
        const T d = f_ml[((size_t)b * (npad + nghost) + ci) * 3 + a] - f_dft[((size_t)b * npad + ci) * 3 + a];
        fs = fma(d, d, fs);
    }
    fs = warp_sum(fs);
    if (lane == 0) sh[warp] = fs;
    __syncthreads();
    if (threadIdx.x == 0) {
        T f2 = T(0);
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) f2 += sh[w];
        T v2 = T(0);
        if (v_ml)
            for (int k = 0; k < 9; k++) { const T d = v_ml[9 * b + k] - v_dft[9 * b + k]; v2 = fma(d, d, v2); }
        const T de = e_ml[b] - e_dft[b];
        T l = fw / T(3 * n) * f2 + ew / T(n) * de * de;
        if (v_ml) l += vw / T(9 * n) * v2;
        loss[b] = n > 0 ? l : T(0);
        atomicAdd(se + 0, e_per_atom ? (n > 0 ? (de / T(n)) * (de / T(n)) : T(0)) : de * de);
        atomicAdd(se + 1, f2);
        atomicAdd(se + 2, v2);
        atomicAdd(se + 3, T(n));
    }
}
template <typename T>
__global__ void mtp_rmse_kernel(T *__restrict__ rmse, const T *__restrict__ se, int B)
{
    if (threadIdx.x == 0) {
        rmse[0] = sqrt(se[0] / T(B));
        rmse[1] = sqrt(se[1] / (T(3) * se[3]));
        rmse[2] = sqrt(se[2] / T(9 * B));
    }
}

// value and directional derivative of the degree-D monomial sums:
//   accM[q] += sum_lanes f mono_q
//   accD[q] += sum_lanes ( a mono_q + bx ax mono(q - ex) + by ay mono(q - ey) + bz az mono(q - ez) )
template <typename T, int KD, int D>
__device__ __forceinline__ void fwd2_degree(T f, T a, T bx, T by, T bz, const Powers<T, KD> &p, T *accM, T *accD, int lane)
{
    constexpr int ND = ndeg(D);
    constexpr int GS = 16;
    static_for<0, (ND + GS - 1) / GS>([&](auto g) {
        constexpr int G = decltype(g)::value;
        constexpr int CNT = (ND - GS * G) < GS ? (ND - GS * G) : GS;
        constexpr int N = pow2ceil(CNT);
        T v[N], w[N];
        static_for<0, N>([&](auto i) {
            constexpr int I = decltype(i)::value;
            if constexpr (I < CNT) {
                constexpr Exp3 e = deg_exp(D, GS * G + I);
                const T m = mono<T, KD, D, GS * G + I>(p);
                v[I] = f * m;
                T d = a * m;
                if constexpr (e.x > 0) d = fma(bx * T(e.x), p.x[e.x - 1] * p.y[e.y] * p.z[e.z], d);
                if constexpr (e.y > 0) d = fma(by * T(e.y), p.x[e.x] * p.y[e.y - 1] * p.z[e.z], d);
                if constexpr (e.z > 0) d = fma(bz * T(e.z), p.x[e.x] * p.y[e.y] * p.z[e.z - 1], d);
                w[I] = d;
            } else {
                v[I] = T(0);
                w[I] = T(0);
            }
        });
        const T rv = warp_xreduce<T, N>(v, lane);
        const T rw = warp_xreduce<T, N>(w, lane);
        constexpr int SH = 5 - ilog2(N);
        const int idx = lane >> SH;
        if ((lane & ((1 << SH) - 1)) == 0 && idx < CNT) {
            accM[GS * G + idx] += rv;
            accD[GS * G + idx] += rw;
        }
    });
}
template <typename T, int KD>
__device__ __forceinline__ void fwd2_mu(int kmu, T f, T a, T bx, T by, T bz, const Powers<T, KD> &p, T *accM, T *accD, int lane)
{
#define AI2B_FWD2_DEG(D)                                                                          \
    if constexpr (D <= KD) {                                                                      \
        if (kmu < D) return;                                                                      \
        fwd2_degree<T, KD, D>(f, a, bx, by, bz, p, accM + ncan(D - 1), accD + ncan(D - 1), lane); \
    }
    AI2B_FWD2_DEG(0) AI2B_FWD2_DEG(1) AI2B_FWD2_DEG(2) AI2B_FWD2_DEG(3) AI2B_FWD2_DEG(4)
    AI2B_FWD2_DEG(5) AI2B_FWD2_DEG(6) AI2B_FWD2_DEG(7) AI2B_FWD2_DEG(8)
#undef AI2B_FWD2_DEG
}

// polynomial value only: P += sum x[q] mono_q
template <typename T, int KD>
__device__ __forceinline__ void value_mu(int kmu, const T *__restrict__ x, const Powers<T, KD> &p, T &P)
{
#define AI2B_VAL_DEG(D)                                                                        \
    if constexpr (D <= KD) {                                                                   \
        if (kmu < D) return;                                                                   \
        static_for<0, ndeg(D)>([&](auto qq) {                                                  \
            constexpr int Q = decltype(qq)::value;                                             \
            P = fma(x[ncan(D - 1) + Q], mono<T, KD, D, Q>(p), P);                              \
        });                                                                                    \
    }
    AI2B_VAL_DEG(0) AI2B_VAL_DEG(1) AI2B_VAL_DEG(2) AI2B_VAL_DEG(3) AI2B_VAL_DEG(4)
    AI2B_VAL_DEG(5) AI2B_VAL_DEG(6) AI2B_VAL_DEG(7) AI2B_VAL_DEG(8)
#undef AI2B_VAL_DEG
}

// ---- kernel A': basic moments and their directional derivatives ----------------------------------
template <typename T, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 3) mtp_loss_fwd_kernel(const MtpProgramDev P, const MtpArgs<T> A, const LossArgs<T> L)
{
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T *Md = reinterpret_cast<T *>(smem_raw) + (size_t)warp * (2 * A.ndp + 2 * MTP_MAX_MU * 32);
    T *Dd = Md + A.ndp;
    T *fr = Dd + A.ndp;
    T *fdv = fr + MTP_MAX_MU * 32;
    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS;
    for (int t = blockIdx.x * MTP_WARPS + warp; t < ntot; t += nw) {
        const int b = find_structure(A.prefix, A.B, t);
        const size_t slot = (size_t)b * A.npad + (t - A.prefix[b]);
        const int ci = A.bilist[slot], n = A.binum[b];
        const int nn = min(A.numneigh[slot], A.umax);
        const int *types = A.types + (size_t)b * (A.npad + A.nghost);
        const int ti = types[ci];
        for (int i = lane; i < 2 * A.ndp; i += 32) Md[i] = T(0);
        __syncwarp();
        for (int j0 = 0; j0 < nn; j0 += 32) {
            PairState<T, CSP, true> ps;
            ps.setup(P, A, A.rcs + slot * A.umax * 3, A.firstneigh + slot * A.umax, types, ti, nn, j0 + lane, lane, fr, fdv);
            T px = 0, py = 0, pz = 0;
            if (ps.act) pair_weight(A, L, b, n, ci, ps.nj, ps.x, ps.y, ps.z, px, py, pz);
            const T ppar = px * ps.ux + py * ps.uy + pz * ps.uz;
            const T qx = (px - ppar * ps.ux) * ps.rinv, qy = (py - ppar * ps.uy) * ps.rinv, qz = (pz - ppar * ps.uz) * ps.rinv;
            Powers<T, KD> pw;
            pw.set(ps.ux, ps.uy, ps.uz);
            for (int m = 0; m < P.nmus; m++) {
                const T f = fr[m * 32 + lane], fd = fdv[m * 32 + lane];
                fwd2_mu<T, KD>(P.kmu[m], f, fd * ppar, f * qx, f * qy, f * qz, pw, Md + P.doff[m], Dd + P.doff[m], lane);
            }
        }
        __syncwarp();
        T *om = A.Mb + (size_t)t * A.nbp, *od = L.Db + (size_t)t * A.nbp;
        for (int i = lane; i < A.nbp; i += 32) {
            const int d = i < P.nb ? P.basic_dense[i] : -1;
            om[i] = d >= 0 ? Md[d] : T(0);
            od[i] = d >= 0 ? Dd[d] : T(0);
        }
        __syncwarp();
    }
}

// ---- kernel B': all product-row sweeps, lanes = atoms ----------------------------------------------
template <typename T, int TA, bool SMEMTAB>
__global__ void __launch_bounds__(MTP_CWARPS * 32, 1) mtp_loss_contract_kernel(const MtpProgramDev P, const MtpArgs<T> A, const LossArgs<T> L)
{
    extern __shared__ __align__(32) unsigned char smem_raw[];
    constexpr int LD = TA + 1;
    constexpr int G = 32 / TA;
    constexpr int NWORK = MTP_CWARPS * G;
    const size_t narr = (size_t)P.nm * LD;
    T *M = reinterpret_cast<T *>(smem_raw);
    T *D = M + narr, *E = D + narr, *Gm = E + narr;
    const size_t arr_bytes = (sizeof(T) * 4 * narr + 15) & ~size_t(15);
    int2 *s_fwd = reinterpret_cast<int2 *>(smem_raw + arr_bytes);
    int2 *s_rev = s_fwd + P.nt;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int a = lane % TA, wid = warp * G + lane / TA;
    const T *Ma = M + a, *Da = D + a, *Ea = E + a, *Ga = Gm + a;
    const int ntot = A.prefix[A.B];
    const int t0 = blockIdx.x * TA;
    if (t0 >= ntot) return;
    const int nthreads = MTP_CWARPS * 32;

    for (int i = threadIdx.x; i < 4 * (int)narr; i += nthreads) M[i] = T(0);
    auto scale = [](int2 r) { return make_int2(((r.x & 0xffff) * LD) | (((r.x >> 16) & 0xffff) * LD) << 16, r.y); };
    if (SMEMTAB) {
#pragma unroll 4
        for (int i = threadIdx.x; i < P.nt; i += nthreads) s_fwd[i] = scale(P.fwd_rows[i]);
#pragma unroll 4
        for (int i = threadIdx.x; i < 2 * P.nt; i += nthreads) s_rev[i] = scale(P.rev_ents[i]);
    }
    auto frow = [&](int r) { return SMEMTAB ? s_fwd[r] : scale(P.fwd_rows[r]); };
    auto rrow = [&](int r) { return SMEMTAB ? s_rev[r] : scale(P.rev_ents[r]); };
    __syncthreads();
#pragma unroll 4
    for (int idx = threadIdx.x; idx < TA * A.nbp; idx += nthreads) {
        const int at = idx / A.nbp, i = idx - at * A.nbp;
        if (i < P.nb && t0 + at < ntot) {
            const int t = t0 + at;
            // rows per atom, or [tile of 32 atoms][row][32]
            const size_t src = A.tiled ? ((size_t)(t >> 5) * A.nbp + i) * 32 + (t & 31) : (size_t)t * A.nbp + i;
            M[i * LD + at] = A.Mb[src];
            D[i * LD + at] = L.Db[src];
        }
    }
    __syncthreads();

    // products with their directional derivative (linearMtpLoss.h:391-398)
    for (int lev = 0; lev < P.nlev; lev++) {
        const int dend = P.fwd_lev_off[lev + 1];
        int d = P.fwd_lev_off[lev] + wid;
        int4 nxt = d < dend ? P.fwd_dst[d] : make_int4(0, 0, 0, 0);
        for (; d < dend; d += NWORK) {
            const int4 ds = nxt;
            if (d + NWORK < dend) nxt = P.fwd_dst[d + NWORK];
            T am0 = T(0), am1 = T(0), ad0 = T(0), ad1 = T(0);
            int r = ds.y;
            for (; r + 1 < ds.z; r += 2) {
                const int2 r0 = frow(r), r1 = frow(r + 1);
                const unsigned a0 = r0.x & 0xffff, b0 = (unsigned)r0.x >> 16, a1 = r1.x & 0xffff, b1 = (unsigned)r1.x >> 16;
                const T m0 = T(__int_as_float(r0.y)), m1 = T(__int_as_float(r1.y));
                const T xa0 = m0 * Ma[a0], xb0 = Ma[b0], xa1 = m1 * Ma[a1], xb1 = Ma[b1];
                am0 = fma(xa0, xb0, am0);
                am1 = fma(xa1, xb1, am1);
                ad0 = fma(m0 * Da[a0], xb0, fma(xa0, Da[b0], ad0));
                ad1 = fma(m1 * Da[a1], xb1, fma(xa1, Da[b1], ad1));
            }
            if (r < ds.z) {
                const int2 r0 = frow(r);
                const unsigned a0 = r0.x & 0xffff, b0 = (unsigned)r0.x >> 16;
                const T m0 = T(__int_as_float(r0.y));
                const T xa0 = m0 * Ma[a0], xb0 = Ma[b0];
                am0 = fma(xa0, xb0, am0);
                ad0 = fma(m0 * Da[a0], xb0, fma(xa0, Da[b0], ad0));
            }
            M[ds.x * LD + a] += am0 + am1;
            D[ds.x * LD + a] += ad0 + ad1;
        }
        __syncthreads();
    }

    for (int s = wid; s < P.ns; s += NWORK) E[P.map[s] * LD + a] = A.lin[s] / A.qs[s];
    __syncthreads();

    // first-order adjoint E (deepest sources first), and the direct part of the second-order
    // adjoint: G_m = sum mult E_dst D_other (needs E final, so it runs as its own pass below)
    for (int k = 0; k < P.nlev; k++) {
        const int dend = P.rev_lev_off[k + 1];
        int d = P.rev_lev_off[k] + wid;
        int4 nxt = d < dend ? P.rev_mom[d] : make_int4(0, 0, 0, 0);
        for (; d < dend; d += NWORK) {
            const int4 ms = nxt;
            if (d + NWORK < dend) nxt = P.rev_mom[d + NWORK];
            T acc0 = T(0), acc1 = T(0);
            int e = ms.y;
            for (; e + 1 < ms.z; e += 2) {
                const int2 r0 = rrow(e), r1 = rrow(e + 1);
                acc0 = fma(T(__int_as_float(r0.y)) * Ea[(unsigned)r0.x >> 16], Ma[r0.x & 0xffff], acc0);
                acc1 = fma(T(__int_as_float(r1.y)) * Ea[(unsigned)r1.x >> 16], Ma[r1.x & 0xffff], acc1);
            }
            if (e < ms.z) {
                const int2 r0 = rrow(e);
                acc0 = fma(T(__int_as_float(r0.y)) * Ea[(unsigned)r0.x >> 16], Ma[r0.x & 0xffff], acc0);
            }
            E[ms.x * LD + a] += acc0 + acc1;
        }
        __syncthreads();
    }
    {   // G, direct part (linearMtpLoss.h:417-423): every source moment, any order
        const int dend = P.rev_lev_off[P.nlev];
        for (int d = wid; d < dend; d += NWORK) {
            const int4 ms = P.rev_mom[d];
            T acc0 = T(0), acc1 = T(0);
            int e = ms.y;
            for (; e + 1 < ms.z; e += 2) {
                const int2 r0 = rrow(e), r1 = rrow(e + 1);
                acc0 = fma(T(__int_as_float(r0.y)) * Ea[(unsigned)r0.x >> 16], Da[r0.x & 0xffff], acc0);
                acc1 = fma(T(__int_as_float(r1.y)) * Ea[(unsigned)r1.x >> 16], Da[r1.x & 0xffff], acc1);
            }
            if (e < ms.z) {
                const int2 r0 = rrow(e);
                acc0 = fma(T(__int_as_float(r0.y)) * Ea[(unsigned)r0.x >> 16], Da[r0.x & 0xffff], acc0);
            }
            Gm[ms.x * LD + a] = acc0 + acc1;
        }
        __syncthreads();
    }
    // G pushed back through the product rows (linearMtpLoss.h:425-434), deepest sources first
    for (int k = 0; k < P.nlev; k++) {
        const int dend = P.rev_lev_off[k + 1];
        for (int d = P.rev_lev_off[k] + wid; d < dend; d += NWORK) {
            const int4 ms = P.rev_mom[d];
            T acc0 = T(0), acc1 = T(0);
            int e = ms.y;
            for (; e + 1 < ms.z; e += 2) {
                const int2 r0 = rrow(e), r1 = rrow(e + 1);
                acc0 = fma(T(__int_as_float(r0.y)) * Ga[(unsigned)r0.x >> 16], Ma[r0.x & 0xffff], acc0);
                acc1 = fma(T(__int_as_float(r1.y)) * Ga[(unsigned)r1.x >> 16], Ma[r1.x & 0xffff], acc1);
            }
            if (e < ms.z) {
                const int2 r0 = rrow(e);
                acc0 = fma(T(__int_as_float(r0.y)) * Ga[(unsigned)r0.x >> 16], Ma[r0.x & 0xffff], acc0);
            }
            Gm[ms.x * LD + a] += acc0 + acc1;
        }
        __syncthreads();
    }

    // per-atom bookkeeping
    const int t = t0 + a;
    const bool valid = t < ntot;
    int b = 0, ti = 0;
    T ce = T(0);
    if (valid) {
        b = find_structure(A.prefix, A.B, t);
        const size_t slot = (size_t)b * A.npad + (t - A.prefix[b]);
        ti = (A.types + (size_t)b * (A.npad + A.nghost))[A.bilist[slot]];
        ce = T(2) * L.ew / T(A.binum[b]) * (L.e_ml[b] - L.e_dft[b]);
    }
    // rows for the coefficient kernel: E and X = ce E + G of the basic moments
    for (int i = wid; i < P.nb; i += NWORK) {
        if (valid) {
            A.Eb[(size_t)t * A.nbp + i] = Ea[i * LD];
            L.Xb[(size_t)t * A.nbp + i] = fma(ce, Ea[i * LD], Ga[i * LD]);
        }
    }
    // gradients w.r.t. the linear coefficients and the type bias: one atomic per (structure, entry)
    // present among the TA atoms of a lane group (fixed-trip shuffles: the whole group takes part)
    const unsigned grp = (TA == 32) ? FULL_MASK : (((1u << TA) - 1u) << (lane / TA * TA));
    const int base = lane / TA * TA;
    auto group_add = [&](T val, int key, T *dst) {
        T tot = T(0);
        int leader = TA;
        for (int k = 0; k < TA; k++) {
            const T vk = __shfl_sync(grp, val, base + k);
            const int kk = __shfl_sync(grp, key, base + k);
            if (kk == key) { tot += vk; leader = min(leader, k); }
        }
        if (key >= 0 && a == leader) atomicAdd(dst, tot);
    };
    for (int s = wid; s < P.ns; s += NWORK) {
        const int m = P.map[s];
        const T val = valid ? (ce * Ma[m * LD] + Da[m * LD]) / A.qs[s] : T(0);
        group_add(val, valid ? b : -1, L.dlinear + (size_t)b * P.ns + s);
    }
    if (wid == 0) group_add(ce, valid ? b * A.ntypes + ti : -1, L.dbias + (size_t)b * A.ntypes + ti);
}

// ---- kernel C': gradient w.r.t. the radial coefficients -------------------------------------------
template <typename T, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 3) mtp_loss_coeff_kernel(const MtpProgramDev P, const MtpArgs<T> A, const LossArgs<T> L)
{
    using V2 = typename Vec2<T>::type;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // per warp: E4[4 ndp] X1[ndp] Ed[nbp] Xd[nbp] am, bm[2 * MU * 32]
    T *E4 = reinterpret_cast<T *>(smem_raw) + (size_t)warp * (5 * A.ndp + 2 * A.nbp + 2 * MTP_MAX_MU * 32);
    T *X1 = E4 + 4 * A.ndp;
    T *Ed = X1 + A.ndp;
    T *Xd = Ed + A.nbp;
    T *am = Xd + A.nbp;
    T *bm = am + MTP_MAX_MU * 32;
    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS;
    const int nval = P.nmus * CSP;   // values per neighbour type: (mu, xi)

    for (int t = blockIdx.x * MTP_WARPS + warp; t < ntot; t += nw) {
        const int b = find_structure(A.prefix, A.B, t);
        const size_t slot = (size_t)b * A.npad + (t - A.prefix[b]);
        const int ci = A.bilist[slot], n = A.binum[b];
        const int nn = min(A.numneigh[slot], A.umax);
        const int *types = A.types + (size_t)b * (A.npad + A.nghost);
        const int ti = types[ci];
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;

        for (int i = lane; i < A.nbp; i += 32) {
            Ed[i] = A.Eb[(size_t)t * A.nbp + i];
            Xd[i] = L.Xb[(size_t)t * A.nbp + i];
        }
        __syncwarp();
        for (int c = lane; c < P.ndense; c += 32) {
            const int4 g = P.e4g[c];
            const int mu = P.e4m[c];
            V2 lo, hi;
            lo.x = g.x >= 0 ? Ed[g.x] : T(0);
            lo.y = g.y >= 0 ? T(mu & 255) * Ed[g.y] : T(0);
            hi.x = g.z >= 0 ? T((mu >> 8) & 255) * Ed[g.z] : T(0);
            hi.y = g.w >= 0 ? T((mu >> 16) & 255) * Ed[g.w] : T(0);
            *reinterpret_cast<V2 *>(E4 + 4 * c) = lo;
            *reinterpret_cast<V2 *>(E4 + 4 * c + 2) = hi;
            X1[c] = g.x >= 0 ? Xd[g.x] : T(0);
        }
        __syncwarp();

        T *gout = L.dcoeffs + (size_t)b * L.ncoef;
        for (int j0 = 0; j0 < nn; j0 += 32) {
            const int j = j0 + lane;
            bool act = j < nn;
            T x = 0, y = 0, z = 0;
            int nj = 0;
            if (act) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j]; }
            const T r = gsqrt(x * x + y * y + z * z);
            act = act && (r <= A.rmax) && (r > T(0));
            const T rinv = act ? T(1) / r : T(0);
            const int tj = act ? types[nj] : -1;
            const T ux = x * rinv, uy = y * rinv, uz = z * rinv;
            T q[CSP], dq[CSP];
            mtp_radial_basis<T, CSP>(act ? r : A.rmax, A.rmax, A.rmin, A.scaling, q, dq);
            T px = 0, py = 0, pz = 0;
            if (act) pair_weight(A, L, b, n, ci, nj, x, y, z, px, py, pz);
            const T ppar = px * ux + py * uy + pz * uz;
            const T qx = (px - ppar * ux) * rinv, qy = (py - ppar * uy) * rinv, qz = (pz - ppar * uz) * rinv;
            Powers<T, KD> pw;
            pw.set(ux, uy, uz);
            for (int m = 0; m < P.nmus; m++) {
                T Pv = 0, Gx = 0, Gy = 0, Gz = 0, Xv = 0;
                eval_mu<T, KD>(P.kmu[m], E4 + 4 * P.doff[m], pw, Pv, Gx, Gy, Gz);
                value_mu<T, KD>(P.kmu[m], X1 + P.doff[m], pw, Xv);
                am[m * 32 + lane] = act ? Xv + qx * Gx + qy * Gy + qz * Gz : T(0);
                bm[m * 32 + lane] = act ? ppar * Pv : T(0);
            }
            // per neighbour type: sum over lanes of Q_xi a_mu + Q'_xi b_mu, 16 (mu, xi) values at a time
            for (int tt = 0; tt < A.ntypes; tt++) {
                if (!__any_sync(FULL_MASK, tj == tt)) continue;
                const bool mine = tj == tt;
                T *grow = gout + (size_t)(ti * A.ntypes + tt) * P.nmus * A.cs;
                for (int v0 = 0; v0 < nval; v0 += 16) {
                    T v[16];
                    static_for<0, 16>([&](auto ii) {
                        constexpr int I = decltype(ii)::value;
                        constexpr int XI = I % CSP;
                        const int m = (v0 + I) / CSP;      // warp-uniform
                        v[I] = mine ? fma(q[XI], am[m * 32 + lane], dq[XI] * bm[m * 32 + lane]) : T(0);
                    });
                    const T tot = warp_xreduce<T, 16>(v, lane);
                    const int k = v0 + (lane >> 1);
                    const int m = k / CSP, xi = k - m * CSP;
                    if ((lane & 1) == 0 && k < nval && xi < A.cs) atomicAdd(grow + m * A.cs + xi, tot);
                }
            }
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
struct LossWs {
    MtpWs base;
    size_t db, xb, total;
};
static LossWs loss_ws_layout(const MtpProgramDev &P, int B, int npad, int ntypes, size_t elem)
{
    LossWs L;
    L.base = mtp_ws_layout(P, B, npad, ntypes, elem);
    const size_t atoms = ((size_t)(B > 0 ? B : 0) * (npad > 0 ? npad : 0) + 31) & ~size_t(31);   // whole tiles of 32 atoms
    L.db = L.base.total;
    L.xb = L.db + up256(atoms * nbasic_pad(P) * elem);
    L.total = L.xb + up256(atoms * nbasic_pad(P) * elem);
    return L;
}

static size_t loss_contract_smem(const MtpProgramDev &P, size_t elem, int ta, bool tables)
{
    const size_t arrays = elem * (size_t)P.nm * (ta + 1) * 4;
    const size_t tab = tables ? sizeof(int2) * (size_t)P.nt * 3 : 0;
    return ((arrays + 15) & ~size_t(15)) + tab + 16;
}

template <typename T, int TA, bool SMEMTAB>
static int launch_loss_contract(const MtpProgramDev &P, const MtpArgs<T> &A, const LossArgs<T> &L, long atoms_upper, cudaStream_t st)
{
    const size_t smem = loss_contract_smem(P, sizeof(T), TA, SMEMTAB);
    auto kern = mtp_loss_contract_kernel<T, TA, SMEMTAB>;
    static KernelSetup setup;
    if (int rc = kernel_setup(setup, kern, smem)) return rc;
    kern<<<(unsigned)((atoms_upper + TA - 1) / TA), MTP_CWARPS * 32, smem, st>>>(P, A, L);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

template <typename T, int KD, int CSP>
static int launch_loss_bwd_v(const ai2b_mtp_program *prog, MtpArgs<T> A, LossArgs<T> L, void *ws, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    const LossWs W = loss_ws_layout(P, A.B, A.npad, A.ntypes, sizeof(T));
    unsigned char *w = reinterpret_cast<unsigned char *>(ws);
    A.prefix = reinterpret_cast<int *>(w + W.base.prefix);
    T *cpad = reinterpret_cast<T *>(w + W.base.cpad);
    A.coeffs_pad = cpad;
    A.Mb = reinterpret_cast<T *>(w + W.base.mb);
    A.Eb = reinterpret_cast<T *>(w + W.base.eb);
    L.Db = reinterpret_cast<T *>(w + W.db);
    L.Xb = reinterpret_cast<T *>(w + W.xb);
    A.ndp = ndense_pad(P);
    A.nbp = nbasic_pad(P);
    A.coeffs_pad = mtp_prepare<T>(A.binum, A.B, const_cast<int *>(A.prefix), A.coeffs, cpad, A.ntypes * A.ntypes * P.nmus, A.cs, CSP, st);
    AI2B_CUDA(cudaGetLastError());
    const long atoms_upper = (long)A.B * A.npad;
    const long need = (atoms_upper + MTP_WARPS - 1) / MTP_WARPS;
    // basic moments and their directional derivatives: the lanes-as-atoms kernels where they exist for these tables
    bool atoms_path = false;
    if constexpr (KD <= 6 && CSP == 8) atoms_path = mtp_atoms_supported(P, A.ntypes, A.cs, sizeof(T), (long)A.npad + A.nghost);
    if (atoms_path) {
        A.tiled = 1;
        if (int rc = mtp_fwd_atoms<T>(P, A, st)) return rc;
        if (int rc = mtp_dfwd_atoms<T>(P, A, L, st)) return rc;
    } else {
        const size_t smem = sizeof(T) * (size_t)(2 * A.ndp + 2 * MTP_MAX_MU * 32) * MTP_WARPS;
        auto kern = mtp_loss_fwd_kernel<T, KD, CSP>;
        static KernelSetup setup;
        int per_sm = 1;
        if (int rc = kernel_setup(setup, kern, smem, MTP_WARPS * 32, &per_sm)) return rc;
        long blocks = (long)sm_count() * per_sm;
        if (blocks > need) blocks = need;
        kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A, L);
        AI2B_CUDA(cudaGetLastError());
    }
    {
        const size_t cap = 222 * 1024;
        int rc = AI2B_ERR_UNSUPPORTED;
        bool done = false;
#define AI2B_TRY(TA_)                                                                                                   \
    if (!done && (long)P.nm * (TA_ + 1) <= 65535) {                                                                     \
        if (loss_contract_smem(P, sizeof(T), TA_, true) <= cap) { rc = launch_loss_contract<T, TA_, true>(P, A, L, atoms_upper, st); done = true; } \
        else if (loss_contract_smem(P, sizeof(T), TA_, false) <= cap) { rc = launch_loss_contract<T, TA_, false>(P, A, L, atoms_upper, st); done = true; } \
    }
        AI2B_TRY(32) AI2B_TRY(16) AI2B_TRY(8)
#undef AI2B_TRY
        if (!done) set_error("MTP tables with %d moments do not fit the loss-gradient kernel's shared memory", P.nm);
        if (rc) return rc;
    }
    {
        const size_t smem = sizeof(T) * (size_t)(5 * A.ndp + 2 * A.nbp + 2 * MTP_MAX_MU * 32) * MTP_WARPS;
        auto kern = mtp_loss_coeff_kernel<T, KD, CSP>;
        static KernelSetup setup;
        int per_sm = 1;
        if (int rc = kernel_setup(setup, kern, smem, MTP_WARPS * 32, &per_sm)) return rc;
        long blocks = (long)sm_count() * per_sm;
        if (blocks > need) blocks = need;
        kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A, L);
        AI2B_CUDA(cudaGetLastError());
    }
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" size_t ai2b_mtp_loss_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int natoms_pad, int ntypes)
{
    if (!prog) return 0;
    return loss_ws_layout(prog->dev, batch_size, natoms_pad, ntypes > 0 ? ntypes : 1, sizeof(double)).total + 256;
}

template <typename T>
static int loss_forward(int e_per_atom, T *loss, T *rmse, int B, int npad, int nghost, const int *binum, const int *bilist, T ew, T fw,
                        T vw, const T *e_ml, const T *e_dft, const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, void *ws,
                        size_t ws_bytes, void *stream)
{
    AI2B_REQUIRE(B >= 0 && npad >= 0 && nghost >= 0, AI2B_ERR_INVALID, "loss: negative size");
    if (B == 0) return AI2B_OK;
    AI2B_REQUIRE(loss && rmse && binum && bilist && e_ml && e_dft && f_ml && f_dft && (!v_ml == !v_dft), AI2B_ERR_INVALID,
                 "loss: NULL argument");
    AI2B_REQUIRE(ws && ws_bytes >= 4 * sizeof(T), AI2B_ERR_WORKSPACE, "loss: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    T *se = reinterpret_cast<T *>(ws);
    AI2B_CUDA(cudaMemsetAsync(se, 0, 4 * sizeof(T), st));
    mtp_loss_kernel<T><<<B, 256, 0, st>>>(loss, se, e_per_atom, npad, nghost, binum, bilist, ew, fw, vw, e_ml, e_dft, f_ml, f_dft, v_ml,
                                          v_dft);
    mtp_rmse_kernel<T><<<1, 32, 0, st>>>(rmse, se, B);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

#define AI2B_DEF_LOSS(SUF, T)                                                                                      \
    extern "C" int ai2b_mtp_loss_##SUF(T *loss, T *rmse, int B, int npad, int nghost, const int *binum,            \
                                       const int *bilist, T ew, T fw, T vw, const T *e_ml, const T *e_dft,         \
                                       const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, void *ws,     \
                                       size_t ws_bytes, void *stream)                                              \
    {                                                                                                              \
        return loss_forward<T>(0, loss, rmse, B, npad, nghost, binum, bilist, ew, fw, vw, e_ml, e_dft, f_ml, f_dft, \
                               v_ml, v_dft, ws, ws_bytes, stream);                                                 \
    }                                                                                                              \
    extern "C" int ai2b_nep_loss_##SUF(T *loss, T *rmse, int B, int npad, int nghost, const int *binum,            \
                                       const int *bilist, T ew, T fw, T vw, const T *e_ml, const T *e_dft,         \
                                       const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, void *ws,     \
                                       size_t ws_bytes, void *stream)                                              \
    {                                                                                                              \
        return loss_forward<T>(1, loss, rmse, B, npad, nghost, binum, bilist, ew, fw, vw, e_ml, e_dft, f_ml, f_dft, \
                               v_ml, v_dft, ws, ws_bytes, stream);                                                 \
    }                                                                                                              \
    extern "C" int ai2b_mtp_loss_backward_##SUF(                                                                   \
        const ai2b_mtp_program *prog, T *dcoeffs, T *dlinear, T *dbias, T ew, T fw, T vw, const T *e_ml,           \
        const T *e_dft, const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, int cs, T scaling,           \
        const T *coeffs, const T *lin, const T *bias, int B, int npad, const int *binum, const int *bilist,        \
        const int *numneigh, const int *firstneigh, const T *rcs, const int *types, int ntypes, int umax,          \
        int nghost, T rmax, T rmin, const T *qs, void *ws, size_t ws_bytes, void *stream)                          \
    {                                                                                                              \
        AI2B_REQUIRE(prog && dcoeffs && dlinear && dbias && e_ml && e_dft && f_ml && f_dft && (!v_ml == !v_dft) && \
                         coeffs && lin && qs && binum && bilist && numneigh && firstneigh && rcs && types,         \
                     AI2B_ERR_INVALID, "ai2b_mtp_loss_backward: NULL argument");                                   \
        (void)bias;                                                                                                \
        AI2B_REQUIRE(cs >= 1 && cs <= 16, AI2B_ERR_UNSUPPORTED, "chebyshev_size %d outside 1..16", cs);            \
        AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0 && ntypes >= 1, AI2B_ERR_INVALID, "negative size");          \
        AI2B_REQUIRE(nghost == 0, AI2B_ERR_UNSUPPORTED, "the loss gradient is defined for nghost = 0 only");       \
        const MtpProgramDev &P = prog->dev;                                                                        \
        const int ncoef = ntypes * ntypes * P.nmus * cs;                                                           \
        cudaStream_t st = (cudaStream_t)stream;                                                                    \
        if (B == 0) return AI2B_OK;                                                                                \
        AI2B_CUDA(cudaMemsetAsync(dcoeffs, 0, sizeof(T) * (size_t)B * ncoef, st));                                 \
        AI2B_CUDA(cudaMemsetAsync(dlinear, 0, sizeof(T) * (size_t)B * P.ns, st));                                  \
        AI2B_CUDA(cudaMemsetAsync(dbias, 0, sizeof(T) * (size_t)B * ntypes, st));                                  \
        if (npad == 0) return AI2B_OK;                                                                             \
        const size_t need = loss_ws_layout(P, B, npad, ntypes, sizeof(T)).total;                                   \
        AI2B_REQUIRE(ws && ws_bytes >= need, AI2B_ERR_WORKSPACE, "MTP loss workspace too small: %zu < %zu bytes",  \
                     ws_bytes, need);                                                                              \
        MtpArgs<T> A{nullptr, nullptr, nullptr, nullptr, coeffs, lin, bias, qs, nullptr, binum, bilist, numneigh,  \
                     firstneigh, types, rcs, nullptr, nullptr, nullptr, B, npad, ntypes, umax, nghost, cs, 0, 0,   \
                     scaling, rmax, rmin};                                                                         \
        LossArgs<T> L{e_ml, e_dft, f_ml, f_dft, v_ml, v_dft, dcoeffs, dlinear, dbias, nullptr, nullptr, ew, fw,    \
                      vw, ncoef};                                                                                  \
        if (P.kmax <= 6 && cs <= 8) return launch_loss_bwd_v<T, 6, 8>(prog, A, L, ws, st);                         \
        return launch_loss_bwd_v<T, 8, 16>(prog, A, L, ws, st);                                                    \
    }

AI2B_DEF_LOSS(f64, double)
AI2B_DEF_LOSS(f32, float)
