// NEP training path: per-structure gradient of the loss w.r.t. coeffs, w0, b0, w1, type_bias.
// Included by nep_kernels.cu after the shared helpers (nep_radial, nep_blm, c_C3B).
//
// Reference: NepLoss<T>::find_loss_backward / find_ef_loss_backward
// (source/descriptor/nep/include/nepLoss.h, launcher nepLoss_cpu_launcher.h:69-160,213-330; CUDA
// source/descriptor/nep/gpu/include/nepLoss.cuh). Formulation used here: with
//   lam = 2 e_w / n (E - E*),  P_a = 2 f_w / (3n) (F_a - F*_a),  Qm = 2 v_w / (9n) (V - V*)
// the force and virial terms of the loss are Phi = sum_ij g_ij . p_ij with the per-pair weight
// p_ij = P_i - P_j - Qm r_ij and g_ij the pair gradient, so dL/dtheta = lam dE/dtheta + dPhi/dtheta
// and, per atom, Phi_i = sum_k (dE_i/dq_k) u_k, u_k = directional derivative of descriptor k along p.
// One warp per atom, one structure per blockIdx.y:
//   A  lanes = neighbours: sums q, S and their directional derivatives u, DS (warp transpose-reductions)
//   B  network forward with the second-order terms, lanes = neurons; adjoints of q and u
//   C  lanes = neighbours again: the coefficient gradient is  sum_j f_xi (X + GY) + f'_xi Y (r^.p)
//      per (function, xi), with polynomials X, Y whose coefficients come from step B; reduced over the
//      lanes of each neighbour type
// Gradients accumulate in shared memory per block and reach global memory once per block.
#pragma once

namespace ai2b {

constexpr int NEPL_WARPS = 4;

template <typename T>
struct NepLossArgs {
    T *dco, *dw0, *db0, *dw1, *dbi;
    const T *e_ml, *e_dft, *f_ml, *f_dft, *v_ml, *v_dft;   // v_* NULL: energy + force loss
    T ew, fw, vw;
};

// elements (of T) of the block accumulators and of one warp's scratch
__host__ __device__ inline size_t nepl_block_elems(int ntypes, int nfun, int cs, int nneu, int nd)
{
    return (size_t)ntypes * ntypes * nfun * cs + (size_t)ntypes * nneu * (nd + 2) + ntypes;
}
__host__ __device__ inline size_t nepl_warp_elems(int nd, int nS, int nneu, int nfun, int cs, int ntypes)
{
    const size_t red = (size_t)ntypes * nfun * cs;
    return 4 * (size_t)nd + 4 * (size_t)nS + 3 * (size_t)nneu + ((red + 31) & ~size_t(31)) + 64;
}

// sum over the warp of `count` <= NMAX per-lane values produced by f(k); result k lands in out[k].
// NMAX is a compile-time bound so that f sees compile-time indices (its arrays stay in registers).
template <typename T, int NMAX, typename F>
__device__ __forceinline__ void warp_reduce_many(int count, F f, T *out, int lane)
{
#pragma unroll
    for (int k0 = 0; k0 < NMAX; k0 += 32) {
        if (k0 < count) {
            T v[32];
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = (k0 + i < count) ? f(k0 + i) : T(0);
            const T r = warp_xreduce<T, 32>(v, lane);
            if (k0 + lane < count) out[k0 + lane] = r;
        }
    }
}

template <typename T, int CSP, bool VIRIAL>
__global__ void __launch_bounds__(NEPL_WARPS * 32) nep_loss_backward_kernel(const NepArgs<T> A, const T *__restrict__ coeffs,
                                                                              const NepLossArgs<T> L)
{
    extern __shared__ __align__(16) unsigned char nepl_smem[];
    __shared__ T iq[96];   // 1 / q_scaler
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.y;
    const int nfun = A.n_r + A.n_a, nlm = A.l_max * A.l_max + 2 * A.l_max, nS = A.n_a * nlm, nd = A.nd, nneu = A.nneu;
    const size_t nblk = nepl_block_elems(A.ntypes, nfun, A.cs, nneu, nd);
    T *g_co = reinterpret_cast<T *>(nepl_smem);                       // [ntypes^2][nfun][cs]
    T *g_w0 = g_co + (size_t)A.ntypes * A.ntypes * nfun * A.cs;       // [ntypes][nneu][nd]
    T *g_b0 = g_w0 + (size_t)A.ntypes * nneu * nd;                    // [ntypes][nneu]
    T *g_w1 = g_b0 + (size_t)A.ntypes * nneu;
    T *g_bi = g_w1 + (size_t)A.ntypes * nneu;                         // [ntypes]
    T *ws = g_co + nblk + (size_t)warp * nepl_warp_elems(nd, nS, nneu, nfun, A.cs, A.ntypes);
    T *q = ws, *u = q + nd, *av = u + nd, *be = av + nd;              // descriptors, directional derivative, dE/dq, dPhi/dq~
    T *S = be + nd, *DS = S + nS, *xc = DS + nS, *yc = xc + nS;       // sums, their derivatives, polynomial coefficients
    T *th = yc + nS, *sp = th + nneu, *d2v = sp + nneu;
    T *red = d2v + nneu;
    for (size_t i = threadIdx.x; i < nblk; i += blockDim.x) g_co[i] = T(0);
    for (int k = threadIdx.x; k < A.nd; k += blockDim.x) iq[k] = T(1) / A.qs[k];
    __syncthreads();

    const int n = A.binum[b];
    const int *types = A.types + (size_t)b * A.npad;
    const T *fm = L.f_ml + (size_t)b * A.npad * 3, *fd = L.f_dft + (size_t)b * A.npad * 3;
    const T lam = T(2) * L.ew / T(n) * (L.e_ml[b] - L.e_dft[b]), cf = T(2) * L.fw / T(3 * n), cv = VIRIAL ? T(2) * L.vw / T(9 * n) : T(0);
    T dV[9];
#pragma unroll
    for (int k = 0; k < 9; k++) dV[k] = VIRIAL ? L.v_ml[9 * b + k] - L.v_dft[9 * b + k] : T(0);

    // per-neighbour quantities of lane j (recomputed in both passes)
    struct Pair {
        bool on, ang;
        int tj;
        T r, rinv, ux, uy, uz, vp, px, py, pz;   // p_perp / r in (px,py,pz)
        T fr[CSP], dfr[CSP], fa[CSP], dfa[CSP];
    };
    auto load_pair = [&](Pair &P, const T *rc, const int *fn, int ci, int nn, int j) {
        P.on = j < nn;
        T x = 0, y = 0, z = 0;
        int nj = 0;
        if (P.on) { x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2]; nj = fn[j]; }
        P.r = gsqrt(x * x + y * y + z * z);
        P.on = P.on && P.r <= A.rc_r && P.r > T(0);
        P.tj = P.on ? types[nj] : 0;
        P.rinv = P.on ? T(1) / P.r : T(0);
        P.ux = x * P.rinv; P.uy = y * P.rinv; P.uz = z * P.rinv;
        T p0 = 0, p1 = 0, p2 = 0;
        if (P.on) {
            p0 = cf * (fm[3 * ci] - fd[3 * ci]) - cf * (fm[3 * nj] - fd[3 * nj]) - cv * (dV[0] * x + dV[1] * y + dV[2] * z);
            p1 = cf * (fm[3 * ci + 1] - fd[3 * ci + 1]) - cf * (fm[3 * nj + 1] - fd[3 * nj + 1]) - cv * (dV[3] * x + dV[4] * y + dV[5] * z);
            p2 = cf * (fm[3 * ci + 2] - fd[3 * ci + 2]) - cf * (fm[3 * nj + 2] - fd[3 * nj + 2]) - cv * (dV[6] * x + dV[7] * y + dV[8] * z);
        }
        P.vp = P.ux * p0 + P.uy * p1 + P.uz * p2;
        P.px = (p0 - P.vp * P.ux) * P.rinv; P.py = (p1 - P.vp * P.uy) * P.rinv; P.pz = (p2 - P.vp * P.uz) * P.rinv;
        P.ang = P.on && P.r <= A.rc_a && A.l_max > 0;
        nep_radial<T, CSP>(P.on ? P.r : A.rc_r, A.rc_r, P.fr, P.dfr);
        nep_radial<T, CSP>(P.ang ? P.r : A.rc_a, A.rc_a, P.fa, P.dfa);
    };
    auto contract = [&](const T *crow, const T (&f)[CSP]) {
        T g = T(0);
#pragma unroll
        for (int k = 0; k < CSP; k++) g = fma(k < A.cs ? crow[k] : T(0), f[k], g);
        return g;
    };

    for (int ii = blockIdx.x * NEPL_WARPS + warp; ii < n; ii += gridDim.x * NEPL_WARPS) {
        const size_t slot = (size_t)b * A.npad + ii;
        const int ci = A.bilist[slot], nn = min(A.numneigh[slot], A.umax), ti = types[ci];
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;
        const T *ctab = coeffs + (size_t)ti * A.ntypes * nfun * A.cs;
        for (int i = lane; i < 4 * nd + 4 * nS; i += 32) ws[i] = T(0);
        __syncwarp();

        // ---- A: sums and directional derivatives ----------------------------------------------
        for (int j0 = 0; j0 < nn; j0 += 32) {
            Pair P;
            load_pair(P, rc, fn, ci, nn, j0 + lane);
            const T *crow = ctab + (size_t)P.tj * nfun * A.cs;
            warp_reduce_many<T, 32>(2 * A.n_r, [&](int k) {
                const int nidx = k >> 1;
                if (!P.on) return T(0);
                return (k & 1) ? contract(crow + nidx * A.cs, P.dfr) * P.vp : contract(crow + nidx * A.cs, P.fr);
            }, red, lane);
            __syncwarp();
            if (lane < A.n_r) { q[lane] += red[2 * lane]; u[lane] += red[2 * lane + 1]; }
            __syncwarp();
            if (A.l_max > 0) {
                T bl[NEP_NLM], gb[NEP_NLM][3];
                nep_blm<T, true>(P.ux, P.uy, P.uz, bl, gb);
                for (int mu = 0; mu < A.n_a; mu++) {
                    const T g = P.ang ? contract(crow + (A.n_r + mu) * A.cs, P.fa) : T(0);
                    const T dg = P.ang ? contract(crow + (A.n_r + mu) * A.cs, P.dfa) : T(0);
                    warp_reduce_many<T, 2 * NEP_NLM>(2 * nlm, [&](int k) {
                        const int lm = k >> 1;
                        if (k & 1) return dg * bl[lm] * P.vp + g * (gb[lm][0] * P.px + gb[lm][1] * P.py + gb[lm][2] * P.pz);
                        return g * bl[lm];
                    }, red, lane);
                    __syncwarp();
                    if (lane < nlm) { S[mu * nlm + lane] += red[2 * lane]; DS[mu * nlm + lane] += red[2 * lane + 1]; }
                    __syncwarp();
                }
            }
        }
        for (int pq = lane; pq < A.n_a * A.l_max; pq += 32) {
            const int mu = pq / A.l_max, l = pq % A.l_max + 1;
            T aq = T(0), au = T(0);
            for (int mp = 0; mp < 2 * l + 1; mp++) {
                const int lm = l * l - 1 + mp;
                const T w = (mp == 0 ? T(1) : T(2)) * (T)c_C3B[lm];
                aq += w * S[mu * nlm + lm] * S[mu * nlm + lm];
                au += T(2) * w * S[mu * nlm + lm] * DS[mu * nlm + lm];
            }
            q[A.n_r + pq] = aq; u[A.n_r + pq] = au;
        }
        __syncwarp();

        // ---- B: network with second-order terms ---------------------------------------------------
        const T *W0 = A.w0 + (size_t)ti * nneu * nd, *B0 = A.b0 + (size_t)ti * nneu, *W1 = A.w1 + (size_t)ti * nneu;
        for (int pn = lane; pn < nneu; pn += 32) {
            T h = B0[pn], sv = T(0);
            for (int k = 0; k < nd; k++) { const T w = W0[pn * nd + k] * iq[k]; h = fma(w, q[k], h); sv = fma(w, u[k], sv); }
            const T t = gtanh(h), d1 = T(1) - t * t, d2 = T(-2) * t * d1;
            th[pn] = W1[pn] * d1;          // weight of W0 in dE/dq
            sp[pn] = W1[pn] * sv * d2;     // weight of W0 in dPhi/dq~
            d2v[pn] = sv;
            const T gb0 = lam * W1[pn] * d1 + W1[pn] * sv * d2;
            atomicAdd(g_w1 + ti * nneu + pn, lam * t + d1 * sv);
            atomicAdd(g_b0 + ti * nneu + pn, gb0);
            for (int k = 0; k < nd; k++)
                atomicAdd(g_w0 + ((size_t)ti * nneu + pn) * nd + k, (gb0 * q[k] + W1[pn] * d1 * u[k]) * iq[k]);
        }
        if (lane == 0) atomicAdd(g_bi + ti, lam);
        __syncwarp();
        for (int k = lane; k < nd; k += 32) {
            T a0 = T(0), b0v = T(0);
            for (int pn = 0; pn < nneu; pn++) { const T w = W0[pn * nd + k]; a0 = fma(th[pn], w, a0); b0v = fma(sp[pn], w, b0v); }
            av[k] = a0 * iq[k];
            be[k] = lam * av[k] + b0v * iq[k];       // coefficient of dq_k/dc (av: coefficient of du_k/dc)
        }
        __syncwarp();
        for (int i = lane; i < nS; i += 32) {
            const int mu = i / nlm, lm = i % nlm;
            int l = 1;
            while ((l + 1) * (l + 1) - 1 <= lm) ++l;
            const int k = A.n_r + mu * A.l_max + l - 1;
            const T w2c = (lm == l * l - 1 ? T(1) : T(2)) * T(2) * (T)c_C3B[lm];
            xc[i] = w2c * (be[k] * S[i] + av[k] * DS[i]);
            yc[i] = w2c * av[k] * S[i];
        }
        __syncwarp();

        // ---- C: coefficient gradient, reduced over the lanes of each neighbour type ------------------
        for (int j0 = 0; j0 < nn; j0 += 32) {
            Pair P;
            load_pair(P, rc, fn, ci, nn, j0 + lane);
            T bl[NEP_NLM], gb[NEP_NLM][3];
            nep_blm<T, true>(P.ux, P.uy, P.uz, bl, gb);
            // per function: value weight and derivative weight
            auto weights = [&](int fidx, T &wv, T &wd) {
                if (fidx < A.n_r) { wv = be[fidx]; wd = av[fidx] * P.vp; return; }
                const int mu = fidx - A.n_r;
                T X = T(0), Y = T(0), GY = T(0);
                if (P.ang) {
#pragma unroll
                    for (int lm = 0; lm < NEP_NLM; lm++) {
                        if (lm < nlm) {
                            const T yv = yc[mu * nlm + lm];
                            X = fma(xc[mu * nlm + lm], bl[lm], X);
                            Y = fma(yv, bl[lm], Y);
                            GY = fma(yv, gb[lm][0] * P.px + gb[lm][1] * P.py + gb[lm][2] * P.pz, GY);
                        }
                    }
                }
                wv = X + GY; wd = Y * P.vp;
            };
            // every lane adds its neighbour's terms to the block accumulator of its (ti, tj) pair
            // (shared-memory atomics; lanes of the same neighbour type meet on the same addresses)
            for (int fidx = 0; fidx < nfun; fidx++) {
                T wv, wd;
                weights(fidx, wv, wd);
                const bool rad = fidx < A.n_r;
                if (rad ? P.on : P.ang) {
                    T *dst = g_co + (((size_t)ti * A.ntypes + P.tj) * nfun + fidx) * A.cs;
#pragma unroll
                    for (int xi = 0; xi < CSP; xi++)
                        if (xi < A.cs) atomicAdd(dst + xi, wv * (rad ? P.fr[xi] : P.fa[xi]) + wd * (rad ? P.dfr[xi] : P.dfa[xi]));
                }
            }
        }
        __syncwarp();
    }
    __syncthreads();
    // block accumulators -> per-structure gradients
    const size_t nco = (size_t)A.ntypes * A.ntypes * nfun * A.cs, nw0 = (size_t)A.ntypes * nneu * nd, nb0 = (size_t)A.ntypes * nneu;
    for (size_t i = threadIdx.x; i < nco; i += blockDim.x) if (g_co[i] != T(0)) atomicAdd(L.dco + b * nco + i, g_co[i]);
    for (size_t i = threadIdx.x; i < nw0; i += blockDim.x) if (g_w0[i] != T(0)) atomicAdd(L.dw0 + b * nw0 + i, g_w0[i]);
    for (size_t i = threadIdx.x; i < nb0; i += blockDim.x) {
        if (g_b0[i] != T(0)) atomicAdd(L.db0 + b * nb0 + i, g_b0[i]);
        if (g_w1[i] != T(0)) atomicAdd(L.dw1 + b * nb0 + i, g_w1[i]);
    }
    for (int i = threadIdx.x; i < A.ntypes; i += blockDim.x) if (g_bi[i] != T(0)) atomicAdd(L.dbi + (size_t)b * A.ntypes + i, g_bi[i]);
}

// the kernels that add into the per-structure gradients start from zeros
template <typename T>
static int nepl_zero_outputs(const NepArgs<T> &A, const NepLossArgs<T> &L, cudaStream_t st)
{
    const int nfun = A.n_r + A.n_a;
    const size_t nco = (size_t)A.ntypes * A.ntypes * nfun * A.cs, nw0 = (size_t)A.ntypes * A.nneu * A.nd, nb0 = (size_t)A.ntypes * A.nneu;
    AI2B_CUDA(cudaMemsetAsync(L.dco, 0, sizeof(T) * A.B * nco, st));
    AI2B_CUDA(cudaMemsetAsync(L.dw0, 0, sizeof(T) * A.B * nw0, st));
    AI2B_CUDA(cudaMemsetAsync(L.db0, 0, sizeof(T) * A.B * nb0, st));
    AI2B_CUDA(cudaMemsetAsync(L.dw1, 0, sizeof(T) * A.B * nb0, st));
    AI2B_CUDA(cudaMemsetAsync(L.dbi, 0, sizeof(T) * A.B * A.ntypes, st));
    return AI2B_OK;
}

// eight-lanes-per-atom kernel for small models (nep_loss_fast.cuh); *done = false: not applicable
template <typename T, int NMAX>
static int launch_nep_loss_fast(const NepArgs<T> &A, const T *coeffs, const NepLossArgs<T> &L, cudaStream_t st, bool *done);

template <typename T>
static int launch_nep_loss_backward(NepArgs<T> A, const T *coeffs, NepLossArgs<T> L, cudaStream_t st)
{
    AI2B_REQUIRE(A.cs >= 1 && A.cs <= 16, AI2B_ERR_UNSUPPORTED, "chebyshev_size %d outside 1..16", A.cs);
    AI2B_REQUIRE(A.l_max >= 0 && A.l_max <= 4, AI2B_ERR_INVALID, "l_max %d outside 0..4", A.l_max);
    AI2B_REQUIRE(A.n_r >= 0 && A.n_a >= 0 && A.n_r + A.n_a > 0 && A.nneu >= 1 && A.ntypes >= 1, AI2B_ERR_INVALID, "bad NEP sizes");
    AI2B_REQUIRE(A.n_r <= 16 && A.ntypes * A.cs <= 32 * 8, AI2B_ERR_UNSUPPORTED, "NEP loss gradient: n_radial > 16 or ntypes * chebyshev_size > 256");
    AI2B_REQUIRE(A.B >= 0 && A.npad >= 0 && A.umax >= 0 && A.nghost == 0, AI2B_ERR_INVALID, "NEP loss gradient: bad batch sizes (nghost must be 0)");
    A.nd = A.l_max == 0 ? A.n_r : A.n_r + A.n_a * A.l_max;
    A.nS = A.l_max == 0 ? 0 : A.n_a * (A.l_max * A.l_max + 2 * A.l_max);
    const int nfun = A.n_r + A.n_a;
    if (A.B == 0) return AI2B_OK;
    if (A.npad == 0) return nepl_zero_outputs(A, L, st);
    const size_t red_need = std::max<size_t>({(size_t)2 * A.n_r, (size_t)2 * (A.l_max * A.l_max + 2 * A.l_max), (size_t)A.ntypes * A.cs});
    AI2B_REQUIRE(red_need <= (size_t)A.ntypes * nfun * A.cs + 64, AI2B_ERR_UNSUPPORTED, "NEP loss gradient: reduction scratch too small");
    const size_t smem = sizeof(T) * (nepl_block_elems(A.ntypes, nfun, A.cs, A.nneu, A.nd) +
                                     NEPL_WARPS * nepl_warp_elems(A.nd, A.nS, A.nneu, nfun, A.cs, A.ntypes)) + 16;
    AI2B_REQUIRE(smem <= 200 * 1024, AI2B_ERR_UNSUPPORTED, "NEP loss gradient: model needs %zu bytes of shared memory per block", smem);
    AI2B_REQUIRE(A.B <= 65535, AI2B_ERR_UNSUPPORTED, "NEP loss gradient: more than 65535 structures per call");
    {
        bool done = false;
        const int rc = launch_nep_loss_fast<T, 4>(A, coeffs, L, st, &done);
        if (rc != AI2B_OK || done) return rc;
    }
    const bool vir = L.v_ml != nullptr;
    {
        const int rc = nepl_zero_outputs(A, L, st);
        if (rc != AI2B_OK) return rc;
    }
    auto run = [&](auto kern) -> int {
        AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int sms = 148, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        long bx = ((long)A.npad + NEPL_WARPS - 1) / NEPL_WARPS;
        const long cap = std::max(1L, (long)sms * 8 / A.B);   // enough blocks to fill the GPU; each ends with one flush of its accumulators
        if (bx > cap) bx = cap;
        kern<<<dim3((unsigned)bx, (unsigned)A.B), NEPL_WARPS * 32, smem, st>>>(A, coeffs, L);
        AI2B_CUDA(cudaGetLastError());
        return AI2B_OK;
    };
    if (A.cs <= 8) return vir ? run(nep_loss_backward_kernel<T, 8, true>) : run(nep_loss_backward_kernel<T, 8, false>);
    return vir ? run(nep_loss_backward_kernel<T, 16, true>) : run(nep_loss_backward_kernel<T, 16, false>);
}

}  // namespace ai2b
