// Linear MTP: energy, force, virial and descriptors on sm_100a.
//
// One warp evaluates one centre atom at a time; lanes are the atom's neighbours.
//   1. pair set-up: r, unit vector, radial functions f_mu / f'_mu (registers -> shared memory)
//   2. forward: dense moment sums per mu (compile-time monomials + warp transpose-reduce)
//   3. product rows by dependency depth (lanes = destinations), site energy
//   4. adjoint sweep as a gather per source moment (lanes = sources), deepest first
//   5. adjoints of the basic moments -> polynomial coefficients, evaluated per neighbour with
//      their gradient; pair force g = f' P u + f/r (G - (u.G) u); F_i += g, F_j -= g, V -= g (x) r
// Reference semantics: source/descriptor/mtpr/include/mtpBasis.h:400-534, linearMtp.h:190-352.
#include "mtp_poly.cuh"

namespace ai2b {

constexpr int MTP_WARPS = 4;   // warps (atoms in flight) per block

enum MtpMode { MODE_EFV = 0, MODE_EF = 1, MODE_DESC = 2 };

template <typename T>
struct MtpArgs {
    T *etot, *force, *virial, *desc;
    const T *coeffs, *lin, *bias, *qs;
    const T *coeffs_pad;   // [ntypes*ntypes][nmus][CSP] zero-padded copy of coeffs (workspace)
    const int *binum, *bilist, *numneigh, *firstneigh, *types;
    const T *rcs;
    const int *prefix;   // [B+1] exclusive prefix sum of binum (workspace)
    int B, npad, ntypes, umax, nghost, cs;
    T scaling, rmax, rmin;
};

// exclusive prefix sum of binum -> prefix[0..B]; one block
__global__ void prefix_binum_kernel(const int *__restrict__ binum, int B, int *__restrict__ prefix)
{
    __shared__ int carry;
    __shared__ int wsum[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { carry = 0; prefix[0] = 0; }
    __syncthreads();
    for (int base = 0; base < B; base += blockDim.x) {
        int i = base + threadIdx.x;
        int v = i < B ? binum[i] : 0;
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(FULL_MASK, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = lane < (int)(blockDim.x >> 5) ? wsum[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int n = __shfl_up_sync(FULL_MASK, w, o);
                if (lane >= o) w += n;
            }
            wsum[lane] = w;
        }
        __syncthreads();
        int off = carry + (warp > 0 ? wsum[warp - 1] : 0);
        if (i < B) prefix[i + 1] = off + inc;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = off + inc;
        __syncthreads();
    }
}

__host__ __device__ inline int mtp_warp_elems(const MtpProgramDev &P)
{
    // per-warp shared memory, in elements of T: E4[4*ndense] M[nm] Eb[nm] Md[ndense] fr,fd[2*nmus*32]
    auto r4 = [](int n) { return (n + 3) & ~3; };
    return 4 * r4(P.ndense) + 2 * r4(P.nm) + r4(P.ndense) + 2 * MTP_MAX_MU * 32;
}

template <typename T>
__global__ void mtp_pad_coeffs_kernel(const T *__restrict__ c, T *__restrict__ out, int rows, int cs, int csp)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * csp) return;
    int r = i / csp, k = i % csp;
    out[i] = k < cs ? c[r * cs + k] : T(0);
}

template <typename T, int MODE, int KD, int CSP>
__global__ void __launch_bounds__(MTP_WARPS * 32, 3) mtp_atom_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
    using V2 = typename Vec2<T>::type;
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto r4 = [](int n) { return (n + 3) & ~3; };
    T *E4 = reinterpret_cast<T *>(smem_raw) + (size_t)warp * mtp_warp_elems(P);
    T *M = E4 + 4 * r4(P.ndense);
    T *Eb = M + r4(P.nm);
    T *Md = Eb + r4(P.nm);
    T *fr = Md + r4(P.ndense);
    T *fdv = fr + MTP_MAX_MU * 32;

    const int ntot = A.prefix[A.B];
    const int nw = gridDim.x * MTP_WARPS, gw = blockIdx.x * MTP_WARPS + warp;
    const int chunk = (ntot + nw - 1) / nw;
    const int t0 = gw * chunk, t1 = min(ntot, t0 + chunk);

    int cur_b = -1, b_end = 0;
    T eacc = T(0);
    T vir[9];
#pragma unroll
    for (int k = 0; k < 9; k++) vir[k] = T(0);

    auto flush = [&]() {
        if (cur_b < 0) return;
        if (MODE != MODE_DESC) {
            if (lane == 0) atomicAdd(A.etot + cur_b, eacc);
            if (MODE == MODE_EFV) {
#pragma unroll
                for (int k = 0; k < 9; k++) {
                    T s = warp_sum(vir[k]);
                    if (lane == 0) atomicAdd(A.virial + 9 * cur_b + k, s);
                    vir[k] = T(0);
                }
            }
        }
        eacc = T(0);
    };

    for (int t = t0; t < t1; t++) {
        if (t >= b_end || cur_b < 0) {
            flush();
            int lo = 0, hi = A.B;   // largest b with prefix[b] <= t
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (A.prefix[mid] <= t) lo = mid; else hi = mid;
            }
            cur_b = lo;
            b_end = A.prefix[lo + 1];
        }
        const int b = cur_b;
        const int ii = t - A.prefix[b];
        const size_t slot = (size_t)b * A.npad + ii;
        const int ci = A.bilist[slot];
        const int nn = min(A.numneigh[slot], A.umax);
        const int *types = A.types + (size_t)b * (A.npad + (MODE == MODE_DESC ? 0 : A.nghost));
        const int ti = types[ci];
        const int *fn = A.firstneigh + slot * A.umax;
        const T *rc = A.rcs + slot * A.umax * 3;

        for (int i = lane; i < P.ndense; i += 32) Md[i] = T(0);
        for (int i = P.nb + lane; i < P.nm; i += 32) M[i] = T(0);
        __syncwarp();

        // pair state of the (last) chunk, reused by the force pass when the atom has <= 32 neighbours
        T x = 0, y = 0, z = 0, ux = 0, uy = 0, uz = 0, rinv = 0;
        int nj = 0;
        bool act = false;
        auto pair_setup = [&](int j0) {
            const int j = j0 + lane;
            act = j < nn;
            x = y = z = T(0);
            nj = 0;
            if (act) {
                x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
                nj = fn[j];
            }
            const T r = gsqrt(x * x + y * y + z * z);
            act = act && (r <= A.rmax) && (r > T(0));
            int tj = 0;
            if (act) { tj = types[nj]; rinv = T(1) / r; } else { rinv = T(0); }
            ux = x * rinv; uy = y * rinv; uz = z * rinv;
            T q[CSP], dq[CSP];
            mtp_radial_basis<T, CSP>(act ? r : A.rmax, A.rmax, A.rmin, A.scaling, q, dq);
            const T *crow = A.coeffs_pad + (size_t)(ti * A.ntypes + tj) * P.nmus * CSP;
            for (int m = 0; m < P.nmus; m++) {
                T f = T(0), fd = T(0);
#pragma unroll
                for (int k = 0; k < CSP; k += 2) {
                    const V2 c2 = *reinterpret_cast<const V2 *>(crow + m * CSP + k);
                    f = fma(c2.x, q[k], f); fd = fma(c2.x, dq[k], fd);
                    f = fma(c2.y, q[k + 1], f); fd = fma(c2.y, dq[k + 1], fd);
                }
                fr[m * 32 + lane] = act ? f : T(0);
                fdv[m * 32 + lane] = act ? fd : T(0);
            }
        };

        // ---- forward: dense basic-moment sums ------------------------------------------------
        for (int j0 = 0; j0 < nn || j0 == 0; j0 += 32) {
            pair_setup(j0);
            Powers<T, KD> pw;
            pw.set(ux, uy, uz);
            for (int m = 0; m < P.nmus; m++) fwd_mu<T, KD>(P.kmu[m], fr[m * 32 + lane], pw, Md + P.doff[m], lane);
        }
        __syncwarp();
        for (int i = lane; i < P.nb; i += 32) M[i] = Md[P.basic_dense[i]];
        __syncwarp();

        // ---- products, by dependency depth ---------------------------------------------------
        for (int lev = 0; lev < P.nlev; lev++) {
            for (int d = P.fwd_lev_off[lev] + lane; d < P.fwd_lev_off[lev + 1]; d += 32) {
                const int4 ds = P.fwd_dst[d];
                const int *ab = P.fwd_ab;
                const T *mult = fwd_mult<T>(P);
                T acc0 = T(0), acc1 = T(0);
                int r = ds.y;
                for (; r + 1 < ds.z; r += 2) {
                    const int x0 = ab[r], x1 = ab[r + 1];
                    const T m0 = mult[r], m1 = mult[r + 1];
                    acc0 = fma(m0 * M[x0 & 0xffff], M[x0 >> 16], acc0);
                    acc1 = fma(m1 * M[x1 & 0xffff], M[x1 >> 16], acc1);
                }
                if (r < ds.z) {
                    const int x0 = ab[r];
                    acc0 = fma(mult[r] * M[x0 & 0xffff], M[x0 >> 16], acc0);
                }
                M[ds.x] += acc0 + acc1;
            }
            __syncwarp();
        }

        if (MODE == MODE_DESC) {
            for (int s = lane; s < P.ns; s += 32) A.desc[slot * P.ns + s] = M[P.map[s]];
            __syncwarp();
            continue;
        }

        // ---- site energy and adjoint seeds ------------------------------------------------------
        for (int i = lane; i < P.nm; i += 32) Eb[i] = T(0);
        __syncwarp();
        T es = T(0);
        for (int s = lane; s < P.ns; s += 32) {
            const int m = P.map[s];
            const T l = A.lin[s], q = A.qs[s];
            es += l * M[m] / q;
            Eb[m] = l / q;
        }
        es = warp_sum(es);
        eacc += es + A.bias[ti];
        __syncwarp();

        // ---- adjoint sweep (gather per source moment, deepest sources first) --------------------
        for (int k = 0; k < P.nlev; k++) {
            for (int d = P.rev_lev_off[k] + lane; d < P.rev_lev_off[k + 1]; d += 32) {
                const int4 ms = P.rev_mom[d];
                const int *od = P.rev_od;
                const T *mult = rev_mult<T>(P);
                T acc0 = T(0), acc1 = T(0);
                int e = ms.y;
                for (; e + 1 < ms.z; e += 2) {
                    const int x0 = od[e], x1 = od[e + 1];
                    const T m0 = mult[e], m1 = mult[e + 1];
                    acc0 = fma(m0 * Eb[x0 >> 16], M[x0 & 0xffff], acc0);
                    acc1 = fma(m1 * Eb[x1 >> 16], M[x1 & 0xffff], acc1);
                }
                if (e < ms.z) {
                    const int x0 = od[e];
                    acc0 = fma(mult[e] * Eb[x0 >> 16], M[x0 & 0xffff], acc0);
                }
                Eb[ms.x] += acc0 + acc1;
            }
            __syncwarp();
        }

        // ---- adjoints of the basic moments -> polynomial coefficient quadruples -----------------
        for (int c = lane; c < P.ndense; c += 32) {
            const int4 g = P.e4g[c];
            const int mu = P.e4m[c];
            E4[4 * c + 0] = g.x >= 0 ? Eb[g.x] : T(0);
            E4[4 * c + 1] = g.y >= 0 ? T(mu & 255) * Eb[g.y] : T(0);
            E4[4 * c + 2] = g.z >= 0 ? T((mu >> 8) & 255) * Eb[g.z] : T(0);
            E4[4 * c + 3] = g.w >= 0 ? T((mu >> 16) & 255) * Eb[g.w] : T(0);
        }
        __syncwarp();

        // ---- force / virial pass ------------------------------------------------------------------
        T *frc = A.force + (size_t)b * (A.npad + A.nghost) * 3;
        T fcx = T(0), fcy = T(0), fcz = T(0);
        for (int j0 = 0; j0 < nn; j0 += 32) {
            if (nn > 32) pair_setup(j0);
            Powers<T, KD> pw;
            pw.set(ux, uy, uz);
            T gx = T(0), gy = T(0), gz = T(0);
            for (int m = 0; m < P.nmus; m++) {
                T Pv = T(0), Gx = T(0), Gy = T(0), Gz = T(0);
                eval_mu<T, KD>(P.kmu[m], E4 + 4 * P.doff[m], pw, Pv, Gx, Gy, Gz);
                const T f = fr[m * 32 + lane], fd = fdv[m * 32 + lane];
                const T ug = ux * Gx + uy * Gy + uz * Gz;
                const T a = fd * Pv - f * rinv * ug, c = f * rinv;
                gx += a * ux + c * Gx;
                gy += a * uy + c * Gy;
                gz += a * uz + c * Gz;
            }
            if (act) {
                fcx += gx; fcy += gy; fcz += gz;
                atomicAdd(frc + 3 * nj + 0, -gx);
                atomicAdd(frc + 3 * nj + 1, -gy);
                atomicAdd(frc + 3 * nj + 2, -gz);
                if (MODE == MODE_EFV) {
                    vir[0] -= gx * x; vir[1] -= gx * y; vir[2] -= gx * z;
                    vir[3] -= gy * x; vir[4] -= gy * y; vir[5] -= gy * z;
                    vir[6] -= gz * x; vir[7] -= gz * y; vir[8] -= gz * z;
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
static int g_sm_count = 0;
static int sm_count()
{
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

static size_t mtp_ws_bytes(const MtpProgramDev &P, int B, int ntypes, size_t elem)
{
    size_t pre = (((size_t)(B > 0 ? B : 0) + 1) * sizeof(int) + 255) & ~size_t(255);
    size_t co = ((size_t)ntypes * ntypes * P.nmus * 16 * elem + 255) & ~size_t(255);
    return pre + co;
}

template <typename T, int MODE, int KD, int CSP>
static int launch_mtp_v(const ai2b_mtp_program *prog, MtpArgs<T> A, void *ws, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    int *prefix = reinterpret_cast<int *>(ws);
    T *cpad = reinterpret_cast<T *>(reinterpret_cast<unsigned char *>(ws) + ((((size_t)A.B + 1) * sizeof(int) + 255) & ~size_t(255)));
    A.prefix = prefix;
    A.coeffs_pad = cpad;
    prefix_binum_kernel<<<1, 256, 0, st>>>(A.binum, A.B, prefix);
    const int rows = A.ntypes * A.ntypes * P.nmus;
    mtp_pad_coeffs_kernel<T><<<(rows * CSP + 255) / 256, 256, 0, st>>>(A.coeffs, cpad, rows, A.cs, CSP);
    AI2B_CUDA(cudaGetLastError());

    const size_t smem = sizeof(T) * (size_t)mtp_warp_elems(P) * MTP_WARPS;
    AI2B_REQUIRE(smem <= 227 * 1024, AI2B_ERR_UNSUPPORTED, "MTP tables need %zu bytes of shared memory per block", smem);
    auto kern = mtp_atom_kernel<T, MODE, KD, CSP>;
    static size_t configured = 0;   // per instantiation
    static int per_sm = 0;
    if (smem > configured || per_sm == 0) {
        AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MTP_WARPS * 32, smem));
        if (per_sm < 1) per_sm = 1;
        configured = smem;
    }
    const long slots = (long)A.B * A.npad;
    long blocks = (long)sm_count() * per_sm;
    const long need = (slots + MTP_WARPS - 1) / MTP_WARPS;
    if (blocks > need) blocks = need;
    kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

template <typename T, int MODE>
static int launch_mtp(const ai2b_mtp_program *prog, MtpArgs<T> A, void *ws, size_t ws_bytes, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    AI2B_REQUIRE(A.cs >= 1 && A.cs <= 16, AI2B_ERR_UNSUPPORTED, "chebyshev_size %d outside 1..16", A.cs);
    AI2B_REQUIRE(A.B >= 0 && A.npad >= 0 && A.umax >= 0 && A.ntypes >= 1 && A.nghost >= 0, AI2B_ERR_INVALID, "negative size");
    if (A.B == 0 || A.npad == 0) return AI2B_OK;
    const size_t need = mtp_ws_bytes(P, A.B, A.ntypes, sizeof(T));
    AI2B_REQUIRE(ws && ws_bytes >= need, AI2B_ERR_WORKSPACE, "MTP workspace too small: %zu < %zu bytes", ws_bytes, need);
    // fast variant: monomial degree <= 6 (template level <= 16) and <= 8 radial basis functions
    if (P.kmax <= 6 && A.cs <= 8) return launch_mtp_v<T, MODE, 6, 8>(prog, A, ws, st);
    return launch_mtp_v<T, MODE, 8, 16>(prog, A, ws, st);
}

}  // namespace ai2b

using namespace ai2b;

extern "C" size_t ai2b_mtp_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int ntypes)
{
    if (!prog) return 0;
    return mtp_ws_bytes(prog->dev, batch_size, ntypes > 0 ? ntypes : 1, sizeof(double));
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
        MtpArgs<T> A{etot, force, virial, nullptr, coeffs, lin, bias, qs, nullptr, binum, bilist, numneigh, firstneigh, \
                     types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, scaling, rmax, rmin};             \
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
        MtpArgs<T> A{nullptr, nullptr, nullptr, desc, coeffs, nullptr, nullptr, nullptr, nullptr, binum, bilist,        \
                     numneigh, firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, scaling,    \
                     rmax, rmin};                                                                              \
        return launch_mtp<T, MODE_DESC>(prog, A, ws, ws_bytes, st);                                            \
    }

AI2B_DEF_MTP(f64, double)
AI2B_DEF_MTP(f32, float)
