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

template <typename T, int MODE>
__global__ void __launch_bounds__(MTP_WARPS * 32) mtp_atom_kernel(const MtpProgramDev P, const MtpArgs<T> A)
{
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
            T f[MTP_MAX_MU], fd[MTP_MAX_MU];
            mtp_radial<T>(act ? r : A.rmax, A.rmax, A.rmin, A.cs, P.nmus, A.scaling,
                          A.coeffs + (size_t)(ti * A.ntypes + tj) * P.nmus * A.cs, f, fd);
#pragma unroll
            for (int m = 0; m < MTP_MAX_MU; m++)
                if (m < P.nmus) {
                    fr[m * 32 + lane] = act ? f[m] : T(0);
                    fdv[m * 32 + lane] = act ? fd[m] : T(0);
                }
        };

        // ---- forward: dense basic-moment sums ------------------------------------------------
        for (int j0 = 0; j0 < nn || j0 == 0; j0 += 32) {
            pair_setup(j0);
            Powers<T> pw;
            pw.set(ux, uy, uz);
            for (int m = 0; m < P.nmus; m++) fwd_mu<T>(P.kmu[m], fr[m * 32 + lane], pw, Md + P.doff[m], lane);
        }
        __syncwarp();
        for (int i = lane; i < P.nb; i += 32) M[i] = Md[P.basic_dense[i]];
        __syncwarp();

        // ---- products, by dependency depth ---------------------------------------------------
        for (int lev = 0; lev < P.nlev; lev++) {
            for (int d = P.fwd_lev_off[lev] + lane; d < P.fwd_lev_off[lev + 1]; d += 32) {
                const int4 ds = P.fwd_dst[d];
                T acc = T(0);
                for (int r = ds.y; r < ds.z; r++) {
                    const int2 row = P.fwd_rows[r];
                    acc = fma(T(row.y) * M[row.x & 0xffff], M[row.x >> 16], acc);
                }
                M[ds.x] += acc;
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
                T acc = T(0);
                for (int e = ms.y; e < ms.z; e++) {
                    const int2 en = P.rev_ents[e];
                    acc = fma(T(en.y) * Eb[en.x >> 16], M[en.x & 0xffff], acc);
                }
                Eb[ms.x] += acc;
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
            Powers<T> pw;
            pw.set(ux, uy, uz);
            T gx = T(0), gy = T(0), gz = T(0);
            for (int m = 0; m < P.nmus; m++) {
                T Pv = T(0), Gx = T(0), Gy = T(0), Gz = T(0);
                eval_mu<T>(P.kmu[m], E4 + 4 * P.doff[m], pw, Pv, Gx, Gy, Gz);
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

template <typename T, int MODE>
static int launch_mtp(const ai2b_mtp_program *prog, MtpArgs<T> A, void *ws, size_t ws_bytes, cudaStream_t st)
{
    const MtpProgramDev &P = prog->dev;
    AI2B_REQUIRE(A.cs >= 1 && A.cs <= 64, AI2B_ERR_INVALID, "chebyshev_size %d outside 1..64", A.cs);
    AI2B_REQUIRE(A.B >= 0 && A.npad >= 0 && A.umax >= 0 && A.ntypes >= 1 && A.nghost >= 0, AI2B_ERR_INVALID, "negative size");
    if (A.B == 0 || A.npad == 0) return AI2B_OK;
    AI2B_REQUIRE(ws && ws_bytes >= ai2b_mtp_workspace_bytes(prog, A.B, A.npad), AI2B_ERR_WORKSPACE,
                 "MTP workspace too small: %zu < %zu bytes", ws_bytes, ai2b_mtp_workspace_bytes(prog, A.B, A.npad));
    int *prefix = reinterpret_cast<int *>(ws);
    A.prefix = prefix;
    prefix_binum_kernel<<<1, 256, 0, st>>>(A.binum, A.B, prefix);
    AI2B_CUDA(cudaGetLastError());

    const size_t smem = sizeof(T) * (size_t)mtp_warp_elems(P) * MTP_WARPS;
    AI2B_REQUIRE(smem <= 227 * 1024, AI2B_ERR_UNSUPPORTED, "MTP tables need %zu bytes of shared memory per block", smem);
    auto kern = mtp_atom_kernel<T, MODE>;
    static size_t configured = 0;   // per instantiation
    if (smem > configured) {
        AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    int per_sm = 0;
    AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MTP_WARPS * 32, smem));
    if (per_sm < 1) per_sm = 1;
    const long slots = (long)A.B * A.npad;
    long blocks = (long)sm_count() * per_sm;
    const long need = (slots + MTP_WARPS - 1) / MTP_WARPS;
    if (blocks > need) blocks = need;
    kern<<<(unsigned)blocks, MTP_WARPS * 32, smem, st>>>(P, A);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" size_t ai2b_mtp_workspace_bytes(const ai2b_mtp_program *prog, int batch_size, int natoms_pad)
{
    (void)prog; (void)natoms_pad;
    return (((size_t)(batch_size > 0 ? batch_size : 0) + 1) * sizeof(int) + 255) & ~size_t(255);
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
        MtpArgs<T> A{etot, force, virial, nullptr, coeffs, lin, bias, qs, binum, bilist, numneigh, firstneigh, \
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
        MtpArgs<T> A{nullptr, nullptr, nullptr, desc, coeffs, nullptr, nullptr, nullptr, binum, bilist,        \
                     numneigh, firstneigh, types, rcs, nullptr, B, npad, ntypes, umax, nghost, cs, scaling,    \
                     rmax, rmin};                                                                              \
        return launch_mtp<T, MODE_DESC>(prog, A, ws, ws_bytes, st);                                            \
    }

AI2B_DEF_MTP(f64, double)
AI2B_DEF_MTP(f32, float)
