// Device and host pieces shared by the linear-MTP kernel files (energy/force and loss gradient).
#pragma once
#include "mtp_poly.cuh"

namespace ai2b {

constexpr int MTP_WARPS = 4;      // warps (atoms in flight) per block of the per-atom kernels
constexpr int MTP_CWARPS = 32;    // warps per block of the contraction kernel

enum MtpMode { MODE_EFV = 0, MODE_EF = 1, MODE_DESC = 2 };

template <typename T>
struct MtpArgs {
    T *etot, *force, *virial, *desc;
    const T *coeffs, *lin, *bias, *qs;
    const T *coeffs_pad;   // [ntypes*ntypes][nmus][CSP] zero-padded copy of coeffs (workspace)
    const int *binum, *bilist, *numneigh, *firstneigh, *types;
    const T *rcs;
    const int *prefix;     // [B+1] exclusive prefix sum of binum (workspace)
    T *Mb, *Eb;            // basic moments / their adjoints, in alpha_index_basic order (workspace):
                           // [atoms][nbp], or [tile][nbp][32 atoms] when `tiled` is set
    int B, npad, ntypes, umax, nghost, cs, ndp, nbp;
    T scaling, rmax, rmin;
    int tiled = 0;
    int zero_outputs = 0;   // 1: etot, force and virial are zeroed by the set-up launch; 2: by the forward kernel (no set-up launch)
};

// Inputs and outputs of the loss-gradient path (mtp_loss.cu).
template <typename T>
struct LossArgs {
    const T *e_ml, *e_dft, *f_ml, *f_dft, *v_ml, *v_dft;   // v_* NULL: energy + force loss
    T *dcoeffs, *dlinear, *dbias;                           // [B,ncoef], [B,ns], [B,ntypes]
    T *Db, *Xb;                                             // [atoms][nbp] workspace rows
    T ew, fw, vw;
    int ncoef;
};

// pair weight vector p of the loss gradient
template <typename T>
__device__ __forceinline__ void pair_weight(const MtpArgs<T> &A, const LossArgs<T> &L, int b, int n, int ci, int nj, T x, T y, T z,
                                            T &px, T &py, T &pz)
{
    const T cf = T(2) * L.fw / T(3 * n);
    const T *fm = L.f_ml + (size_t)b * (A.npad + A.nghost) * 3, *fd = L.f_dft + (size_t)b * A.npad * 3;
    px = cf * ((fm[3 * ci + 0] - fd[3 * ci + 0]) - (fm[3 * nj + 0] - fd[3 * nj + 0]));
    py = cf * ((fm[3 * ci + 1] - fd[3 * ci + 1]) - (fm[3 * nj + 1] - fd[3 * nj + 1]));
    pz = cf * ((fm[3 * ci + 2] - fd[3 * ci + 2]) - (fm[3 * nj + 2] - fd[3 * nj + 2]));
    if (L.v_ml) {
        const T cv = T(2) * L.vw / T(9 * n);
        const T *vm = L.v_ml + 9 * b, *vd = L.v_dft + 9 * b;
        px -= cv * ((vm[0] - vd[0]) * x + (vm[1] - vd[1]) * y + (vm[2] - vd[2]) * z);
        py -= cv * ((vm[3] - vd[3]) * x + (vm[4] - vd[4]) * y + (vm[5] - vd[5]) * z);
        pz -= cv * ((vm[6] - vd[6]) * x + (vm[7] - vd[7]) * y + (vm[8] - vd[8]) * z);
    }
}

// Lanes-as-atoms forward / force kernels (mtp_atoms.cu): available for the tables they are compiled for.
bool mtp_atoms_supported(const MtpProgramDev &P, int ntypes, int cs, size_t elem, long atom_ids);
template <typename T> int mtp_fwd_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, cudaStream_t st);
template <typename T, int MODE> int mtp_force_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, cudaStream_t st);
// directional derivatives of the basic moments along the loss gradient's pair weights -> L.Db (tiled)
template <typename T> int mtp_dfwd_atoms(const MtpProgramDev &P, const MtpArgs<T> &A, const LossArgs<T> &L, cudaStream_t st);

// exclusive prefix sum of binum -> prefix[0..B]; one block
static __device__ __forceinline__ void prefix_binum_block(const int *__restrict__ binum, int B, int *__restrict__ prefix)
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

// Outputs the set-up launch zeroes (instead of one memset per array ahead of it).
template <typename T>
struct MtpZero {
    T *p[3] = {nullptr, nullptr, nullptr};
    size_t n[3] = {0, 0, 0};
};

// Set-up of one call in a single launch of 256-thread blocks: block 0 writes the structures'
// atom offsets, the next blocks copy the radial coefficients into rows zero-padded to csp entries
// (no such blocks are launched when the rows already have that length), the rest zero the outputs.
template <typename T>
__global__ void mtp_prep_kernel(const int *__restrict__ binum, int B, int *__restrict__ prefix, const T *__restrict__ c,
                                T *__restrict__ out, int rows, int cs, int csp, int pad_blocks, MtpZero<T> Z)
{
    if (blockIdx.x == 0) {
        prefix_binum_block(binum, B, prefix);
        return;
    }
    if ((int)blockIdx.x <= pad_blocks) {
        int i = (blockIdx.x - 1) * blockDim.x + threadIdx.x;
        if (i >= rows * csp) return;
        int r = i / csp, k = i % csp;
        out[i] = k < cs ? c[r * cs + k] : T(0);
        return;
    }
    const size_t nz = gridDim.x - 1 - pad_blocks;
    const size_t i0 = (size_t)(blockIdx.x - 1 - pad_blocks) * blockDim.x + threadIdx.x;
#pragma unroll
    for (int a = 0; a < 3; a++)
        for (size_t i = i0; i < Z.n[a]; i += nz * blockDim.x) Z.p[a][i] = T(0);
}

// Launches the set-up kernel; returns the coefficient table the evaluation kernels should read.
template <typename T>
static const T *mtp_prepare(const int *binum, int B, int *prefix, const T *coeffs, T *cpad, int rows, int cs, int csp, cudaStream_t st,
                            const MtpZero<T> &Z = MtpZero<T>())
{
    // the kernels read coefficient pairs with one vector load
    const bool pad = cs != csp || (reinterpret_cast<size_t>(coeffs) % (2 * sizeof(T))) != 0;
    const int pad_blocks = pad ? (rows * csp + 255) / 256 : 0;
    const size_t nzero = Z.n[0] + Z.n[1] + Z.n[2];
    size_t zb = (nzero + 4 * 256 - 1) / (4 * 256);      // four elements per thread
    if (zb > 4096) zb = 4096;
    mtp_prep_kernel<T><<<1 + pad_blocks + (unsigned)zb, 256, 0, st>>>(binum, B, prefix, coeffs, cpad, rows, cs, csp, pad_blocks, Z);
    return pad ? cpad : coeffs;
}

// Atoms of the call. A single structure needs no offset table (the set-up launch that writes it may then be left out).
template <typename T>
__device__ __forceinline__ int total_atoms(const MtpArgs<T> &A) { return A.B == 1 ? A.binum[0] : A.prefix[A.B]; }

// structure index of flat atom t: largest b with prefix[b] <= t
__device__ __forceinline__ int find_structure(const int *__restrict__ prefix, int B, int t)
{
    int lo = 0, hi = B;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (prefix[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// One neighbour per lane: geometry and the radial functions of all mu (into shared memory).
template <typename T, int CSP, bool DERIV>
struct PairState {
    T x, y, z, ux, uy, uz, rinv;
    int nj;
    bool act;
    __device__ __forceinline__ void setup(const MtpProgramDev &P, const MtpArgs<T> &A, const T *rc, const int *fn, const int *types,
                                          int ti, int nn, int j, int lane, T *fr, T *fdv, int frs = 32)
    {
        act = j < nn;
        x = y = z = T(0);
        nj = 0;
        if (act) {
            x = rc[3 * j]; y = rc[3 * j + 1]; z = rc[3 * j + 2];
            nj = fn[j];
        }
        compute(P, A, types, ti, lane, fr, fdv, frs);
    }
    // x, y, z, nj and act (= the slot holds a neighbour) are already set
    // tj_pre >= 0: the neighbour's type has been looked up already
    __device__ __forceinline__ void compute(const MtpProgramDev &P, const MtpArgs<T> &A, const int *types, int ti, int lane, T *fr,
                                            T *fdv, int frs = 32, int tj_pre = -1)
    {
        using V2 = typename Vec2<T>::type;
        const int tj_early = tj_pre >= 0 ? tj_pre : (act ? types[nj] : 0);   // in flight during the square root
        const T r = gsqrt(x * x + y * y + z * z);
        act = act && (r <= A.rmax) && (r > T(0));
        const int tj = act ? tj_early : 0;
        rinv = act ? T(1) / r : T(0);
        ux = x * rinv; uy = y * rinv; uz = z * rinv;
        T q[CSP], dq[CSP];
        mtp_radial_basis<T, CSP>(act ? r : A.rmax, A.rmax, A.rmin, A.scaling, q, dq);
        const T *crow = A.coeffs_pad + (size_t)(ti * A.ntypes + tj) * P.nmus * CSP;
        for (int m = 0; m < P.nmus; m++) {
            T f = T(0), fd = T(0);
#pragma unroll
            for (int k = 0; k < CSP; k += 2) {
                const V2 c2 = *reinterpret_cast<const V2 *>(crow + m * CSP + k);
                f = fma(c2.x, q[k], f);
                f = fma(c2.y, q[k + 1], f);
                if (DERIV) { fd = fma(c2.x, dq[k], fd); fd = fma(c2.y, dq[k + 1], fd); }
            }
            fr[m * frs + lane] = act ? f : T(0);      // frs: row stride of the per-mu arrays
            if (DERIV) fdv[m * frs + lane] = act ? fd : T(0);
        }
    }
};


// ---------------------------------------------------------------------------------------------
// host helpers
// ---------------------------------------------------------------------------------------------
static inline size_t up256(size_t n) { return (n + 255) & ~size_t(255); }
static inline int ndense_pad(const MtpProgramDev &P) { return (P.ndense + 3) & ~3; }
static inline int nbasic_pad(const MtpProgramDev &P) { return (P.nb + 3) & ~3; }

struct MtpWs {
    size_t prefix, cpad, mb, eb, total;
};
static inline MtpWs mtp_ws_layout(const MtpProgramDev &P, int B, int npad, int ntypes, size_t elem)
{
    MtpWs L;
    // rounded up to whole tiles of 32 atoms (the tiled layout of the basic moments)
    const size_t atoms = ((size_t)(B > 0 ? B : 0) * (npad > 0 ? npad : 0) + 31) & ~size_t(31);
    L.prefix = 0;
    L.cpad = up256(((size_t)(B > 0 ? B : 0) + 1) * sizeof(int));
    L.mb = L.cpad + up256((size_t)ntypes * ntypes * P.nmus * 16 * elem);
    L.eb = L.mb + up256(atoms * nbasic_pad(P) * elem);
    // the adjoints of a tile may be kept in dense monomial order (ndense >= basic moments)
    const size_t erow = (size_t)(ndense_pad(P) > nbasic_pad(P) ? ndense_pad(P) : nbasic_pad(P));
    L.total = L.eb + up256(atoms * erow * elem);
    return L;
}

}  // namespace ai2b
