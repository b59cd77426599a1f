// Cell-list neighbour build on sm_100a, bit-compatible with the reference's CPU list.
//
// Reference semantics (source/nblist/include/structure.h:589-710, binLinkedList.h:658-696,983-1031,
// neighborList.h:532-578): the cell is replicated over images n_k in [-e_k, e_k],
// e_k = ceil(rcut / interplanar distance) on periodic axes; image position
// ((r_j + a0*nx) + a1*ny) + a2*nz; (j, n) is a neighbour of i iff 1e-3 < d2 < rcut^2 with
// d = image - r_i (squares accumulated in double when T = float); row = index j, rcs = d;
// padding -1 / 0. The order inside a row is not part of the contract.
//
// Here: atoms are binned once by their fractional coordinates wrapped into the cell (bins at
// least rcut / 2 thick, so a centre looks at 5 x 5 x 5 bins: 125 candidates at one atom per bin
// where bins of a full cutoff give 216), each centre atom is handled by one warp that walks the
// neighbouring bins with lanes over candidate atoms, applies the reference's predicate with the
// reference's operation order (no FMA contraction), and compacts hits with a warp ballot. Bins
// that follow one another along the third axis are contiguous in bin order, so the 5 bins of a
// column are ONE range of atoms: the warp's table holds 25 ranges (plus the wrapped remainders
// for centres next to a periodic face) instead of 125 bins. The padded row is written once, by
// the same warp. The launches of one build (set-up, count, scan, fill, build) go out as a chain
// (launch_chained() in common.cuh), so each becomes resident while the one before it drains.
#include "common.cuh"
#include <cooperative_groups.h>

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace ai2b {

template <typename T> struct Vec4;
template <> struct Vec4<double> { using type = double4; };
template <> struct Vec4<float> { using type = float4; };
// Lattice wraps packed into one word, 10 bits per axis with bias 512: sums and differences of packed
// words are field-wise sums and differences as long as every true field stays inside +-511. The fourth
// component of a bin-ordered position carries the atom's packed wrap.
constexpr int NB_WRAP_MAX = 127;
constexpr int NB_SUB = 2;            // bins per cutoff length along each axis
constexpr int NB_PACK_ZERO = 512 | (512 << 10) | (512 << 20);
__host__ __device__ inline int nb_pack3(int a, int b, int c) { return (a + 512) | ((b + 512) << 10) | ((c + 512) << 20); }
__device__ __forceinline__ float nb_bits_to(float, int v) { return __int_as_float(v); }
__device__ __forceinline__ double nb_bits_to(double, int v) { return __longlong_as_double((long long)v); }
__device__ __forceinline__ int nb_bits_of(float v) { return __float_as_int(v); }
__device__ __forceinline__ int nb_bits_of(double v) { return (int)__double_as_longlong(v); }

struct NbGrid {          // lives in the workspace; written by nb_grid_kernel
    int nb[3];           // bins per fractional axis
    int R[3];            // bins to search on each side
    int total;
    int zmerge;          // the bins of a column along the third axis are taken as one range (needs nb[2] >= 2 R[2] + 1 if periodic)
    float pre_lo, pre_hi;   // single-precision pre-test on positions wrapped into the cell: 1e-3 and rcut^2 widened by its rounding error
    int bigwrap;         // set by nb_count_kernel when an atom lies more than NB_WRAP_MAX periods outside the cell
    double lo[3];        // non-periodic axes: lowest fractional coordinate
    double scale[3];     // bin = (s - lo) * scale
};

template <typename T>
struct NbParams {
    T cell[9];           // rows = lattice vectors (as given, type T)
    double inv[9];       // inverse cell: frac_k = sum_c r_c * inv[3*c + k]
    double dplane[3];    // interplanar distances (double, for bin sizing only)
    int per[3], e[3];
    int nbh[3];          // bins of the periodic axes (host-computed); cap for the others
    double rcut_m;       // rcut with a safety margin, for bin sizing
    double rc2;          // rcut^2 as the reference forms it
    float rc2_lo, rc2_hi, eps_lo, eps_hi;   // the two thresholds -/+ 2e-6 relative (float builds)
    int n, umax, maxbins;
    int ncentre;         // rows are built for atoms [cbegin, ncentre); the rest are neighbours only (ghosts)
    int cbegin;          // first centre; its row is row 0 of the outputs
};

__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }

// fractional -> Cartesian with the reference's operation order (structure.h:561-581)
template <typename T>
__global__ void nb_frac2cart_kernel(NbParams<T> P, const T *__restrict__ frac, T *__restrict__ cart)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P.n) return;
    T f0 = frac[3 * i], f1 = frac[3 * i + 1], f2 = frac[3 * i + 2];
#pragma unroll
    for (int c = 0; c < 3; c++)
        cart[3 * i + c] = add_rn(add_rn(mul_rn(f0, P.cell[c]), mul_rn(f1, P.cell[3 + c])), mul_rn(f2, P.cell[6 + c]));
}

template <typename T>
__device__ __forceinline__ void frac_of(const NbParams<T> &P, const T *pos, int i, double *s)
{
    double x = pos[3 * i], y = pos[3 * i + 1], z = pos[3 * i + 2];
#pragma unroll
    for (int k = 0; k < 3; k++) s[k] = x * P.inv[k] + y * P.inv[3 + k] + z * P.inv[6 + k];
}

__device__ __forceinline__ unsigned long long enc_double(double d)
{
    unsigned long long u = (unsigned long long)__double_as_longlong(d);
    return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}
__device__ __forceinline__ double dec_double(unsigned long long u)
{
    u = (u >> 63) ? (u & 0x7fffffffffffffffull) : ~u;
    return __longlong_as_double((long long)u);
}

// extents of the fractional coordinates (only launched when an axis is not periodic)
template <typename T>
__global__ void nb_extent_kernel(NbParams<T> P, const T *__restrict__ pos, unsigned long long *__restrict__ ext)
{
    double lo[3] = {1e300, 1e300, 1e300}, hi[3] = {-1e300, -1e300, -1e300};
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < P.n; i += gridDim.x * blockDim.x) {
        double s[3];
        frac_of(P, pos, i, s);
#pragma unroll
        for (int k = 0; k < 3; k++) { lo[k] = fmin(lo[k], s[k]); hi[k] = fmax(hi[k], s[k]); }
    }
#pragma unroll
    for (int k = 0; k < 3; k++) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            lo[k] = fmin(lo[k], __shfl_xor_sync(FULL_MASK, lo[k], o));
            hi[k] = fmax(hi[k], __shfl_xor_sync(FULL_MASK, hi[k], o));
        }
        if ((threadIdx.x & 31) == 0) {
            atomicMin(ext + k, enc_double(lo[k]));
            atomicMax(ext + 3 + k, enc_double(hi[k]));
        }
    }
}

__global__ void nb_init_kernel(unsigned long long *ext, int *status)
{
    if (threadIdx.x < 3) { ext[threadIdx.x] = ~0ull; ext[3 + threadIdx.x] = 0ull; }
    if (threadIdx.x < 2) status[threadIdx.x] = 0;
}

// Bounds of the single-precision pre-test. It works on float copies of the positions wrapped into the cell plus
// the float image shift of the candidate's bin; with coordinates bounded by reach = sum_k (max|s_k| + 2) |a_k| every
// difference carries at most ~6 ulp(reach), so d^2 near the cutoff is off by less than 64 eps reach rcut.
template <typename T>
__host__ __device__ inline void nb_pretest_bounds(const NbParams<T> &P, const double *lo, const double *scale_or_hi, bool have_hi, NbGrid *g)
{
    double reach = 0.0;
    for (int k = 0; k < 3; k++) {
        const double len = sqrt((double)P.cell[3 * k] * (double)P.cell[3 * k] + (double)P.cell[3 * k + 1] * (double)P.cell[3 * k + 1] +
                                (double)P.cell[3 * k + 2] * (double)P.cell[3 * k + 2]);
        double smax = 1.0;
        if (!P.per[k]) {
            const double hi = have_hi ? scale_or_hi[k] : lo[k] + g->nb[k] / g->scale[k];
            smax = fmax(fabs(lo[k]), fabs(hi));
        }
        reach += (smax + 2.0) * len;
    }
    const double rc = sqrt(P.rc2);
    const double err = 64.0 * 6e-8 * reach * rc + 1e-6 * P.rc2;
    g->pre_hi = (float)((P.rc2 + err) * (1.0 + 1e-6));
    g->pre_lo = (float)((1e-3 - err) * (1.0 - 1e-6));
}

template <typename T>
__global__ void nb_grid_kernel(NbParams<T> P, const unsigned long long *__restrict__ ext, NbGrid *__restrict__ g)
{
    if (threadIdx.x != 0) return;
    long total = 1;
    for (int k = 0; k < 3; k++) {
        if (P.per[k]) {
            g->nb[k] = P.nbh[k];
            double t = P.dplane[k] / P.nbh[k];
            g->R[k] = (int)ceil(P.rcut_m / t);
            g->lo[k] = 0.0;
            g->scale[k] = (double)P.nbh[k];
        } else {
            double lo = dec_double(ext[k]), hi = dec_double(ext[3 + k]);
            double span = fmax(hi - lo, 1e-12);
            int nb = (int)floor(span * P.dplane[k] * NB_SUB / P.rcut_m);
            nb = max(1, min(nb, P.nbh[k]));
            g->nb[k] = nb;
            g->R[k] = NB_SUB;
            g->lo[k] = lo;
            g->scale[k] = nb / span;
        }
        total *= g->nb[k];
    }
    g->total = (int)total;   // <= maxbins by construction of nbh
    g->zmerge = (!P.per[2] || g->nb[2] >= 2 * g->R[2] + 1) ? 1 : 0;
    g->bigwrap = 0;
    nb_pretest_bounds(P, g->lo, nullptr, false, g);
}

template <typename T>
__device__ __forceinline__ void bin_of(const NbParams<T> &P, const NbGrid &g, const double *s, int *b, int *w)
{
#pragma unroll
    for (int k = 0; k < 3; k++) {
        if (P.per[k]) {
            double fl = floor(s[k]);
            w[k] = (int)fl;
            int bb = (int)((s[k] - fl) * g.scale[k]);
            b[k] = min(max(bb, 0), g.nb[k] - 1);
        } else {
            w[k] = 0;
            int bb = (int)((s[k] - g.lo[k]) * g.scale[k]);
            b[k] = min(max(bb, 0), g.nb[k] - 1);
        }
    }
}

// pass 1: bin index + lattice wrap of every atom, bin populations
template <typename T>
__global__ void nb_count_kernel(NbParams<T> P, NbGrid *gp, const T *__restrict__ pos,
                                int4 *__restrict__ ainfo, int *__restrict__ bin_count)
{
    chain_release();
    chain_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P.n) return;
    const NbGrid g = *gp;
    double s[3];
    int b[3], w[3];
    frac_of(P, pos, i, s);
    bin_of(P, g, s, b, w);
    int bin = (b[0] * g.nb[1] + b[1]) * g.nb[2] + b[2];
    ainfo[i] = make_int4(bin, w[0], w[1], w[2]);
    if (abs(w[0]) > NB_WRAP_MAX || abs(w[1]) > NB_WRAP_MAX || abs(w[2]) > NB_WRAP_MAX) gp->bigwrap = 1;
    atomicAdd(bin_count + bin, 1);
}

// exclusive scan of bin_count[0..total) -> bin_start[0..total], three small kernels
constexpr int SCAN_BLOCK = 1024;
__global__ void nb_scan1_kernel(const NbGrid *__restrict__ gp, const int *__restrict__ in, int *__restrict__ out, int *__restrict__ bsum)
{
    __shared__ int ws[32];
    const int total = gp->total;
    int i = blockIdx.x * SCAN_BLOCK + threadIdx.x;
    if (blockIdx.x * SCAN_BLOCK >= total + 1) return;
    int v = i < total ? in[i] : 0, inc = v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, inc, o); if (lane >= o) inc += n; }
    if (lane == 31) ws[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = ws[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, w, o); if (lane >= o) w += n; }
        ws[lane] = w;
    }
    __syncthreads();
    int excl = inc - v + (warp > 0 ? ws[warp - 1] : 0);
    if (i <= total) out[i] = excl;
    if (threadIdx.x == SCAN_BLOCK - 1) bsum[blockIdx.x] = excl + v;
}
__global__ void nb_scan2_kernel(const NbGrid *__restrict__ gp, int *__restrict__ bsum)
{
    // serial-by-chunks exclusive scan of the block sums (at most a few thousand entries)
    __shared__ int ws[32];
    __shared__ int carry;
    const int nblk = (gp->total + 1 + SCAN_BLOCK - 1) / SCAN_BLOCK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < nblk; base += SCAN_BLOCK) {
        int i = base + threadIdx.x;
        int v = i < nblk ? bsum[i] : 0, inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, inc, o); if (lane >= o) inc += n; }
        if (lane == 31) ws[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = ws[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, w, o); if (lane >= o) w += n; }
            ws[lane] = w;
        }
        __syncthreads();
        int excl = carry + inc - v + (warp > 0 ? ws[warp - 1] : 0);
        if (i < nblk) bsum[i] = excl;
        __syncthreads();
        if (threadIdx.x == SCAN_BLOCK - 1) carry = excl + v;
        __syncthreads();
    }
}
__global__ void nb_scan3_kernel(const NbGrid *__restrict__ gp, int *__restrict__ out, const int *__restrict__ bsum, int *__restrict__ cursor)
{
    const int total = gp->total;
    int i = blockIdx.x * SCAN_BLOCK + threadIdx.x;
    if (i > total) return;
    int v = out[i] + bsum[blockIdx.x];
    out[i] = v;
    if (i < total) cursor[i] = v;
}


// all axes periodic: grid parameters are known on the host, so one kernel zeroes the bin counters,
// resets the status words and writes the grid description
__global__ void nb_setup_periodic_kernel(NbGrid host_grid, NbGrid *__restrict__ g, int *__restrict__ count, int ncount, int *__restrict__ status)
{
    chain_release();
    chain_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < ncount) count[i] = 0;
    if (i == 0) {
        status[0] = 0; status[1] = 0;
        *g = host_grid;
    }
}

// exclusive scan by one block (grids of up to 64 K bins): bin_start and cursor. Chunks of SCAN_BLOCK * SCAN_ITEMS
// counters: loaded along the array into shared memory, every thread scans SCAN_ITEMS consecutive counters by itself
// (rows padded by one word, so the threads' rows start in different banks), ONE block-wide scan of the thread totals,
// and the results leave along the array again.
constexpr int SCAN_ITEMS = 8;
__global__ void __launch_bounds__(SCAN_BLOCK) nb_scan_small_kernel(const NbGrid *__restrict__ gp, const int *__restrict__ in, int *__restrict__ out,
                                                                  int *__restrict__ cursor)
{
    chain_release();
    chain_wait();
    __shared__ int buf[SCAN_BLOCK * (SCAN_ITEMS + 1)];
    __shared__ int ws[32];
    const int total = gp->total;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int carry = 0;      // every thread keeps the running total
    for (int base = 0; base <= total; base += SCAN_BLOCK * SCAN_ITEMS) {
#pragma unroll
        for (int k = 0; k < SCAN_ITEMS; k++) {
            const int e = k * SCAN_BLOCK + threadIdx.x, i = base + e;
            buf[(e / SCAN_ITEMS) * (SCAN_ITEMS + 1) + e % SCAN_ITEMS] = i < total ? in[i] : 0;
        }
        __syncthreads();
        int v[SCAN_ITEMS], sum = 0;
#pragma unroll
        for (int k = 0; k < SCAN_ITEMS; k++) {
            v[k] = sum;                                         // exclusive within the thread
            sum += buf[threadIdx.x * (SCAN_ITEMS + 1) + k];
        }
        int inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, inc, o); if (lane >= o) inc += n; }
        if (lane == 31) ws[warp] = inc;
        __syncthreads();
        int w = ws[lane];                                       // every warp scans the 32 warp totals itself
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, w, o); if (lane >= o) w += n; }
        const int before = __shfl_sync(FULL_MASK, w, max(warp - 1, 0));
        const int all = __shfl_sync(FULL_MASK, w, 31);
        const int off = carry + inc - sum + (warp > 0 ? before : 0);
#pragma unroll
        for (int k = 0; k < SCAN_ITEMS; k++) buf[threadIdx.x * (SCAN_ITEMS + 1) + k] = off + v[k];
        carry += all;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SCAN_ITEMS; k++) {
            const int e = k * SCAN_BLOCK + threadIdx.x, i = base + e;
            const int r = buf[(e / SCAN_ITEMS) * (SCAN_ITEMS + 1) + e % SCAN_ITEMS];
            if (i <= total) out[i] = r;
            if (i < total) cursor[i] = r;
        }
        __syncthreads();     // the buffer and the warp totals are reused by the next chunk
    }
}

// The same scan by a cluster of SCAN_CLUSTER blocks (grids of up to SCAN_CLUSTER * SCAN_BLOCK * SCAN_ITEMS bins): every
// block scans one chunk, the block totals are read from the other blocks' shared memory.
constexpr int SCAN_CLUSTER = 4;
__global__ void __cluster_dims__(SCAN_CLUSTER, 1, 1) __launch_bounds__(SCAN_BLOCK)
nb_scan_cluster_kernel(const NbGrid *__restrict__ gp, const int *__restrict__ in, int *__restrict__ out, int *__restrict__ cursor)
{
    chain_release();
    chain_wait();
    namespace cg = cooperative_groups;
    __shared__ int buf[SCAN_BLOCK * (SCAN_ITEMS + 1)];
    __shared__ int ws[32];
    __shared__ int block_total;
    cg::cluster_group cl = cg::this_cluster();
    const int rank = (int)cl.block_rank();
    const int total = gp->total;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int base = rank * SCAN_BLOCK * SCAN_ITEMS;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int e = k * SCAN_BLOCK + threadIdx.x, i = base + e;
        buf[(e / SCAN_ITEMS) * (SCAN_ITEMS + 1) + e % SCAN_ITEMS] = i < total ? in[i] : 0;
    }
    __syncthreads();
    int v[SCAN_ITEMS], sum = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        v[k] = sum;
        sum += buf[threadIdx.x * (SCAN_ITEMS + 1) + k];
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, inc, o); if (lane >= o) inc += n; }
    if (lane == 31) ws[warp] = inc;
    __syncthreads();
    int w = ws[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, w, o); if (lane >= o) w += n; }
    const int before = __shfl_sync(FULL_MASK, w, max(warp - 1, 0));
    if (threadIdx.x == 0) block_total = __shfl_sync(FULL_MASK, w, 31);
    else (void)__shfl_sync(FULL_MASK, w, 31);
    cl.sync();
    int carry = 0;
    for (int r = 0; r < rank; r++) carry += *cl.map_shared_rank(&block_total, r);
    const int off = carry + inc - sum + (warp > 0 ? before : 0);
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) buf[threadIdx.x * (SCAN_ITEMS + 1) + k] = off + v[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int e = k * SCAN_BLOCK + threadIdx.x, i = base + e;
        const int r = buf[(e / SCAN_ITEMS) * (SCAN_ITEMS + 1) + e % SCAN_ITEMS];
        if (i <= total) out[i] = r;
        if (i < total) cursor[i] = r;
    }
    cl.sync();      // no block leaves while another may still read its total
}

// pass 2: atoms into bin order: position (type T) + {original index, wrap}
template <typename T>
__global__ void nb_fill_kernel(NbParams<T> P, const T *__restrict__ pos, const int4 *__restrict__ ainfo,
                               int *__restrict__ cursor, typename Vec4<T>::type *__restrict__ spos, int4 *__restrict__ sinfo,
                               float4 *__restrict__ sposw, int4 *__restrict__ sbin, const NbGrid *__restrict__ gp)
{
    chain_release();
    chain_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P.n) return;
    const int4 a = ainfo[i];
    int k = atomicAdd(cursor + a.x, 1);
    {   // bin coordinates of the atom, so that the row pass needs no integer division per centre
        const int nb2 = gp->nb[2], nb1 = gp->nb[1];
        const int t = a.x / nb2;
        sbin[k] = make_int4(t / nb1, t % nb1, a.x % nb2, a.x);
    }
    typename Vec4<T>::type p;
    p.x = pos[3 * i]; p.y = pos[3 * i + 1]; p.z = pos[3 * i + 2];
    p.w = nb_bits_to(T(0), nb_pack3(a.y, a.z, a.w));   // meaningful while no wrap exceeds NB_WRAP_MAX (else unused)
    spos[k] = p;
    sinfo[k] = make_int4(i, a.y, a.z, a.w);
    // single-precision copy of the position brought into the cell, for the pre-test
    const double w0 = a.y, w1 = a.z, w2 = a.w;
    float4 q;
    q.x = (float)((double)p.x - (w0 * (double)P.cell[0] + w1 * (double)P.cell[3] + w2 * (double)P.cell[6]));
    q.y = (float)((double)p.y - (w0 * (double)P.cell[1] + w1 * (double)P.cell[4] + w2 * (double)P.cell[7]));
    q.z = (float)((double)p.z - (w0 * (double)P.cell[2] + w1 * (double)P.cell[5] + w2 * (double)P.cell[8]));
    q.w = 0.f;
    sposw[k] = q;
}

constexpr int NB_WARPS = 8;
constexpr int NB_CAND = 512;

// pass 3: one warp per centre atom (taken in bin order, so neighbouring warps share bins)
// TO = element type of the rcs rows (T, or float rows from double positions: what an MD host that keeps
// double coordinates and a single-precision model does on the CPU)
template <typename T, typename TO>
__global__ void __launch_bounds__(NB_WARPS * 32, 4)
nb_build_kernel(NbParams<T> P, const NbGrid *__restrict__ gp, const int *__restrict__ bin_start,
                const int4 *__restrict__ ainfo, const typename Vec4<T>::type *__restrict__ spos,
                const int4 *__restrict__ sinfo, const float4 *__restrict__ sposw, const int4 *__restrict__ sbin, int *__restrict__ numneigh,
                int *__restrict__ firstneigh, TO *__restrict__ rcs, int *__restrict__ status)
{
    chain_release();
    chain_wait();
    __shared__ int s_start[NB_WARPS][32], s_pre[NB_WARPS][33], s_shift[NB_WARPS][32];
    __shared__ float4 s_sv[NB_WARPS][32];      // image shift of a table entry as a single-precision vector
    // candidate c of the current group of bins -> its atom (bin order) and its bin's slot, filled by the
    // lanes that own the bins; groups with more than NB_CAND candidates search s_pre instead
    __shared__ int s_cand[NB_WARPS][NB_CAND];
    __shared__ unsigned char s_slot[NB_WARPS][NB_CAND];
    const NbGrid g = *gp;
    const bool packed = g.bigwrap == 0;   // every wrap fits the packed form
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = gridDim.x * NB_WARPS;
    const int nx = 2 * g.R[0] + 1, ny = 2 * g.R[1] + 1, nz = 2 * g.R[2] + 1;
    const bool zmerge = g.zmerge != 0;
    const int nnb_full = zmerge ? nx * ny : nx * ny * nz;   // table entries of a centre away from the third axis' faces
    const unsigned lt_mask = (1u << lane) - 1u;
    int local_max = 0;
    // merged columns: the (d0, d1) offsets of the table entries this lane builds (entry lane, entry lane + 32) never change
    int ent_d0[2] = {0, 0}, ent_d1[2] = {0, 0};
    const bool ent_fast = zmerge && nnb_full <= 64;
    if (ent_fast) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
            int kk = lane + 32 * u;
            if (kk >= nnb_full) kk -= nnb_full;          // second half of a split table: the same columns again
            if (kk >= nnb_full) kk = 0;
            ent_d0[u] = kk / ny - g.R[0];
            ent_d1[u] = kk % ny - g.R[1];
        }
    }

    // Large systems: warps take runs of up to 16 bin-ordered atoms, dealt round-robin, so consecutive centres
    // touch the same bins and candidates, while ghost regions (atoms that are neighbours only) spread over
    // all warps. Small systems: single atoms are dealt round-robin (runs would leave most warps without work).
    const int gw = blockIdx.x * NB_WARPS + warp;
    const int per_warp = (P.n + nwarps - 1) / nwarps;
    const int RUN = min(16, max(1, per_warp / 4));    // at least four runs per warp, so that the last round of runs is short
    const int nruns = (P.n + RUN - 1) / RUN;
    for (int run = gw; run < nruns; run += nwarps)
    for (int k = 0; k < RUN; k++) {
        const int a = run * RUN + k;
        if (a >= P.n) break;
        const typename Vec4<T>::type pi = spos[a];
        const float4 piw = sposw[a];
        const int4 si = sinfo[a];
        const int i = si.x;
        const int wi = nb_pack3(si.y, si.z, si.w);   // its bias is the one that survives in shift - wrap_j + wrap_i
        if (i >= P.ncentre || i < P.cbegin) continue;
        const int4 cb = sbin[a];
        const int bx = cb.x, by = cb.y, bz = cb.z;
        int count = 0;
        int *frow = firstneigh + (size_t)(i - P.cbegin) * P.umax;
        TO *rrow = rcs + (size_t)(i - P.cbegin) * P.umax * 3;

        // With merged columns a centre within R bins of a periodic face of the third axis has, per column, a second
        // range: the part of its 2R+1 bins that lies across the face (entries nnb_full .. 2 nnb_full - 1).
        const bool zsplit = zmerge && P.per[2] && (bz - g.R[2] < 0 || bz + g.R[2] >= g.nb[2]);
        const int nnb = zsplit ? 2 * nnb_full : nnb_full;
        // (the candidate table of a centre is consumed by the pre-test's in-place compaction, so it is rebuilt
        // for every centre; with bins of half a cutoff two consecutive centres rarely share a bin anyway)
        constexpr bool reuse = false;
        for (int base = 0; base < nnb; base += 32) {
            // lanes = table entries (neighbouring bins, or columns of bins) of this group
            const int k = base + lane;
            int start = 0, len = 0, shift = 0;
            float4 sv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!reuse && k < nnb) {
                const int kk = zmerge ? (k >= nnb_full ? k - nnb_full : k) : k;
                int d[3], b[3], m[3];
                if (ent_fast && base == 0) { d[0] = ent_d0[0]; d[1] = ent_d1[0]; d[2] = 0; }
                else if (ent_fast && base == 32) { d[0] = ent_d0[1]; d[1] = ent_d1[1]; d[2] = 0; }
                else if (zmerge) { d[0] = kk / ny - g.R[0]; d[1] = kk % ny - g.R[1]; d[2] = 0; }
                else { d[0] = kk / (ny * nz) - g.R[0]; d[1] = (kk / nz) % ny - g.R[1]; d[2] = kk % nz - g.R[2]; }
                b[0] = bx + d[0]; b[1] = by + d[1]; b[2] = bz + d[2];
                bool ok = true;
#pragma unroll
                for (int c = 0; c < 3; c++) {
                    if (P.per[c]) {
                        int q;   // floor(b / nb); one period off at most unless the grid is tiny
                        if (b[c] >= 0 && b[c] < g.nb[c]) q = 0;
                        else if (b[c] < 0 && b[c] >= -g.nb[c]) q = -1;
                        else if (b[c] >= g.nb[c] && b[c] < 2 * g.nb[c]) q = 1;
                        else q = b[c] >= 0 ? b[c] / g.nb[c] : -((-b[c] + g.nb[c] - 1) / g.nb[c]);
                        m[c] = q; b[c] -= q * g.nb[c];
                    } else {
                        m[c] = 0;
                        ok = ok && b[c] >= 0 && b[c] < g.nb[c];
                    }
                }
                int zlo = b[2], zhi = b[2];          // bins of the third axis this entry covers (inside the grid)
                if (zmerge) {
                    zlo = bz - g.R[2]; zhi = bz + g.R[2];
                    if (k < nnb_full) {              // the part inside the cell
                        zlo = max(zlo, 0); zhi = min(zhi, g.nb[2] - 1);
                        m[2] = 0;
                        ok = ok && zlo <= zhi;
                    } else if (zlo < 0) {            // the part below the face: bins nb + zlo .. nb - 1 of the image one period down
                        zlo += g.nb[2]; zhi = g.nb[2] - 1; m[2] = -1;
                    } else {                         // the part above the face
                        zhi -= g.nb[2]; zlo = 0; m[2] = 1;
                    }
                }
                if (ok) {
                    const int col = (b[0] * g.nb[1] + b[1]) * g.nb[2];
                    start = bin_start[col + zlo];
                    len = bin_start[col + zhi + 1] - start;
                    shift = (m[0] + 512) | ((m[1] + 512) << 10) | ((m[2] + 512) << 20);
                    // image counts are -1, 0 or 1 unless the grid is tiny: selects instead of int -> float conversions
                    auto tof = [](int v) { return v == 0 ? 0.f : v == 1 ? 1.f : v == -1 ? -1.f : (float)v; };
                    const float f0 = tof(m[0]), f1 = tof(m[1]), f2 = tof(m[2]);
                    sv.x = f0 * (float)P.cell[0] + f1 * (float)P.cell[3] + f2 * (float)P.cell[6];
                    sv.y = f0 * (float)P.cell[1] + f1 * (float)P.cell[4] + f2 * (float)P.cell[7];
                    sv.z = f0 * (float)P.cell[2] + f1 * (float)P.cell[5] + f2 * (float)P.cell[8];
                }
            }
            int total;
            if (!reuse) {
                int inc = len;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { int n = __shfl_up_sync(FULL_MASK, inc, o); if (lane >= o) inc += n; }
                total = __shfl_sync(FULL_MASK, inc, 31);
                __syncwarp();
                s_start[warp][lane] = start;
                s_pre[warp][lane] = inc - len;
                s_shift[warp][lane] = shift;
                s_sv[warp][lane] = sv;
                if (lane == 31) s_pre[warp][32] = total;
                if (total <= NB_CAND) {
                    const int pre = inc - len;
                    for (int q = 0; q < len; q++) { s_cand[warp][pre + q] = start + q; s_slot[warp][pre + q] = (unsigned char)lane; }
                }
                __syncwarp();
            } else {
                total = s_pre[warp][32];
            }

            // Pre-test, lanes = candidate atoms of the whole group: single-precision distance between the positions
            // wrapped into the cell, shifted by the entry's image vector. Candidates that are certainly outside the
            // cutoff shell drop out here without any of the image bookkeeping; the survivors are compacted in place.
            int nsurv = total;
            if (total <= NB_CAND) {
                nsurv = 0;
                for (int c0 = 0; c0 < total; c0 += 32) {
                    const int c = c0 + lane;
                    bool pass = false;
                    int aj = 0, lo = 0;
                    if (c < total) {
                        aj = s_cand[warp][c];
                        lo = s_slot[warp][c];
                        const float4 pw = sposw[aj];
                        const float4 v = s_sv[warp][lo];
                        const float dx = (pw.x + v.x) - piw.x, dy = (pw.y + v.y) - piw.y, dz = (pw.z + v.z) - piw.z;
                        const float sq = dx * dx + dy * dy + dz * dz;
                        pass = sq < g.pre_hi && sq > g.pre_lo;
                    }
                    const unsigned bal = __ballot_sync(FULL_MASK, pass);
                    __syncwarp();
                    if (pass) {
                        const int p = nsurv + __popc(bal & lt_mask);
                        s_cand[warp][p] = aj;
                        s_slot[warp][p] = (unsigned char)lo;
                    }
                    nsurv += __popc(bal);
                }
                __syncwarp();
            }

            // exact test, lanes = surviving candidates
            for (int c0 = 0; c0 < nsurv; c0 += 32) {
                const int c = c0 + lane;
                const bool have = c < nsurv;
                bool hit = false;
                int jidx = 0;
                T d0 = 0, d1 = 0, d2 = 0;
                int aj = 0, lo = 0;
                if (have) {
                    if (total <= NB_CAND) {
                        aj = s_cand[warp][c];
                        lo = s_slot[warp][c];
                    } else {
                        int hi = 32;    // largest slot with pre[slot] <= c
                        while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (s_pre[warp][mid] <= c) lo = mid; else hi = mid; }
                        aj = s_start[warp][lo] + (c - s_pre[warp][lo]);
                    }
                }
                const int sh = s_shift[warp][lo];
                typename Vec4<T>::type pj;
                pj.x = pj.y = pj.z = pj.w = T(0);
                if (have) pj = spos[aj];
                // periods between the candidate's stored position and the image this bin slot means
                int n0 = 0, n1 = 0, n2 = 0;
                bool away;       // some period is non-zero
                if (packed) {
                    // bin shift - candidate's wrap + centre's wrap, all three axes in one word
                    const int nw = sh - nb_bits_of(pj.w) + wi;
                    away = nw != NB_PACK_ZERO;
                    n0 = (nw & 1023) - 512; n1 = ((nw >> 10) & 1023) - 512; n2 = ((nw >> 20) & 1023) - 512;
                } else {
                    int4 sj = make_int4(0, 0, 0, 0);
                    if (have) sj = sinfo[aj];
                    n0 = (sh & 1023) - 512 - sj.y + si.y;
                    n1 = ((sh >> 10) & 1023) - 512 - sj.z + si.z;
                    n2 = ((sh >> 20) & 1023) - 512 - sj.w + si.w;
                    away = (n0 | n1 | n2) != 0;
                }
                const bool covered = have && (!away || (abs(n0) <= P.e[0] && abs(n1) <= P.e[1] && abs(n2) <= P.e[2]));
                T ix = pj.x, iy = pj.y, iz = pj.z;
                // The home image needs no arithmetic: x + a*0 is x bit for bit, except for x = -0.0 (whose
                // sum with +0 is +0), so exact zeros take the full path.
                const bool moved = covered && (away || pj.x == T(0) || pj.y == T(0) || pj.z == T(0));
                if (moved) {
                    const T f0 = T(n0), f1 = T(n1), f2 = T(n2);
                    ix = add_rn(add_rn(add_rn(pj.x, mul_rn(P.cell[0], f0)), mul_rn(P.cell[3], f1)), mul_rn(P.cell[6], f2));
                    iy = add_rn(add_rn(add_rn(pj.y, mul_rn(P.cell[1], f0)), mul_rn(P.cell[4], f1)), mul_rn(P.cell[7], f2));
                    iz = add_rn(add_rn(add_rn(pj.z, mul_rn(P.cell[2], f0)), mul_rn(P.cell[5], f1)), mul_rn(P.cell[8], f2));
                }
                d0 = sub_rn(ix, pi.x); d1 = sub_rn(iy, pi.y); d2 = sub_rn(iz, pi.z);
                // Reference predicate: squares accumulate in double for both types (pow(T,int) promotes
                // float), the sum is rounded to T and compared with rc^2 and 1e-3. For float a
                // single-precision sum is within a few ulp of that value, so it decides every pair outside
                // a 2e-6 relative band around the two thresholds; only pairs inside the band take the
                // exact route.
                bool undecided = covered;
                if (sizeof(T) == 4) {
                    const float s = (float)d0 * (float)d0 + (float)d1 * (float)d1 + (float)d2 * (float)d2;
                    hit = covered && s < P.rc2_lo && s > P.eps_hi;
                    undecided = covered && !hit && !(s > P.rc2_hi || s < P.eps_lo);
                }
                if (undecided) {
                    const double dd = add_rn(add_rn(mul_rn((double)d0, (double)d0), mul_rn((double)d1, (double)d1)),
                                             mul_rn((double)d2, (double)d2));
                    const double ddT = (double)(T)dd;
                    hit = (ddT < P.rc2) && (ddT > 1e-3);
                }
                if (hit) jidx = sinfo[aj].x;
                const unsigned bal = __ballot_sync(FULL_MASK, hit);
                if (hit) {
                    const int p = count + __popc(bal & lt_mask);
                    if (p < P.umax) {
                        frow[p] = jidx;
                        rrow[3 * p] = (TO)d0; rrow[3 * p + 1] = (TO)d1; rrow[3 * p + 2] = (TO)d2;
                    }
                }
                count += __popc(bal);
            }
            __syncwarp();
        }
        for (int k = count + lane; k < P.umax; k += 32) {
            frow[k] = -1;
            rrow[3 * k] = TO(0); rrow[3 * k + 1] = TO(0); rrow[3 * k + 2] = TO(0);
        }
        if (lane == 0) numneigh[i - P.cbegin] = min(count, P.umax);
        local_max = max(local_max, count);
    }
    if (lane == 0 && local_max > 0) {
        atomicMax(status, local_max);
        if (local_max > P.umax) status[1] = 1;
    }
}


// pass 3, lanes = centres: every lane owns one centre atom (32 consecutive atoms in bin order per warp) and walks
// through the columns of bins around it by itself, so a hit is appended to the lane's own row with a plain
// counter: no candidate table, no ballots, no compaction, and the single-precision pre-test is one load and a
// few operations per candidate. Neighbouring lanes are neighbouring atoms, so their candidates come from the same
// cache lines. Used for large systems when the bins of a column along the third axis form one range (zmerge); the
// predicate is the one of nb_build_kernel, line for line. Rows are padded by the whole warp afterwards, one row at a time, with
// stores that run along the row.
constexpr int NBL_WARPS = 4;
constexpr int NBL_MIN_ATOMS = 220000;     // systems from this size on take this kernel
template <typename T, typename TO>
__global__ void __launch_bounds__(NBL_WARPS * 32)
nb_build_lanes_kernel(NbParams<T> P, const NbGrid *__restrict__ gp, const int *__restrict__ bin_start,
                      const typename Vec4<T>::type *__restrict__ spos, const int4 *__restrict__ sinfo,
                      const float4 *__restrict__ sposw, const int4 *__restrict__ sbin, int *__restrict__ numneigh,
                      int *__restrict__ firstneigh, TO *__restrict__ rcs, int *__restrict__ status)
{
    chain_release();
    chain_wait();
    const NbGrid g = *gp;
    const bool packed = g.bigwrap == 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = gridDim.x * NBL_WARPS, gw = blockIdx.x * NBL_WARPS + warp;
    const int ny = 2 * g.R[1] + 1, ncol = (2 * g.R[0] + 1) * ny;
    const int R2 = g.R[2], nb2 = g.nb[2];
    const float c0x = (float)P.cell[0], c0y = (float)P.cell[1], c0z = (float)P.cell[2];
    const float c1x = (float)P.cell[3], c1y = (float)P.cell[4], c1z = (float)P.cell[5];
    const float c2x = (float)P.cell[6], c2y = (float)P.cell[7], c2z = (float)P.cell[8];
    int local_max = 0;

    for (int a0 = gw * 32; a0 < P.n; a0 += nwarps * 32) {
        const int a = a0 + lane;
        bool centre = a < P.n;
        typename Vec4<T>::type pi;
        pi.x = pi.y = pi.z = pi.w = T(0);
        float4 piw = make_float4(0.f, 0.f, 0.f, 0.f);
        int4 si = make_int4(0, 0, 0, 0), cb = make_int4(0, 0, 0, 0);
        if (centre) { pi = spos[a]; piw = sposw[a]; si = sinfo[a]; cb = sbin[a]; }
        const int i = si.x;
        centre = centre && i < P.ncentre && i >= P.cbegin;
        if (!__any_sync(FULL_MASK, centre)) continue;
        const int wi = nb_pack3(si.y, si.z, si.w);
        const int bx = cb.x, by = cb.y, bz = cb.z;
        const int rowi = centre ? i - P.cbegin : 0;
        int *frow = firstneigh + (size_t)rowi * P.umax;
        TO *rrow = rcs + (size_t)rowi * P.umax * 3;
        int count = 0;
        // a centre within R bins of a periodic face of the third axis has, per column, a second range across the face
        const bool zsplit = centre && P.per[2] && (bz - R2 < 0 || bz + R2 >= nb2);
        const int nparts = __any_sync(FULL_MASK, zsplit) ? 2 : 1;

        // one column of bins (or its part across a periodic face of the third axis): range of candidates in bin
        // order, image counts, single-precision image vector
        struct Range { int aj, end, m0, m1, m2; float svx, svy, svz; };
        auto range_of = [&](int c, int part) {
            Range r;
            r.aj = r.end = 0;
            const int d0 = c / ny - g.R[0], d1 = c % ny - g.R[1];
            int b[2] = {bx + d0, by + d1}, m[2] = {0, 0};
            bool ok = centre && c < ncol;
#pragma unroll
            for (int k = 0; k < 2; k++) {
                if (P.per[k]) {
                    int q;   // floor(b / nb); one period off at most unless the grid is tiny
                    if (b[k] >= 0 && b[k] < g.nb[k]) q = 0;
                    else if (b[k] < 0 && b[k] >= -g.nb[k]) q = -1;
                    else if (b[k] >= g.nb[k] && b[k] < 2 * g.nb[k]) q = 1;
                    else q = b[k] >= 0 ? b[k] / g.nb[k] : -((-b[k] + g.nb[k] - 1) / g.nb[k]);
                    m[k] = q; b[k] -= q * g.nb[k];
                } else {
                    ok = ok && b[k] >= 0 && b[k] < g.nb[k];
                }
            }
            int zlo = bz - R2, zhi = bz + R2, m2 = 0;
            if (part == 0) { zlo = max(zlo, 0); zhi = min(zhi, nb2 - 1); ok = ok && zlo <= zhi; }
            else if (!zsplit) ok = false;
            else if (zlo < 0) { zlo += nb2; zhi = nb2 - 1; m2 = -1; }      // bins of the image one period down
            else { zhi -= nb2; zlo = 0; m2 = 1; }                          // ... one period up
            if (ok) {
                const int col = (b[0] * g.nb[1] + b[1]) * nb2;
                r.aj = bin_start[col + zlo];
                r.end = bin_start[col + zhi + 1];
            }
            r.m0 = m[0]; r.m1 = m[1]; r.m2 = m2;
            const float f0 = (float)m[0], f1 = (float)m[1], f2 = (float)m2;
            r.svx = f0 * c0x + f1 * c1x + f2 * c2x; r.svy = f0 * c0y + f1 * c1y + f2 * c2y; r.svz = f0 * c0z + f1 * c1z + f2 * c2z;
            return r;
        };
        const int nsteps = ncol * nparts;
        Range nxt = range_of(0, 0);
        for (int step = 0; step < nsteps; step++) {
            const Range cur = nxt;
            {   // the next range's bin offsets are in flight while this range is worked on
                const int sn = step + 1;
                nxt = range_of(nparts == 2 ? sn >> 1 : sn, nparts == 2 ? sn & 1 : 0);
            }
            const int sh = (cur.m0 + 512) | ((cur.m1 + 512) << 10) | ((cur.m2 + 512) << 20);
            int aj = cur.aj;
            const int end = cur.end;
            while (__any_sync(FULL_MASK, aj < end)) {
                if (aj < end) {
                    // single-precision pre-test on the positions wrapped into the cell
                    const float4 pw = sposw[aj];
                    const float dx = (pw.x + cur.svx) - piw.x, dy = (pw.y + cur.svy) - piw.y, dz = (pw.z + cur.svz) - piw.z;
                    const float sq = dx * dx + dy * dy + dz * dz;
                    if (sq < g.pre_hi && sq > g.pre_lo) {
                        const typename Vec4<T>::type pj = spos[aj];
                        const int4 sj = sinfo[aj];
                        // periods between the candidate's stored position and the image this range means
                        int n0, n1, n2;
                        bool away;
                        if (packed) {
                            const int nw = sh - nb_bits_of(pj.w) + wi;
                            away = nw != NB_PACK_ZERO;
                            n0 = (nw & 1023) - 512; n1 = ((nw >> 10) & 1023) - 512; n2 = ((nw >> 20) & 1023) - 512;
                        } else {
                            n0 = cur.m0 - sj.y + si.y; n1 = cur.m1 - sj.z + si.z; n2 = cur.m2 - sj.w + si.w;
                            away = (n0 | n1 | n2) != 0;
                        }
                        const bool covered = !away || (abs(n0) <= P.e[0] && abs(n1) <= P.e[1] && abs(n2) <= P.e[2]);
                        T ix = pj.x, iy = pj.y, iz = pj.z;
                        // the home image needs no arithmetic, except for exact zeros (-0.0 + 0 is +0)
                        if (covered && (away || ix == T(0) || iy == T(0) || iz == T(0))) {
                            const T g0 = T(n0), g1 = T(n1), g2 = T(n2);
                            ix = add_rn(add_rn(add_rn(pj.x, mul_rn(P.cell[0], g0)), mul_rn(P.cell[3], g1)), mul_rn(P.cell[6], g2));
                            iy = add_rn(add_rn(add_rn(pj.y, mul_rn(P.cell[1], g0)), mul_rn(P.cell[4], g1)), mul_rn(P.cell[7], g2));
                            iz = add_rn(add_rn(add_rn(pj.z, mul_rn(P.cell[2], g0)), mul_rn(P.cell[5], g1)), mul_rn(P.cell[8], g2));
                        }
                        const T e0 = sub_rn(ix, pi.x), e1 = sub_rn(iy, pi.y), e2 = sub_rn(iz, pi.z);
                        bool hit = false, undecided = covered;
                        if (sizeof(T) == 4) {
                            const float sf = (float)e0 * (float)e0 + (float)e1 * (float)e1 + (float)e2 * (float)e2;
                            hit = covered && sf < P.rc2_lo && sf > P.eps_hi;
                            undecided = covered && !hit && !(sf > P.rc2_hi || sf < P.eps_lo);
                        }
                        if (undecided) {
                            const double dd = add_rn(add_rn(mul_rn((double)e0, (double)e0), mul_rn((double)e1, (double)e1)),
                                                     mul_rn((double)e2, (double)e2));
                            const double ddT = (double)(T)dd;
                            hit = (ddT < P.rc2) && (ddT > 1e-3);
                        }
                        if (hit) {
                            if (count < P.umax) {
                                frow[count] = sj.x;
                                rrow[3 * count] = (TO)e0; rrow[3 * count + 1] = (TO)e1; rrow[3 * count + 2] = (TO)e2;
                            }
                            count++;
                        }
                    }
                }
                aj++;
            }
        }
        if (centre) numneigh[rowi] = min(count, P.umax);
        local_max = max(local_max, centre ? count : 0);
        // padding of the 32 rows, by the whole warp
        for (int l = 0; l < 32; l++) {
            const int cl = __shfl_sync(FULL_MASK, centre ? min(count, P.umax) : P.umax, l);
            const int rl = __shfl_sync(FULL_MASK, rowi, l);
            if (cl >= P.umax) continue;
            int *fr = firstneigh + (size_t)rl * P.umax;
            TO *rr = rcs + (size_t)rl * P.umax * 3;
            for (int k = cl + lane; k < P.umax; k += 32) {
                fr[k] = -1;
                rr[3 * k] = TO(0); rr[3 * k + 1] = TO(0); rr[3 * k + 2] = TO(0);
            }
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) local_max = max(local_max, __shfl_xor_sync(FULL_MASK, local_max, o));
    if (lane == 0 && local_max > 0) {
        atomicMax(status, local_max);
        if (local_max > P.umax) status[1] = 1;
    }
}

// optional pass 4: order each row by distance (the reference's sort=true, neighborList.h:290-335:
// std::sort on sqrt(dx^2+dy^2+dz^2)). Stable rank sort, one warp per row; ties keep build order.
template <typename T>
__global__ void nb_sort_rows_kernel(int n, int umax, const int *__restrict__ numneigh, int *__restrict__ firstneigh, T *__restrict__ rcs)
{
    extern __shared__ __align__(16) unsigned char sort_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    T *key = reinterpret_cast<T *>(sort_smem) + (size_t)warp * umax * 4;
    T *val = key + umax;                                   // 3 * umax
    int *idx = reinterpret_cast<int *>(reinterpret_cast<T *>(sort_smem) + (size_t)wpb * umax * 4) + (size_t)warp * umax;
    for (int i = blockIdx.x * wpb + warp; i < n; i += gridDim.x * wpb) {
        const int nn = min(numneigh[i], umax);
        int *frow = firstneigh + (size_t)i * umax;
        T *rrow = rcs + (size_t)i * umax * 3;
        for (int k = lane; k < nn; k += 32) {
            T a = rrow[3 * k], b = rrow[3 * k + 1], c = rrow[3 * k + 2];
            val[3 * k] = a; val[3 * k + 1] = b; val[3 * k + 2] = c;
            idx[k] = frow[k];
            key[k] = (T)sqrt((double)a * (double)a + (double)b * (double)b + (double)c * (double)c);
        }
        __syncwarp();
        for (int k = lane; k < nn; k += 32) {
            const T kk = key[k];
            int rank = 0;
            for (int m = 0; m < nn; m++) rank += (key[m] < kk || (key[m] == kk && m < k)) ? 1 : 0;
            frow[rank] = idx[k];
            rrow[3 * rank] = val[3 * k]; rrow[3 * rank + 1] = val[3 * k + 1]; rrow[3 * rank + 2] = val[3 * k + 2];
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
struct NbLayout {
    size_t grid, ext, status_unused, cart, ainfo, count, start, cursor, bsum, spos, sinfo, sposw, sbin, total;
};
template <typename T>
static NbLayout nb_layout(int n, int maxbins)
{
    NbLayout L;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t r = o; o += (bytes + 255) & ~size_t(255); return r; };
    L.grid = take(sizeof(NbGrid));
    L.ext = take(6 * sizeof(unsigned long long));
    L.status_unused = take(16);
    L.cart = take(sizeof(T) * 3 * (size_t)n);
    L.ainfo = take(sizeof(int4) * (size_t)n);
    L.count = take(sizeof(int) * ((size_t)maxbins + 1));
    L.start = take(sizeof(int) * ((size_t)maxbins + 2));
    L.cursor = take(sizeof(int) * ((size_t)maxbins + 1));
    L.bsum = take(sizeof(int) * ((size_t)maxbins / SCAN_BLOCK + 2));
    L.spos = take(sizeof(typename Vec4<T>::type) * (size_t)n);
    L.sinfo = take(sizeof(int4) * (size_t)n);
    L.sposw = take(sizeof(float4) * (size_t)n);
    L.sbin = take(sizeof(int4) * (size_t)n);
    L.total = o;
    return L;
}
static int nb_maxbins(int n) { return 2 * (n > 0 ? n : 0) + 4096; }

template <typename T>
static void plane_distances(const T *cell, T *d)
{
    // interplanar distances in type T, same operations as structure.h:818-843
    for (int k = 0; k < 3; k++) {
        const T *a = cell + 3 * ((k == 0) ? 1 : 0), *b = cell + 3 * ((k == 2) ? 1 : 2);
        T n[3] = {a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]};
        T len = (T)std::sqrt((double)(n[0] * n[0] + n[1] * n[1] + n[2] * n[2]));
        T u[3] = {n[0] / len, n[1] / len, n[2] / len};
        const T *c = cell + 3 * k;
        d[k] = (T)std::fabs((double)(c[0] * u[0] + c[1] * u[1] + c[2] * u[2]));
    }
}

// Rows for the centres [cbegin, ncentre) of the n atoms. reuse_bins: the workspace still holds the bins of an
// earlier call with the same atoms, cell, cutoff and flags, so only the row pass runs (d_status is then
// accumulated into, not reset).
template <typename T, typename TO = T>
static int nblist_build(int n, int ncentre, const T *h_cell, const T *d_coords, int is_cart, double rcut_in, const int *pbc, int umax,
                        int *d_numneigh, int *d_firstneigh, TO *d_rcs, int *d_status, void *ws, size_t ws_bytes, cudaStream_t st,
                        int cbegin = 0, bool reuse_bins = false, const double *open_ext = nullptr)
{
    AI2B_REQUIRE(h_cell && pbc && d_status, AI2B_ERR_INVALID, "ai2b_nblist_build: NULL argument");
    AI2B_REQUIRE(n >= 0 && umax >= 0 && rcut_in > 0 && ncentre >= 0 && ncentre <= n && cbegin >= 0 && cbegin <= ncentre,
                 AI2B_ERR_INVALID, "ai2b_nblist_build: bad size, centre range or cutoff");
    if (n == 0 || ncentre == cbegin) return AI2B_OK;
    AI2B_REQUIRE(d_coords && d_numneigh && d_firstneigh && d_rcs, AI2B_ERR_INVALID, "ai2b_nblist_build: NULL argument");
    const int maxbins = nb_maxbins(n);
    const NbLayout L = nb_layout<T>(n, maxbins);
    AI2B_REQUIRE(ws && ws_bytes >= L.total, AI2B_ERR_WORKSPACE, "nblist workspace too small: %zu < %zu bytes", ws_bytes, L.total);

    NbParams<T> P;
    memset(&P, 0, sizeof(P));
    const T rcut = (T)rcut_in;                 // the float build casts rcut first (nblist_bind.cc:133)
    for (int k = 0; k < 9; k++) P.cell[k] = h_cell[k];
    // inverse cell in double
    double a[9];
    for (int k = 0; k < 9; k++) a[k] = (double)h_cell[k];
    double det = a[0] * (a[4] * a[8] - a[5] * a[7]) - a[1] * (a[3] * a[8] - a[5] * a[6]) + a[2] * (a[3] * a[7] - a[4] * a[6]);
    AI2B_REQUIRE(std::fabs(det) > 1e-300, AI2B_ERR_INVALID, "ai2b_nblist_build: singular cell");
    // inv = A^{-1}, with r = f A  =>  f = r A^{-1}
    double c[9] = {a[4] * a[8] - a[5] * a[7], a[2] * a[7] - a[1] * a[8], a[1] * a[5] - a[2] * a[4],
                   a[5] * a[6] - a[3] * a[8], a[0] * a[8] - a[2] * a[6], a[2] * a[3] - a[0] * a[5],
                   a[3] * a[7] - a[4] * a[6], a[1] * a[6] - a[0] * a[7], a[0] * a[4] - a[1] * a[3]};
    for (int k = 0; k < 9; k++) P.inv[k] = c[k] / det;
    T dT[3];
    plane_distances<T>(h_cell, dT);
    P.rcut_m = (double)rcut * 1.0001 + 1e-6;
    P.rc2 = (double)rcut * (double)rcut;
    if (sizeof(T) == 8) { volatile double r2 = (double)rcut * (double)rcut; P.rc2 = r2; }
    P.rc2_lo = (float)(P.rc2 * (1.0 - 2e-6)); P.rc2_hi = (float)(P.rc2 * (1.0 + 2e-6));
    P.eps_lo = (float)(1e-3 * (1.0 - 2e-6)); P.eps_hi = (float)(1e-3 * (1.0 + 2e-6));
    P.n = n; P.umax = umax; P.maxbins = maxbins; P.ncentre = ncentre; P.cbegin = cbegin;
    bool any_open = false;
    long prod = 1;
    for (int k = 0; k < 3; k++) {
        P.per[k] = pbc[k] ? 1 : 0;
        P.dplane[k] = (double)dT[k];
        P.e[k] = pbc[k] ? (int)std::ceil((double)(rcut / dT[k])) : 0;
        AI2B_REQUIRE(P.e[k] < 500, AI2B_ERR_UNSUPPORTED, "cell far smaller than the cutoff (%d images on axis %d)", P.e[k], k);
        if (pbc[k]) {
            int nb = (int)std::floor(P.dplane[k] * NB_SUB / P.rcut_m);
            P.nbh[k] = nb < 1 ? 1 : nb;
        } else {
            any_open = true;
            P.nbh[k] = 1;
        }
        prod *= P.nbh[k];
    }
    // shrink periodic bin counts if the grid would not fit, then hand the rest to the open axes
    while (prod > maxbins) {
        int big = 0;
        for (int k = 1; k < 3; k++) if (P.nbh[k] > P.nbh[big]) big = k;
        prod /= P.nbh[big];
        P.nbh[big] = (P.nbh[big] + 1) / 2;
        prod *= P.nbh[big];
    }
    if (any_open) {
        int nopen = 0;
        for (int k = 0; k < 3; k++) nopen += pbc[k] ? 0 : 1;
        int cap = (int)std::floor(std::pow((double)maxbins / (double)prod, 1.0 / nopen));
        for (int k = 0; k < 3; k++) if (!pbc[k]) P.nbh[k] = cap < 1 ? 1 : cap;
    }
    // The grid is known on the host when every axis is periodic, or when the caller gives the fractional extent
    // of the atoms along the open axes (atoms outside it are clamped into the edge bins, which keeps every
    // pair within reach of the bin search: an extent that is a little off costs time, not pairs).
    NbGrid hg;
    memset(&hg, 0, sizeof(hg));
    const bool host_grid = !any_open || open_ext != nullptr;
    if (host_grid) {
        long total = 1;
        for (int k = 0; k < 3; k++) {
            if (P.per[k]) {
                hg.nb[k] = P.nbh[k];
                hg.R[k] = (int)std::ceil(P.rcut_m / (P.dplane[k] / P.nbh[k]));
                hg.lo[k] = 0.0;
                hg.scale[k] = (double)P.nbh[k];
            } else {
                const double lo = open_ext[k], hi = open_ext[3 + k];
                const double span = std::fmax(hi - lo, 1e-12);
                int nb = (int)std::floor(span * P.dplane[k] * NB_SUB / P.rcut_m);
                nb = nb < 1 ? 1 : (nb > P.nbh[k] ? P.nbh[k] : nb);
                hg.nb[k] = nb;
                hg.R[k] = NB_SUB;
                hg.lo[k] = lo;
                hg.scale[k] = nb / span;
            }
            total *= hg.nb[k];
        }
        hg.total = (int)total;
        hg.zmerge = (!P.per[2] || hg.nb[2] >= 2 * hg.R[2] + 1) ? 1 : 0;
        nb_pretest_bounds(P, hg.lo, nullptr, false, &hg);
        prod = total;
    }

    unsigned char *w = (unsigned char *)ws;
    NbGrid *grid = (NbGrid *)(w + L.grid);
    unsigned long long *ext = (unsigned long long *)(w + L.ext);
    T *cart = (T *)(w + L.cart);
    int4 *ainfo = (int4 *)(w + L.ainfo);
    int *count = (int *)(w + L.count), *start = (int *)(w + L.start), *cursor = (int *)(w + L.cursor), *bsum = (int *)(w + L.bsum);
    auto *spos = (typename Vec4<T>::type *)(w + L.spos);
    int4 *sinfo = (int4 *)(w + L.sinfo);
    float4 *sposw = (float4 *)(w + L.sposw);
    int4 *sbin = (int4 *)(w + L.sbin);

    const int tb = 256, nblk = (n + tb - 1) / tb;
    const T *pos = d_coords;
    if (!is_cart) {
        if (!reuse_bins) nb_frac2cart_kernel<T><<<nblk, tb, 0, st>>>(P, d_coords, cart);
        pos = cart;
    }
    const bool small_grid = host_grid;
    if (reuse_bins) {
        // bins, bin-ordered positions and (for fractional input) Cartesian positions are in the workspace already
    } else if (small_grid) {
        const int ncount = (int)prod + 1;
        AI2B_CUDA(launch_chained(nb_setup_periodic_kernel, (ncount + 255) / 256, 256, 0, st, hg, grid, count, ncount, d_status));
        AI2B_CUDA(launch_chained(nb_count_kernel<T>, nblk, tb, 0, st, P, grid, pos, ainfo, count));
        if (ncount <= SCAN_CLUSTER * SCAN_BLOCK * SCAN_ITEMS) {
            AI2B_CUDA(launch_chained(nb_scan_cluster_kernel, SCAN_CLUSTER, SCAN_BLOCK, 0, st, grid, count, start, cursor));
        } else if (ncount <= 64 * SCAN_BLOCK) {
            AI2B_CUDA(launch_chained(nb_scan_small_kernel, 1, SCAN_BLOCK, 0, st, grid, count, start, cursor));
        } else {   // large grids: block-parallel scan
            const int sblk = (ncount + SCAN_BLOCK - 1) / SCAN_BLOCK;
            nb_scan1_kernel<<<sblk, SCAN_BLOCK, 0, st>>>(grid, count, start, bsum);
            nb_scan2_kernel<<<1, SCAN_BLOCK, 0, st>>>(grid, bsum);
            nb_scan3_kernel<<<sblk, SCAN_BLOCK, 0, st>>>(grid, start, bsum, cursor);
        }
    } else {
        nb_init_kernel<<<1, 32, 0, st>>>(ext, d_status);
        if (any_open) nb_extent_kernel<T><<<(nblk < 1024 ? nblk : 1024), tb, 0, st>>>(P, pos, ext);
        nb_grid_kernel<T><<<1, 32, 0, st>>>(P, ext, grid);
        AI2B_CUDA(cudaMemsetAsync(count, 0, sizeof(int) * ((size_t)maxbins + 1), st));
        nb_count_kernel<T><<<nblk, tb, 0, st>>>(P, grid, pos, ainfo, count);
        const int sblk = (maxbins + 1 + SCAN_BLOCK - 1) / SCAN_BLOCK;
        nb_scan1_kernel<<<sblk, SCAN_BLOCK, 0, st>>>(grid, count, start, bsum);
        nb_scan2_kernel<<<1, SCAN_BLOCK, 0, st>>>(grid, bsum);
        nb_scan3_kernel<<<sblk, SCAN_BLOCK, 0, st>>>(grid, start, bsum, cursor);
    }
    if (!reuse_bins) AI2B_CUDA(launch_chained(nb_fill_kernel<T>, nblk, tb, 0, st, P, pos, ainfo, cursor, spos, sinfo, sposw, sbin, grid));
    const int sms = sm_count();
    // the bins of a column along the third axis form one range unless that axis is periodic and shorter than the
    // search window (known on the host: open axes always search NB_SUB bins)
    const int R2 = P.per[2] ? (int)std::ceil(P.rcut_m / (P.dplane[2] / P.nbh[2])) : NB_SUB;
    const bool zmerge = !P.per[2] || P.nbh[2] >= 2 * R2 + 1;
    // Lanes = centres for large systems: far fewer instructions per atom, but every lane walks through memory on
    // its own, which only pays once there are enough warps per SM to hide that latency. Measured time of the whole
    // build, warp per centre / lane per centre (fp32, rcut 6, 29 neighbours): 55,296 atoms 0.087 / 0.126 ms,
    // 186,624 atoms 0.234 / 0.236 ms, 256,000 atoms 0.280 / 0.265 ms, 780,448 atoms 0.769 / 0.618 ms.
    int min_atoms = NBL_MIN_ATOMS;
    if (const char *env = std::getenv("AI2B_NBL_MIN_ATOMS")) min_atoms = std::atoi(env);   // tuning knob, read per call
    if (zmerge && n >= min_atoms) {
        long blocks = ((long)n + 32 * NBL_WARPS - 1) / (32 * NBL_WARPS);
        if (blocks > (long)sms * 16) blocks = (long)sms * 16;
        AI2B_CUDA(launch_chained(nb_build_lanes_kernel<T, TO>, (unsigned)blocks, NBL_WARPS * 32, 0, st, P, grid, start, spos, sinfo, sposw, sbin,
                                 d_numneigh, d_firstneigh, d_rcs, d_status));
        return AI2B_OK;
    }
    long blocks = ((long)n + NB_WARPS - 1) / NB_WARPS;
    if (blocks > (long)sms * 8) blocks = (long)sms * 8;
    AI2B_CUDA(launch_chained(nb_build_kernel<T, TO>, (unsigned)blocks, NB_WARPS * 32, 0, st, P, grid, start, ainfo, spos, sinfo, sposw, sbin, d_numneigh,
                             d_firstneigh, d_rcs, d_status));
    return AI2B_OK;
}


// ---- padded batch of small cells: one launch --------------------------------------------------------
// A training set holds many small periodic structures (tens to hundreds of atoms); the reference's
// dataset builds one list per frame and pads every array to the largest structure
// (ai2pot/data/mlffdataset.py:61-90). For such cells a cell list brings nothing (1-3 bins per axis):
// every (centre, atom, image) triple of the reference's supercell is tested instead, which is the
// reference's membership rule by construction. One block per (structure, chunk of centres); the
// structure's positions are staged through shared memory in tiles; one warp per centre, lanes over
// the atoms of a tile, the image loops are uniform across the warp.
constexpr int NBB_WARPS = 8;
constexpr int NBB_TILE = 1024;      // atoms staged per tile
constexpr int NBB_CPB = 32;         // centres per block

template <typename T>
struct NbBatchParams {
    int B, npad, umax, is_cart, per[3];
    T rcut;
    double rc2;
    float rc2_lo, rc2_hi, eps_lo, eps_hi;
};

template <typename T>
__global__ void __launch_bounds__(NBB_WARPS * 32)
nb_batch_kernel(NbBatchParams<T> P, const int *__restrict__ binum, const T *__restrict__ cells, const T *__restrict__ coords,
                int *__restrict__ bilist, int *__restrict__ bnumneigh, int *__restrict__ bfirstneigh, T *__restrict__ brcs,
                int *__restrict__ status)
{
    __shared__ T s_pos[NBB_TILE * 3];
    __shared__ T s_cell[9];
    __shared__ int s_e[3];
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = min(max(binum[b], 0), P.npad);
    const int c_begin = blockIdx.x * NBB_CPB;
    if (c_begin >= P.npad) return;
    if (threadIdx.x == 0) {
        // image range per periodic axis: ceil(rcut / interplanar distance), in type T with the operations of
        // source/nblist/include/structure.h:818-843 (no contraction)
        T c[9];
        for (int k = 0; k < 9; k++) c[k] = s_cell[k] = cells[(size_t)b * 9 + k];
        for (int k = 0; k < 3; k++) {
            const T *a = c + 3 * ((k == 0) ? 1 : 0), *bb = c + 3 * ((k == 2) ? 1 : 2);
            const T nx = sub_rn(mul_rn(a[1], bb[2]), mul_rn(a[2], bb[1])), ny = sub_rn(mul_rn(a[2], bb[0]), mul_rn(a[0], bb[2])),
                    nz = sub_rn(mul_rn(a[0], bb[1]), mul_rn(a[1], bb[0]));
            const T len = (T)sqrt((double)add_rn(add_rn(mul_rn(nx, nx), mul_rn(ny, ny)), mul_rn(nz, nz)));
            const T ux = nx / len, uy = ny / len, uz = nz / len;
            const T d = (T)fabs((double)add_rn(add_rn(mul_rn(c[3 * k], ux), mul_rn(c[3 * k + 1], uy)), mul_rn(c[3 * k + 2], uz)));
            int e = 0;
            if (P.per[k]) {
                const double q = ceil((double)(P.rcut / d));
                if (!(q < 500.0)) { e = 0; atomicOr(status + 1, 2); }   // degenerate cell: flagged, no images
                else e = (int)q;
            }
            s_e[k] = e;
        }
    }
    __syncthreads();
    const int e0 = s_e[0], e1 = s_e[1], e2 = s_e[2];
    const T *cpos = coords + (size_t)b * P.npad * 3;
    auto cart = [&](int j, T &x, T &y, T &z) {
        const T f0 = cpos[3 * j], f1 = cpos[3 * j + 1], f2 = cpos[3 * j + 2];
        if (P.is_cart) { x = f0; y = f1; z = f2; return; }
        x = add_rn(add_rn(mul_rn(f0, s_cell[0]), mul_rn(f1, s_cell[3])), mul_rn(f2, s_cell[6]));
        y = add_rn(add_rn(mul_rn(f0, s_cell[1]), mul_rn(f1, s_cell[4])), mul_rn(f2, s_cell[7]));
        z = add_rn(add_rn(mul_rn(f0, s_cell[2]), mul_rn(f1, s_cell[5])), mul_rn(f2, s_cell[8]));
    };
    const unsigned lt_mask = (1u << lane) - 1u;
    // each warp owns NBB_CPB / NBB_WARPS centres; all warps walk the tiles together (block-wide staging)
    constexpr int CPW = NBB_CPB / NBB_WARPS;
    int cnt[CPW];
    T cx[CPW], cy[CPW], cz[CPW];
#pragma unroll
    for (int q = 0; q < CPW; q++) {
        cnt[q] = 0;
        const int i = c_begin + warp * CPW + q;
        cx[q] = cy[q] = cz[q] = T(0);
        if (i < n) cart(i, cx[q], cy[q], cz[q]);
    }
    for (int t0 = 0; t0 < n; t0 += NBB_TILE) {
        const int tn = min(NBB_TILE, n - t0);
        __syncthreads();
        for (int j = threadIdx.x; j < tn; j += blockDim.x) {
            T x, y, z;
            cart(t0 + j, x, y, z);
            s_pos[3 * j] = x; s_pos[3 * j + 1] = y; s_pos[3 * j + 2] = z;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < CPW; q++) {
            const int i = c_begin + warp * CPW + q;
            if (i >= n) continue;
            int *frow = bfirstneigh + ((size_t)b * P.npad + i) * P.umax;
            T *rrow = brcs + ((size_t)b * P.npad + i) * P.umax * 3;
            int count = cnt[q];
            for (int n0 = -e0; n0 <= e0; n0++)
            for (int n1 = -e1; n1 <= e1; n1++)
            for (int n2 = -e2; n2 <= e2; n2++) {
                const T f0 = T(n0), f1 = T(n1), f2 = T(n2);
                // shift of this image, applied in the reference's order ((r + a0 n0) + a1 n1) + a2 n2
                const T s0x = mul_rn(s_cell[0], f0), s0y = mul_rn(s_cell[1], f0), s0z = mul_rn(s_cell[2], f0);
                const T s1x = mul_rn(s_cell[3], f1), s1y = mul_rn(s_cell[4], f1), s1z = mul_rn(s_cell[5], f1);
                const T s2x = mul_rn(s_cell[6], f2), s2y = mul_rn(s_cell[7], f2), s2z = mul_rn(s_cell[8], f2);
                for (int j0 = 0; j0 < tn; j0 += 32) {
                    const int j = j0 + lane;
                    bool hit = false;
                    T d0 = 0, d1 = 0, d2 = 0;
                    if (j < tn) {
                        const T ix = add_rn(add_rn(add_rn(s_pos[3 * j], s0x), s1x), s2x);
                        const T iy = add_rn(add_rn(add_rn(s_pos[3 * j + 1], s0y), s1y), s2y);
                        const T iz = add_rn(add_rn(add_rn(s_pos[3 * j + 2], s0z), s1z), s2z);
                        d0 = sub_rn(ix, cx[q]); d1 = sub_rn(iy, cy[q]); d2 = sub_rn(iz, cz[q]);
                        bool undecided = true;
                        if (sizeof(T) == 4) {
                            const float sq = (float)d0 * (float)d0 + (float)d1 * (float)d1 + (float)d2 * (float)d2;
                            hit = sq < P.rc2_lo && sq > P.eps_hi;
                            undecided = !hit && !(sq > P.rc2_hi || sq < P.eps_lo);
                        }
                        if (undecided) {
                            const double dd = add_rn(add_rn(mul_rn((double)d0, (double)d0), mul_rn((double)d1, (double)d1)),
                                                     mul_rn((double)d2, (double)d2));
                            const double ddT = (double)(T)dd;
                            hit = (ddT < P.rc2) && (ddT > 1e-3);
                        }
                    }
                    const unsigned bal = __ballot_sync(FULL_MASK, hit);
                    if (hit) {
                        const int p = count + __popc(bal & lt_mask);
                        if (p < P.umax) {
                            frow[p] = t0 + j;
                            rrow[3 * p] = d0; rrow[3 * p + 1] = d1; rrow[3 * p + 2] = d2;
                        }
                    }
                    count += __popc(bal);
                }
            }
            cnt[q] = count;
        }
    }
    // padding, counts, centre list; rows of padded atom slots (i >= n) are all padding
    int local_max = 0;
#pragma unroll
    for (int q = 0; q < CPW; q++) {
        const int i = c_begin + warp * CPW + q;
        if (i >= P.npad) continue;
        const int count = i < n ? cnt[q] : 0;
        int *frow = bfirstneigh + ((size_t)b * P.npad + i) * P.umax;
        T *rrow = brcs + ((size_t)b * P.npad + i) * P.umax * 3;
        for (int k = min(count, P.umax) + lane; k < P.umax; k += 32) {
            frow[k] = -1;
            rrow[3 * k] = T(0); rrow[3 * k + 1] = T(0); rrow[3 * k + 2] = T(0);
        }
        if (lane == 0) {
            bnumneigh[(size_t)b * P.npad + i] = min(count, P.umax);
            bilist[(size_t)b * P.npad + i] = i < n ? i : 0;
        }
        local_max = max(local_max, count);
    }
    if (lane == 0 && local_max > 0) {
        atomicMax(status, local_max);
        if (local_max > P.umax) atomicOr(status + 1, 1);
    }
}

template <typename T>
static int nblist_build_batch(int B, int npad, const int *d_binum, const T *d_cells, const T *d_coords, int is_cart, double rcut_in,
                              const int *pbc, int umax, int *d_bilist, int *d_bnumneigh, int *d_bfirstneigh, T *d_brcs, int *d_status,
                              cudaStream_t st)
{
    AI2B_REQUIRE(B >= 0 && npad >= 0 && umax >= 0 && rcut_in > 0, AI2B_ERR_INVALID, "ai2b_nblist_build_batch: bad size or cutoff");
    AI2B_REQUIRE(pbc && d_status, AI2B_ERR_INVALID, "ai2b_nblist_build_batch: NULL argument");
    AI2B_CUDA(cudaMemsetAsync(d_status, 0, 2 * sizeof(int), st));
    if (B == 0 || npad == 0) return AI2B_OK;
    AI2B_REQUIRE(d_binum && d_cells && d_coords && d_bilist && d_bnumneigh && d_bfirstneigh && d_brcs, AI2B_ERR_INVALID,
                 "ai2b_nblist_build_batch: NULL argument");
    AI2B_REQUIRE(B <= 65535, AI2B_ERR_UNSUPPORTED, "ai2b_nblist_build_batch: more than 65535 structures in one call");
    NbBatchParams<T> P;
    memset(&P, 0, sizeof(P));
    P.B = B; P.npad = npad; P.umax = umax; P.is_cart = is_cart ? 1 : 0;
    for (int k = 0; k < 3; k++) P.per[k] = pbc[k] ? 1 : 0;
    const T rcut = (T)rcut_in;                 // the float build casts rcut first (nblist_bind.cc:133)
    P.rcut = rcut;
    P.rc2 = (double)rcut * (double)rcut;
    if (sizeof(T) == 8) { volatile double r2 = (double)rcut * (double)rcut; P.rc2 = r2; }
    P.rc2_lo = (float)(P.rc2 * (1.0 - 2e-6)); P.rc2_hi = (float)(P.rc2 * (1.0 + 2e-6));
    P.eps_lo = (float)(1e-3 * (1.0 - 2e-6)); P.eps_hi = (float)(1e-3 * (1.0 + 2e-6));
    dim3 grid((unsigned)((npad + NBB_CPB - 1) / NBB_CPB), (unsigned)B);
    nb_batch_kernel<T><<<grid, NBB_WARPS * 32, 0, st>>>(P, d_binum, d_cells, d_coords, d_bilist, d_bnumneigh, d_bfirstneigh, d_brcs,
                                                        d_status);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" int ai2b_nblist_build_batch_f64(int batch_size, int natoms_pad, const int *d_binum, const double *d_cells,
                                           const double *d_coords, int is_cart, double rcut, const int *h_pbc, int umax,
                                           int *d_bilist, int *d_bnumneigh, int *d_bfirstneigh, double *d_brcs, int *d_status,
                                           void *stream)
{
    return nblist_build_batch<double>(batch_size, natoms_pad, d_binum, d_cells, d_coords, is_cart, rcut, h_pbc, umax, d_bilist,
                                      d_bnumneigh, d_bfirstneigh, d_brcs, d_status, (cudaStream_t)stream);
}
extern "C" int ai2b_nblist_build_batch_f32(int batch_size, int natoms_pad, const int *d_binum, const float *d_cells,
                                           const float *d_coords, int is_cart, double rcut, const int *h_pbc, int umax,
                                           int *d_bilist, int *d_bnumneigh, int *d_bfirstneigh, float *d_brcs, int *d_status,
                                           void *stream)
{
    return nblist_build_batch<float>(batch_size, natoms_pad, d_binum, d_cells, d_coords, is_cart, rcut, h_pbc, umax, d_bilist,
                                     d_bnumneigh, d_bfirstneigh, d_brcs, d_status, (cudaStream_t)stream);
}

extern "C" size_t ai2b_nblist_workspace_bytes(int natoms, int is_f64)
{
    return is_f64 ? nb_layout<double>(natoms, nb_maxbins(natoms)).total : nb_layout<float>(natoms, nb_maxbins(natoms)).total;
}

extern "C" int ai2b_nblist_build_f64(int natoms, const double *h_cell, const double *d_coords, int is_cart, double rcut,
                                     const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh, double *d_rcs,
                                     int *d_status, void *d_workspace, size_t workspace_bytes, void *stream)
{
    return nblist_build<double>(natoms, natoms, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                                d_status, d_workspace, workspace_bytes, (cudaStream_t)stream);
}
extern "C" int ai2b_nblist_build_f32(int natoms, const float *h_cell, const float *d_coords, int is_cart, double rcut,
                                     const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh, float *d_rcs,
                                     int *d_status, void *d_workspace, size_t workspace_bytes, void *stream)
{
    return nblist_build<float>(natoms, natoms, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                               d_status, d_workspace, workspace_bytes, (cudaStream_t)stream);
}

template <typename T>
static int nblist_sort(int n, int umax, const int *numneigh, int *firstneigh, T *rcs, cudaStream_t st)
{
    AI2B_REQUIRE(n >= 0 && umax >= 0, AI2B_ERR_INVALID, "ai2b_nblist_sort_rows: negative size");
    if (n == 0 || umax == 0) return AI2B_OK;
    AI2B_REQUIRE(numneigh && firstneigh && rcs, AI2B_ERR_INVALID, "ai2b_nblist_sort_rows: NULL argument");
    const int wpb = 4;
    const size_t smem = (size_t)wpb * umax * (4 * sizeof(T) + sizeof(int));
    AI2B_REQUIRE(smem <= 200 * 1024, AI2B_ERR_UNSUPPORTED, "umax %d too large to sort rows in shared memory", umax);
    auto kern = nb_sort_rows_kernel<T>;
    if (smem > 48 * 1024) AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    long blocks = ((long)n + wpb - 1) / wpb;
    if (blocks > 148 * 8) blocks = 148 * 8;
    kern<<<(unsigned)blocks, wpb * 32, smem, st>>>(n, umax, numneigh, firstneigh, rcs);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}
extern "C" int ai2b_nblist_sort_rows_f64(int natoms, int umax, const int *d_numneigh, int *d_firstneigh, double *d_rcs, void *stream)
{
    return nblist_sort<double>(natoms, umax, d_numneigh, d_firstneigh, d_rcs, (cudaStream_t)stream);
}
extern "C" int ai2b_nblist_sort_rows_f32(int natoms, int umax, const int *d_numneigh, int *d_firstneigh, float *d_rcs, void *stream)
{
    return nblist_sort<float>(natoms, umax, d_numneigh, d_firstneigh, d_rcs, (cudaStream_t)stream);
}

// Same build for a local domain with ghost atoms: rows are produced for the first `ncentres`
// atoms only, all `natoms` atoms (centres + ghosts) are candidates. Indices in d_firstneigh are
// positions in d_coords, so ghosts appear as indices >= ncentres (the LAMMPS convention the
// evaluation ops expect with nghost = natoms - ncentres).
extern "C" int ai2b_nblist_build_ghost_f64(int natoms, int ncentres, const double *h_cell, const double *d_coords, int is_cart,
                                           double rcut, const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh,
                                           double *d_rcs, int *d_status, void *d_workspace, size_t workspace_bytes, void *stream)
{
    return nblist_build<double>(natoms, ncentres, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                                d_status, d_workspace, workspace_bytes, (cudaStream_t)stream);
}
extern "C" int ai2b_nblist_build_ghost_f32(int natoms, int ncentres, const float *h_cell, const float *d_coords, int is_cart,
                                           double rcut, const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh,
                                           float *d_rcs, int *d_status, void *d_workspace, size_t workspace_bytes, void *stream)
{
    return nblist_build<float>(natoms, ncentres, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                               d_status, d_workspace, workspace_bytes, (cudaStream_t)stream);
}
// Rows for the centre range [centre_begin, centre_end) only (row 0 of the outputs = centre_begin), all natoms
// atoms as candidates; with reuse_bins != 0 the binning left in the workspace by an earlier call on the same
// atoms is used again (a domain evaluated in several passes bins once per set of candidates).
extern "C" int ai2b_nblist_build_range_f64(int natoms, int centre_begin, int centre_end, const double *h_cell, const double *d_coords,
                                           int is_cart, double rcut, const int *h_pbc, const double *h_open_extent, int umax,
                                           int reuse_bins, int *d_numneigh,
                                           int *d_firstneigh, double *d_rcs, int *d_status, void *d_workspace, size_t workspace_bytes,
                                           void *stream)
{
    return nblist_build<double>(natoms, centre_end, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                                d_status, d_workspace, workspace_bytes, (cudaStream_t)stream, centre_begin, reuse_bins != 0, h_open_extent);
}
extern "C" int ai2b_nblist_build_range_f32(int natoms, int centre_begin, int centre_end, const float *h_cell, const float *d_coords,
                                           int is_cart, double rcut, const int *h_pbc, const double *h_open_extent, int umax,
                                           int reuse_bins, int *d_numneigh,
                                           int *d_firstneigh, float *d_rcs, int *d_status, void *d_workspace, size_t workspace_bytes,
                                           void *stream)
{
    return nblist_build<float>(natoms, centre_end, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                               d_status, d_workspace, workspace_bytes, (cudaStream_t)stream, centre_begin, reuse_bins != 0, h_open_extent);
}
// Double-precision positions, single-precision rows: r_j - r_i is formed in double and rounded once, as
// PairAI2Pot::construct_mlff_input does on the host (interface/lammps/AI2POT/pair_ai2pot.cpp:232-235).
extern "C" int ai2b_nblist_build_ghost_f64_rows32(int natoms, int ncentres, const double *h_cell, const double *d_coords, int is_cart,
                                                  double rcut, const int *h_pbc, int umax, int *d_numneigh, int *d_firstneigh,
                                                  float *d_rcs, int *d_status, void *d_workspace, size_t workspace_bytes,
                                                  void *stream)
{
    return nblist_build<double, float>(natoms, ncentres, h_cell, d_coords, is_cart, rcut, h_pbc, umax, d_numneigh, d_firstneigh, d_rcs,
                                       d_status, d_workspace, workspace_bytes, (cudaStream_t)stream);
}
