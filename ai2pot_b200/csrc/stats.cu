// Dataset statistics that feed the descriptor scaler and the target normaliser before training:
// per-component mean and sum of squared deviations of the descriptors (all atoms / per centre
// type), their max / min, and energy-per-atom / force statistics of the reference data.
//
// Reference semantics: source/descriptor/fitutils/include/descriptorsStatistics.h:76-205 (two
// passes: mean, then M2 = sum (x - mean)^2; max starts at FLT_MIN, min at FLT_MAX),
// targetStatistics.h:44-80. The reference sums sequentially in T; here every sum is accumulated
// in double and rounded once.
#include "common.cuh"

#include <cfloat>

namespace ai2b {

constexpr int ST_THREADS = 256;

__device__ __forceinline__ double block_sum(double v, double *sh)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double r = 0.0;
    for (int w = 0; w < ST_THREADS / 32; w++) r += sh[w];
    return r;
}

// grid (nd, ntypes or 1): block (k, t) owns component k of centre type t (all types if !btypes)
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
desc_stats_kernel(int *__restrict__ natoms_out, T *__restrict__ mean_out, T *__restrict__ m2_out, int B, int npad, int nd,
                  const int *__restrict__ binum, const int *__restrict__ bilist, const int *__restrict__ btypes,
                  const T *__restrict__ bdesc)
{
    __shared__ double sh[ST_THREADS / 32];
    const int k = blockIdx.x, t = blockIdx.y;
    const long rows = (long)B * npad;
    auto selected = [&](long row) {
        const int b = (int)(row / npad), ii = (int)(row % npad);
        if (ii >= binum[b]) return false;
        if (!btypes) return true;
        return btypes[(size_t)b * npad + bilist[(size_t)b * npad + ii]] == t;
    };
    double s = 0.0, c = 0.0;
    for (long row = threadIdx.x; row < rows; row += ST_THREADS)
        if (selected(row)) { s += (double)bdesc[row * nd + k]; c += 1.0; }
    s = block_sum(s, sh);
    c = block_sum(c, sh);
    const T mean = c > 0.0 ? (T)(s / c) : T(0);
    double m2 = 0.0;
    for (long row = threadIdx.x; row < rows; row += ST_THREADS)
        if (selected(row)) { const double d = (double)(T)(bdesc[row * nd + k] - mean); m2 += d * d; }
    m2 = block_sum(m2, sh);
    if (threadIdx.x == 0) {
        mean_out[(size_t)t * nd + k] = mean;
        m2_out[(size_t)t * nd + k] = (T)m2;
        if (k == 0) natoms_out[t] = (int)c;
    }
}

template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
desc_maxmin_kernel(T *__restrict__ max_out, T *__restrict__ min_out, int B, int npad, int nd, const int *__restrict__ binum,
                   const T *__restrict__ bdesc)
{
    __shared__ T smx[ST_THREADS / 32], smn[ST_THREADS / 32];
    const int k = blockIdx.x;
    const long rows = (long)B * npad;
    T mx = (T)FLT_MIN, mn = (T)FLT_MAX;   // the reference's starting values (descriptorsStatistics.h:190-193)
    for (long row = threadIdx.x; row < rows; row += ST_THREADS) {
        const int b = (int)(row / npad), ii = (int)(row % npad);
        if (ii >= binum[b]) continue;
        const T x = bdesc[row * nd + k];
        mx = mx > x ? mx : x;
        mn = mn < x ? mn : x;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const T a = __shfl_xor_sync(FULL_MASK, mx, o), b = __shfl_xor_sync(FULL_MASK, mn, o);
        mx = mx > a ? mx : a;
        mn = mn < b ? mn : b;
    }
    if ((threadIdx.x & 31) == 0) { smx[threadIdx.x >> 5] = mx; smn[threadIdx.x >> 5] = mn; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ST_THREADS / 32; w++) { mx = mx > smx[w] ? mx : smx[w]; mn = mn < smn[w] ? mn : smn[w]; }
        max_out[k] = mx; min_out[k] = mn;
    }
}

// one block: natoms, mean and M2 of the energy per atom over structures, sum of squared force components
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
target_stats_kernel(int *__restrict__ natoms_out, T *__restrict__ out3, int B, int npad, const int *__restrict__ binum,
                    const T *__restrict__ etot, const T *__restrict__ force)
{
    __shared__ double sh[ST_THREADS / 32];
    double n = 0.0, es = 0.0, f2 = 0.0;
    for (int b = threadIdx.x; b < B; b += ST_THREADS) { n += binum[b]; es += (double)(T)(etot[b] / (T)binum[b]); }
    for (long row = threadIdx.x; row < (long)B * npad; row += ST_THREADS) {
        const int b = (int)(row / npad), ii = (int)(row % npad);
        if (ii >= binum[b]) continue;
#pragma unroll
        for (int a = 0; a < 3; a++) { const double f = (double)force[row * 3 + a]; f2 += f * f; }
    }
    n = block_sum(n, sh); es = block_sum(es, sh); f2 = block_sum(f2, sh);
    const T mean = (T)(es / B);
    double m2 = 0.0;
    for (int b = threadIdx.x; b < B; b += ST_THREADS) { const double d = (double)(T)(etot[b] / (T)binum[b] - mean); m2 += d * d; }
    m2 = block_sum(m2, sh);
    if (threadIdx.x == 0) { natoms_out[0] = (int)n; out3[0] = mean; out3[1] = (T)m2; out3[2] = (T)f2; }
}

template <typename T>
static int desc_stats(int *natoms, T *mean, T *m2, int B, int npad, int nd, const int *binum, const int *bilist, const int *btypes,
                      int ntypes, const T *bdesc, cudaStream_t st)
{
    AI2B_REQUIRE(natoms && mean && m2 && binum && bdesc, AI2B_ERR_INVALID, "descriptor statistics: NULL argument");
    AI2B_REQUIRE(B >= 0 && npad >= 0 && nd >= 1 && ntypes >= 1 && ntypes <= 65535, AI2B_ERR_INVALID, "descriptor statistics: bad size");
    AI2B_REQUIRE(!btypes || bilist, AI2B_ERR_INVALID, "descriptor statistics: per-type statistics need bilist");
    desc_stats_kernel<T><<<dim3((unsigned)nd, (unsigned)(btypes ? ntypes : 1)), ST_THREADS, 0, st>>>(natoms, mean, m2, B, npad, nd, binum,
                                                                                                   bilist, btypes, bdesc);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

// out[off_k + i] = sum_b w[b] * part_k[b * n_k + i] for up to WS_MAX_PARTS row-major [B][n_k] arrays in one launch
constexpr int WS_MAX_PARTS = 8;
template <typename T>
struct WsParts {
    const T *p[WS_MAX_PARTS];
    int off[WS_MAX_PARTS + 1];   // start of part k in the output; off[nparts] = total
    int nparts;
};
template <typename T>
__global__ void weighted_sum_rows_kernel(WsParts<T> P, int B, const T *__restrict__ w, T *__restrict__ out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P.off[P.nparts]) return;
    int k = 0;
#pragma unroll
    for (int q = 1; q < WS_MAX_PARTS; q++) if (q < P.nparts && i >= P.off[q]) k = q;
    const int n = P.off[k + 1] - P.off[k];
    const T *src = P.p[k] + (i - P.off[k]);
    T acc0 = T(0), acc1 = T(0);   // two chains: B is a few dozen, the loads are independent
    int b = 0;
    for (; b + 1 < B; b += 2) {
        acc0 = fma(w ? w[b] : T(1), src[(size_t)b * n], acc0);
        acc1 = fma(w ? w[b + 1] : T(1), src[(size_t)(b + 1) * n], acc1);
    }
    if (b < B) acc0 = fma(w ? w[b] : T(1), src[(size_t)b * n], acc0);
    out[i] = acc0 + acc1;
}

template <typename T>
static int weighted_sum_rows(int nparts, const T *const *parts, const int *n, int B, const T *w, T *out, cudaStream_t st)
{
    AI2B_REQUIRE(nparts >= 1 && nparts <= WS_MAX_PARTS && parts && n && out && B >= 0, AI2B_ERR_INVALID,
                 "ai2b_weighted_sum_rows: bad argument (1..%d parts)", WS_MAX_PARTS);
    WsParts<T> P;
    P.nparts = nparts;
    P.off[0] = 0;
    for (int k = 0; k < WS_MAX_PARTS; k++) {
        P.p[k] = k < nparts ? parts[k] : nullptr;
        if (k < nparts) {
            AI2B_REQUIRE(n[k] >= 0 && (n[k] == 0 || parts[k]), AI2B_ERR_INVALID, "ai2b_weighted_sum_rows: part %d is NULL or negative", k);
            P.off[k + 1] = P.off[k] + n[k];
        } else {
            P.off[k + 1] = P.off[k];
        }
    }
    const int total = P.off[nparts];
    if (total == 0) return AI2B_OK;
    weighted_sum_rows_kernel<T><<<(total + 127) / 128, 128, 0, st>>>(P, B, w, out);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

#define AI2B_DEF_STATS(SUF, T)                                                                                         \
    extern "C" int ai2b_desc_stats_all_##SUF(int *d_natoms, T *d_mean, T *d_m2, int B, int npad, int nd,               \
                                             const int *d_binum, const T *d_bdesc, void *stream)                       \
    {                                                                                                                  \
        return desc_stats<T>(d_natoms, d_mean, d_m2, B, npad, nd, d_binum, nullptr, nullptr, 1, d_bdesc,               \
                             (cudaStream_t)stream);                                                                    \
    }                                                                                                                  \
    extern "C" int ai2b_desc_stats_each_##SUF(int *d_natoms, T *d_mean, T *d_m2, int B, int npad, int nd,              \
                                              const int *d_binum, const int *d_bilist, const int *d_btypes,            \
                                              int ntypes, const T *d_bdesc, void *stream)                              \
    {                                                                                                                  \
        AI2B_REQUIRE(d_btypes, AI2B_ERR_INVALID, "ai2b_desc_stats_each: NULL btypes");                                 \
        return desc_stats<T>(d_natoms, d_mean, d_m2, B, npad, nd, d_binum, d_bilist, d_btypes, ntypes, d_bdesc,        \
                             (cudaStream_t)stream);                                                                    \
    }                                                                                                                  \
    extern "C" int ai2b_desc_maxmin_##SUF(T *d_max, T *d_min, int B, int npad, int nd, const int *d_binum,             \
                                          const T *d_bdesc, void *stream)                                              \
    {                                                                                                                  \
        AI2B_REQUIRE(d_max && d_min && d_binum && d_bdesc && nd >= 1 && B >= 0 && npad >= 0, AI2B_ERR_INVALID,         \
                     "ai2b_desc_maxmin: bad argument");                                                                \
        desc_maxmin_kernel<T><<<nd, ST_THREADS, 0, (cudaStream_t)stream>>>(d_max, d_min, B, npad, nd, d_binum, d_bdesc); \
        AI2B_CUDA(cudaGetLastError());                                                                                 \
        return AI2B_OK;                                                                                                \
    }                                                                                                                  \
    extern "C" int ai2b_target_stats_##SUF(int *d_natoms, T *d_out3, int B, int npad, const int *d_binum,              \
                                           const T *d_betot, const T *d_bforce, void *stream)                          \
    {                                                                                                                  \
        AI2B_REQUIRE(d_natoms && d_out3 && d_binum && d_betot && d_bforce && B >= 1 && npad >= 0, AI2B_ERR_INVALID,    \
                     "ai2b_target_stats: bad argument");                                                               \
        target_stats_kernel<T><<<1, ST_THREADS, 0, (cudaStream_t)stream>>>(d_natoms, d_out3, B, npad, d_binum,         \
                                                                          d_betot, d_bforce);                          \
        AI2B_CUDA(cudaGetLastError());                                                                                 \
        return AI2B_OK;                                                                                                \
    }

AI2B_DEF_STATS(f64, double)
AI2B_DEF_STATS(f32, float)

#define AI2B_DEF_WSUM(SUF, T)                                                                                          \
    extern "C" int ai2b_weighted_sum_rows_##SUF(int nparts, const T *const *h_parts, const int *h_n, int B,            \
                                                const T *d_w, T *d_out, void *stream)                                  \
    {                                                                                                                  \
        return weighted_sum_rows<T>(nparts, h_parts, h_n, B, d_w, d_out, (cudaStream_t)stream);                        \
    }
AI2B_DEF_WSUM(f64, double)
AI2B_DEF_WSUM(f32, float)
