// Shared host/device helpers of the ai2pot_b200 CUDA library (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include "../../include/ai2pot_b200.h"

namespace ai2b {

// Records the calling thread's last error message (returned by ai2b_last_error_string()).
void set_error(const char *fmt, ...);

#define AI2B_CUDA(call)                                                                        \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            (void)cudaGetLastError(); /* a non-sticky error must not surface at a later launch check */ \
            ::ai2b::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, \
                              __LINE__);                                                       \
            return AI2B_ERR_CUDA;                                                              \
        }                                                                                      \
    } while (0)

#define AI2B_REQUIRE(cond, code, ...)                                                          \
    do {                                                                                       \
        if (!(cond)) {                                                                         \
            ::ai2b::set_error(__VA_ARGS__);                                                    \
            return (code);                                                                     \
        }                                                                                      \
    } while (0)

// ---- per-device launch set-up ---------------------------------------------------------------------
// The opt-in to more than 48 KB of dynamic shared memory (cudaFuncSetAttribute), the occupancy of a
// kernel and the SM count are properties of one device, so a process that drives several GPUs needs
// them once per device. One KernelSetup object (function-local static) per kernel instantiation
// remembers, for every device ordinal, what has been configured; access is serialised by its mutex
// so that host threads may launch concurrently.
constexpr int MAX_DEVICES = 64;

struct KernelSetup {
    std::mutex mu;
    size_t smem[MAX_DEVICES] = {};       // largest dynamic shared-memory size opted in so far
    size_t occ_smem[MAX_DEVICES] = {};   // shared-memory size per_sm was computed for (+1, 0 = never)
    int per_sm[MAX_DEVICES] = {};
};

// Makes `kern` launchable with `smem` bytes of dynamic shared memory on the current device; if
// per_sm is given, also returns the number of resident blocks of `threads` threads per SM (>= 1).
template <typename Kern>
static int kernel_setup(KernelSetup &ks, Kern kern, size_t smem, int threads = 0, int *per_sm = nullptr)
{
    int dev = 0;
    AI2B_CUDA(cudaGetDevice(&dev));
    const bool cached = dev >= 0 && dev < MAX_DEVICES;
    std::lock_guard<std::mutex> guard(ks.mu);
    if (!cached || smem > ks.smem[dev]) {
        if (smem > 48 * 1024)
            AI2B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (cached) ks.smem[dev] = smem;
    }
    if (per_sm) {
        if (!cached || ks.occ_smem[dev] != smem + 1) {
            int n = 0;
            AI2B_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem));
            if (n < 1) n = 1;
            if (!cached) { *per_sm = n; return AI2B_OK; }
            ks.per_sm[dev] = n;
            ks.occ_smem[dev] = smem + 1;
        }
        *per_sm = ks.per_sm[dev];
    }
    return AI2B_OK;
}

// SM count of the current device (cached per device ordinal).
int sm_count();

constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr int WARP = 32;

template <typename T>
__device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
    return v;
}

// compile-time loop: f(std::integral_constant<int, I>) for I in [I0, N)
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F &&f)
{
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

__host__ __device__ constexpr int pow2ceil(int n)
{
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}
__host__ __device__ constexpr int ilog2(int n)
{
    int l = 0;
    while ((1 << l) < n) ++l;
    return l;
}

// Sum over the 32 lanes of N per-lane values at once ("transpose-reduce"): on return lane l
// holds the warp total of v[l >> (5 - log2 N)]. N is a power of two <= 32. Uses N-1 exchange
// shuffles plus (5 - log2 N) butterfly steps instead of 5 N.
template <typename T, int N>
__device__ __forceinline__ T warp_xreduce(T (&v)[N], int lane)
{
    int o = 16;
#pragma unroll
    for (int h = N / 2; h >= 1; h >>= 1, o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < h; i++) {
            T send = up ? v[i] : v[i + h];
            T keep = up ? v[i + h] : v[i];
            v[i] = keep + __shfl_xor_sync(FULL_MASK, send, o);
        }
    }
    T r = v[0];
    for (; o >= 1; o >>= 1) r += __shfl_xor_sync(FULL_MASK, r, o);
    return r;
}

__device__ __forceinline__ double gsqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float gsqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double grsqrt(double x) { return rsqrt(x); }
__device__ __forceinline__ float grsqrt(float x) { return rsqrtf(x); }

// Chained launches (programmatic dependent launch). The launches of one evaluation form a chain on one stream, each
// kernel reading what the one before it wrote. launch_chained() lets the blocks of a kernel become resident while the
// kernel before it is still draining: they run whatever does not depend on earlier kernels (staging of model tables),
// then chain_wait() holds them until every earlier kernel of the stream has completed and its writes are visible.
// chain_release() in a kernel says that the next kernel of the chain may be made resident as soon as all blocks of
// this one have started. Rules: a kernel launched with launch_chained() executes chain_wait() in every thread before
// its first access to memory that another kernel writes or reads (so completion stays transitive along the chain);
// in a kernel launched the ordinary way both calls do nothing. With AI2B_CHAIN=0 in the environment launch_chained() launches the
// ordinary way.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    const char *env = std::getenv("AI2B_CHAIN");          // AI2B_CHAIN=0: ordinary launches (a switch for debugging), read per launch
    cfg.numAttrs = (env && env[0] == '0') ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(static_cast<Args &&>(args))...);
}

// number of monomials x^a y^b z^c with a+b+c <= k, and of exact degree d
__host__ __device__ constexpr int ncan(int k) { return k < 0 ? 0 : (k + 1) * (k + 2) * (k + 3) / 6; }
__host__ __device__ constexpr int ndeg(int d) { return (d + 1) * (d + 2) / 2; }

struct Exp3 {
    int x, y, z;
};
// q-th monomial of exact degree D in canonical order: x exponent descending, then y descending
__host__ __device__ constexpr Exp3 deg_exp(int D, int q)
{
    int ax = D;
    while (q >= D - ax + 1) {
        q -= (D - ax + 1);
        --ax;
    }
    int ay = D - ax - q;
    return Exp3{ax, ay, D - ax - ay};
}
// canonical index of (ax, ay, az) among all monomials, degree-major
__host__ __device__ constexpr int canon_index(int ax, int ay, int az)
{
    int D = ax + ay + az;
    int q = 0;
    for (int x = D; x > ax; --x) q += D - x + 1;
    q += (D - ax) - ay;
    return ncan(D - 1) + q;
}

}  // namespace ai2b
