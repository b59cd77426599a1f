// FMA-pipe microbenchmark: the measured denominator for the FP64 / FP32 roofline fractions.
// Not part of the product library: built as its own shared object (libai2b_fma_peak.so) that only the
// benchmark loads.
#include <cuda_runtime.h>

namespace ai2b {

template <typename T>
__global__ void fma_chain_kernel(T *out, int iters, T a, T b)
{
    T x[8];
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = T(threadIdx.x + k) * T(1e-3);
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 8; k++) x[k] = fma(x[k], a, b);
    }
    T s = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) s += x[k];
    if (s == T(-1.2345)) out[blockIdx.x * blockDim.x + threadIdx.x] = s;   // never true; keeps the loop alive
}

}  // namespace ai2b

// Launches `blocks` x 256 threads, each doing 8 independent chains of `iters` FMAs.
// flops per launch = blocks * 256 * 8 * iters * 2. d_out must hold blocks*256 elements.
extern "C" int ai2b_bench_fma_chain(int is_f64, int blocks, int iters, void *d_out, void *stream)
{
    if (blocks <= 0 || iters <= 0 || !d_out) return -1;
    if (is_f64) ai2b::fma_chain_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((double *)d_out, iters, 0.999999, 1e-7);
    else ai2b::fma_chain_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float *)d_out, iters, 0.999999f, 1e-7f);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
