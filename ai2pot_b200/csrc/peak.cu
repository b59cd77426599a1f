// FMA-pipe microbenchmark: the measured denominator for the FP64 / FP32 roofline fractions.
#include "common.cuh"

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
extern "C" int ai2b_fma_chain(int is_f64, int blocks, int iters, void *d_out, void *stream)
{
    AI2B_REQUIRE(blocks > 0 && iters > 0 && d_out, AI2B_ERR_INVALID, "ai2b_fma_chain: bad argument");
    if (is_f64) ai2b::fma_chain_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((double *)d_out, iters, 0.999999, 1e-7);
    else ai2b::fma_chain_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float *)d_out, iters, 0.999999f, 1e-7f);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}
