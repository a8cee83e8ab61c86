// Multinomial rows over the full vocabulary (no active top-k), bit for bit as the reference computes
// them on the host:
//   TemperatureLogitTransform   src/cpp/src/sampling/logit_transformers.hpp:299-362
//       p_i = expf((x_i - max) * (1 / T)), sum in index order in single precision, p_i /= sum
//   MinPFilter                  logit_transformers.hpp:157-190   (keep p_i >= float(min_p) * p_max)
//   TopPFilter                  logit_transformers.hpp:94-139    (sort descending, add until the float sum > top_p)
//   Sampler::_multinomial_sample  src/cpp/src/sampling/sampler.cpp:1036-1089
//       total = sum of the kept probabilities in their order, r = total * u, first running sum > r
// Every float the reference produces on the way is reproduced: expf with the host libm's bits and
// the sequential sums through the step algebra of fsum_exact.cuh, so token ids agree with the
// reference except where several kept elements have exactly the same probability and the draw falls
// among them (their relative order after std::sort is not defined; the lowest index is taken here).
//
// One CTA works on one row at a time (persistent grid, rows dealt round robin).  Passes over a row:
//   1. maximum;  2. expf and the index-order sum (tile by tile, a block scan of steps per tile), the
//   exponentials parked in a per-CTA scratch row;  3. division by the sum, probabilities back to the
//   scratch row, and either the index-order total (no top-p) or the first level's bin counts;
//   then, without top-p, one more partial pass that stops at the drawn element; with top-p the
//   walk of fsum_exact.cuh: a few passes that sum whole bins as translations and list the rest.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sampler_b200.h"
#include "fsum_exact.cuh"
#include "sampler_kernels.h"

namespace sampler {

// Two CTA sizes: 512 threads with two CTAs per SM while there are more rows than SMs (two rows share an SM and fill each
// other's sequential phases), 1024 threads with one CTA per SM for small batches (a row's passes take about half as long).
namespace {
namespace sx512 {
#define SX_THREADS 512
#define SX_CTAS_PER_SM 2
#include "sampler_exact_impl.cuh"
#undef SX_THREADS
#undef SX_CTAS_PER_SM
}  // namespace sx512
namespace sx1024 {
#define SX_THREADS 1024
#define SX_CTAS_PER_SM 1
#include "sampler_exact_impl.cuh"
#undef SX_THREADS
#undef SX_CTAS_PER_SM
}  // namespace sx1024

__global__ void expf_selftest_kernel(const float* in, float* out, long long n) {
    __shared__ uint64_t tab[32];
    if (threadIdx.x < 32) tab[threadIdx.x] = fsx::kExp2TabDev[threadIdx.x];
    __syncthreads();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) out[i] = fsx::expf_libm(in[i], tab);
}

}  // namespace

cudaError_t launch_expf_selftest(const float* in, float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    expf_selftest_kernel<<<592, 256, 0, stream>>>(in, out, n);
    return cudaGetLastError();
}

size_t sampler_exact_smem_bytes() { return sizeof(sx512::ExactShared) > sizeof(sx1024::ExactShared) ? sizeof(sx512::ExactShared) : sizeof(sx1024::ExactShared); }

size_t sampler_exact_scratch_bytes(int ctas, long long vocab) { return (size_t)ctas * (size_t)((vocab + 3) & ~3LL) * sizeof(float); }

cudaError_t launch_sampler_exact(const StepArgs& a, float* scratch, int ctas, cudaStream_t stream) {
    if (a.num_rows <= 0 || ctas <= 0) return cudaSuccess;
    const int grid = a.num_rows < ctas ? a.num_rows : ctas;
    if (a.num_rows * 2 <= ctas) {   // at most one row per SM (ctas = 2 per SM): the large CTA
        cudaError_t e = cudaFuncSetAttribute(sx1024::sampler_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(sx1024::ExactShared));
        if (e != cudaSuccess) return e;
        sx1024::sampler_exact_kernel<<<grid, 1024, sizeof(sx1024::ExactShared), stream>>>(a, scratch);
        return cudaGetLastError();
    }
    cudaError_t e = cudaFuncSetAttribute(sx512::sampler_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(sx512::ExactShared));
    if (e != cudaSuccess) return e;
    sx512::sampler_exact_kernel<<<grid, 512, sizeof(sx512::ExactShared), stream>>>(a, scratch);
    return cudaGetLastError();
}

}  // namespace sampler
