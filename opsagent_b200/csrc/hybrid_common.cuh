// hybrid_common.cuh — small device helpers shared by the hybrid family's kernel files: typed loads / stores of the activation type
// (bf16 or fp32, arithmetic always fp32), activations, block reductions, cp.async, and the launch wrapper that joins every kernel to the
// stream's programmatic-dependent-launch chain.
#pragma once
#include <cuda_bf16.h>
#include <math.h>

#include <utility>

#include "common.cuh"
#include "kernels.hpp"

namespace oa {
namespace hyk {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanhf_(float z) { return gelu_tanh_f32(z); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// sum over the block (blockDim.x <= 1024, a multiple of 32); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}

// Every kernel of the family opens with HY_PDL(): it lets the next kernel of the stream become resident early (programmatic dependent
// launch) and then waits until every predecessor grid has completed and its memory is visible — nothing is read or written before that, so
// the kernels stay strictly ordered; what overlaps is only the launch latency and the ramp of the next grid.
#define HY_PDL() do { griddep_launch(); griddep_wait(); } while (0)
template <typename... KArgs, typename... Args>
cudaError_t launch_plain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    return launch_k(kern, grid, block, smem, st, std::forward<Args>(args)...);
}


}  // namespace hyk
}  // namespace oa
