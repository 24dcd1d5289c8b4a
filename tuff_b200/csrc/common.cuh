// Shared device helpers for the sm_100a kernels of this package.
//
// Conventions used by every launcher (`extern "C" int tuff_*`):
//   * tensors are raw device pointers, row-major, sizes passed as ints;
//   * an element type is passed as a code: 0 = float32, 1 = bfloat16;
//   * the last argument is the CUDA stream to launch on;
//   * the return value is the cudaError_t of the launch (0 = success) or a
//     negative value for an argument that the kernel refuses (see TUFF_E_*).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define TUFF_F32 0
#define TUFF_BF16 1

#define TUFF_E_DTYPE (-2)   // unsupported combination of element types
#define TUFF_E_SIZE (-3)    // a size outside what the kernel was written for
#define TUFF_E_ALIGN (-4)   // a pointer or stride that breaks an alignment rule

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024 threads).
// `scratch` holds 32 floats of shared memory.  Every thread gets the total, and
// the order of additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
