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
#include <stdlib.h>

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

// ---- programmatic dependent launch -------------------------------------------------------
// A kernel launched with `launch_pdl` may start while the kernel before it in the stream is
// still running.  It must call pdl_wait() before it reads or writes anything that an earlier
// kernel touches; what it does before that (setting up barriers, prefetching weights, which no
// kernel writes) overlaps the predecessor's tail.  pdl_launch_dependents() lets the next
// kernel in the stream be scheduled as soon as this one's blocks have all started.  Since every
// kernel waits for its predecessor to finish completely before it touches shared data, and
// that predecessor did the same, the chain stays ordered.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Loads of data that an earlier kernel (or a copy) wrote.  A kernel that starts before its
// predecessor has finished shares the SM, and its L1, with kernels that read the same addresses
// earlier; buffers are reused from layer to layer and from step to step, so a line left in L1
// may be stale.  These loads go to L2 (ld.global.cg), which is coherent.  Weights, which no
// kernel writes, may use any load.
__device__ __forceinline__ float ld_act(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_act(const bf16* p) {
    return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}
__device__ __forceinline__ int ld_act(const int* p) { return __ldcg(p); }
__device__ __forceinline__ uint32_t ld_act_u32(const void* p) { return __ldcg(reinterpret_cast<const unsigned int*>(p)); }
__device__ __forceinline__ uint4 ld_act_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Nanoseconds of the GPU's global timer (for the kernels' optional time stamps).
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        // On unless TUFF_PDL=0.  Measured on the 1.2B shape: the prefill of 2,048 tokens 4.17 -> 3.95 ms (the
        // tensor-core products set themselves up beside the norm or convolution before them), a mixed
        // step 3.32 -> 3.13 ms, decode steps within 1 % either way (their products fill the register
        // file, so the next kernel cannot become resident early).
        const char* e = getenv("TUFF_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Number of SMs of the current device (asked once per device): grids of persistent CTAs are sized by it.
static inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 1;
        cached[dev] = v;
    }
    return cached[dev];
}
