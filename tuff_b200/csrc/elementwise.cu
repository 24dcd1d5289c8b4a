// Row-wise kernels: embedding gather, RMSNorm, SwiGLU activation, dtype cast.
//
// What each computes follows the reference's LFM2.5 path:
//   embedding   x = E[token]                                  (src/lfm25_gpu.cu:725-741)
//   RMSNorm     y = x * rsqrt(mean(x^2) + eps) * w, statistics in fp32, the weight
//               multiplies directly                            (src/lfm25_gpu.cu:207-262)
//   SwiGLU      act = gate / (1 + exp(-gate)) * up             (src/lfm25_gpu.cu:583-618)
// The kernels themselves are written for bf16/fp32 activations on sm_100a; the
// reference's are Q8_1/Q4_K kernels for sm_86.
#include "common.cuh"
#include <algorithm>

// ---------------------------------------------------------------- embedding
template <typename WT>
__global__ void embed_kernel(const int* __restrict__ tokens, const WT* __restrict__ table,
                             float* __restrict__ out, int d, int vocab) {
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    int tok = ld_act(tokens + t);
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok) tok = 0;
    const WT* row = table + (size_t)tok * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}

extern "C" int tuff_embed(const int* tokens, const void* table, int table_dtype, float* out,
                          int n_tokens, int d, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == TUFF_F32)
        return launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, out, d, vocab);
    else if (table_dtype == TUFF_BF16)
        return launch_pdl(embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const bf16*)table, out, d, vocab);
    return TUFF_E_DTYPE;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  `row_index` (may be null) picks the input row of
// each output row, which is how the head norms only the rows whose logits are
// wanted.  The sum of squares is accumulated per thread over a fixed stride and
// then across the block, so a row's result does not depend on the batch.
template <typename InT, typename OutT>
__global__ void rmsnorm_kernel(const InT* __restrict__ x, const float* __restrict__ w,
                               OutT* __restrict__ out, const int* __restrict__ row_index,
                               int d, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    pdl_wait();
    const int src = row_index ? ld_act(row_index + r) : r;
    const InT* xr = x + (size_t)src * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = ld_act(xr + i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    pdl_launch_dependents();
    const float scale = rsqrtf(ss / (float)d + eps);
    OutT* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        o[i] = from_f32<OutT>(ld_act(xr + i) * scale * w[i]);
}

// More than a handful of rows: one warp per row, one to eight rows per block (fewer rows, smaller blocks, so
// that they spread over the SMs).  A lane loads its share
// of the row as float4 (all loads in flight at once), keeps it in registers for the scaling, and
// writes packed output; no block-wide barrier.  Rows of up to 32 * 4 * RMS_VEC columns.
constexpr int RMS_VEC = 16;
template <typename OutT>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, OutT* __restrict__ out,
                    const int* __restrict__ row_index, int n_rows, int d, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    pdl_wait();
    pdl_launch_dependents();                     // the next kernel may set itself up beside this one
    if (r >= n_rows) return;
    const int src = row_index ? ld_act(row_index + r) : r;
    const float* xr = x + (size_t)src * d;
    float4 v[RMS_VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        const int k = (i * 32 + lane) * 4;
        if (k < d) v[i] = __ldcg(reinterpret_cast<const float4*>(xr + k));
    }
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        const int k = (i * 32 + lane) * 4;
        if (k < d) {
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)d + eps);
    OutT* o = out + (size_t)r * d;
#pragma unroll
    for (int i = 0; i < RMS_VEC; ++i) {
        const int k = (i * 32 + lane) * 4;
        if (k < d) {
            const float4 g = *reinterpret_cast<const float4*>(w + k);
            const float a = v[i].x * scale * g.x, b = v[i].y * scale * g.y, c = v[i].z * scale * g.z, e = v[i].w * scale * g.w;
            if (sizeof(OutT) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(o) + k) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + k) = make_float4(a, b, c, e);
            }
        }
    }
}

extern "C" int tuff_rmsnorm(const void* x, int x_dtype, const float* w, void* out, int out_dtype,
                            const int* row_index, int n_rows, int d, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    // The warp-per-row kernel adds a row's squares in another order than the block-per-row kernel.  Which of
    // the two runs depends on the number of rows, so only the bf16 path may use it: the 32-bit path gives
    // the same bits for a row whatever else is in the batch.
    if (x_dtype == TUFF_F32 && out_dtype == TUFF_BF16 && n_rows > 16 && d % 4 == 0 && d <= 128 * RMS_VEC && !((uintptr_t)x & 15) &&
        !((uintptr_t)w & 15) && !((uintptr_t)out & 15)) {
        const int warps = n_rows >= 2048 ? 8 : n_rows >= 512 ? 4 : n_rows >= 128 ? 2 : 1;
        const dim3 grid(ceil_div(n_rows, warps)), block(32 * warps);
        return launch_pdl(rmsnorm_rows_kernel<bf16>, grid, block, 0, stream, (const float*)x, w, (bf16*)out, row_index, n_rows, d, eps);
    }
    const int threads = 256;
    int rc = 0;
#define LAUNCH(IT, OT) rc = launch_pdl(rmsnorm_kernel<IT, OT>, dim3(n_rows), dim3(threads), 0, stream, \
        (const IT*)x, w, (OT*)out, row_index, d, eps)
    if (x_dtype == TUFF_F32 && out_dtype == TUFF_F32) LAUNCH(float, float);
    else if (x_dtype == TUFF_F32 && out_dtype == TUFF_BF16) LAUNCH(float, bf16);
    else if (x_dtype == TUFF_BF16 && out_dtype == TUFF_BF16) LAUNCH(bf16, bf16);
    else if (x_dtype == TUFF_BF16 && out_dtype == TUFF_F32) LAUNCH(bf16, float);
    else return TUFF_E_DTYPE;
#undef LAUNCH
    return rc ? rc : launch_status();
}

// ------------------------------------------------------------------- SwiGLU
// gu is [T, 2F]: per block of `blk` outputs, blk gate columns then blk up columns (blk = F: gate
// in columns [0,F), up in [F,2F)).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int n_tokens, int F, int blk) {
    const size_t total = (size_t)n_tokens * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F;
        const int f = (int)(i - t * F);
        const int gc = (f / blk) * 2 * blk + f % blk;
        const float g = to_f32(gu[t * 2 * F + gc]);
        const float u = to_f32(gu[t * 2 * F + gc + blk]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

extern "C" int tuff_swiglu(const void* gu, void* out, int dtype, int n_tokens, int F, int blk, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (blk <= 0) blk = F;
    if (F % blk) return TUFF_E_SIZE;
    const size_t total = (size_t)n_tokens * F;
    const int threads = 256;
    const size_t cap = (size_t)sm_count() * 16;
    const int blocks = (int)std::min((total + threads - 1) / threads, cap);
    if (dtype == TUFF_F32) swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, n_tokens, F, blk);
    else if (dtype == TUFF_BF16) swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, n_tokens, F, blk);
    else return TUFF_E_DTYPE;
    return launch_status();
}

// --------------------------------------------------------------------- cast
template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<B>(to_f32(in[i]));
}

extern "C" int tuff_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    long long want = (n + threads - 1) / threads;
    const int blocks = (int)std::min(want, (long long)sm_count() * 16);
    if (in_dtype == TUFF_F32 && out_dtype == TUFF_BF16) cast_kernel<float, bf16><<<blocks, threads, 0, stream>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == TUFF_BF16 && out_dtype == TUFF_F32) cast_kernel<bf16, float><<<blocks, threads, 0, stream>>>((const bf16*)in, (float*)out, (size_t)n);
    else return TUFF_E_DTYPE;
    return launch_status();
}
