// Plain CUDA-core matrix product  C[M,N] (=|+=) A[M,K] * W[N,K]^T  with fp32
// accumulation by FFMA: no tensor cores and no reduced-precision mode, so it is
// the product of the true 32-bit path and the fallback of the bf16 path for
// shapes that the tensor-core kernels refuse.
//
// W is [out, in] as the checkpoints store it, the layout the reference's
// matrix-vector kernels read (src/lfm25_gpu.cu:148-202); `accumulate` adds into
// an fp32 C, which is how the residual stream takes a projection's result
// (the reference's accum=true: src/lfm25_engine.c:380,405,419).
//
// Every element of C is summed over k = 0..K-1 in ascending order by one thread,
// so its value does not depend on M, on which rows share a tile, or on the grid.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename AT, typename WT, typename CT, bool ACCUM>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const AT* __restrict__ A, const WT* __restrict__ W, CT* __restrict__ C,
                  int M, int N, int K, long long lda, long long ldw, long long ldc) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2;          // 0..63: tile row loaded by this thread
    const int lk = (tid & 3) * 4;     // first of its 4 k values
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lr, gn = n0 + lr;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gk = k0 + lk + j;
                As[lk + j][lr] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
                Ws[lk + j][lr] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            CT* p = C + (size_t)gm * ldc + gn;
            if (ACCUM) *p = from_f32<CT>(to_f32(*p) + acc[i][j]);
            else *p = from_f32<CT>(acc[i][j]);
        }
    }
}
}  // namespace

extern "C" int tuff_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                               int M, int N, int K, long long lda, long long ldw, long long ldc,
                               int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return TUFF_E_SIZE;
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
#define GO(AT, WT, CT, ACC) gemm_plain_kernel<AT, WT, CT, ACC><<<grid, 256, 0, stream>>>( \
        (const AT*)A, (const WT*)W, (CT*)C, M, N, K, lda, ldw, ldc)
    if (accumulate && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if (a_dtype == TUFF_F32 && w_dtype == TUFF_F32 && c_dtype == TUFF_F32) {
        if (accumulate) GO(float, float, float, true); else GO(float, float, float, false);
    } else if (a_dtype == TUFF_BF16 && w_dtype == TUFF_BF16 && c_dtype == TUFF_BF16) {
        GO(bf16, bf16, bf16, false);
    } else if (a_dtype == TUFF_BF16 && w_dtype == TUFF_BF16 && c_dtype == TUFF_F32) {
        if (accumulate) GO(bf16, bf16, float, true); else GO(bf16, bf16, float, false);
    } else if (a_dtype == TUFF_F32 && w_dtype == TUFF_BF16 && c_dtype == TUFF_F32) {
        if (accumulate) GO(float, bf16, float, true); else GO(float, bf16, float, false);
    } else {
        return TUFF_E_DTYPE;
    }
#undef GO
    return launch_status();
}
