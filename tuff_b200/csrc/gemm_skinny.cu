// bf16 matrix product for a handful of tokens (decode):  C[M,N] (=|+=) A[M,K] * W[N,K]^T, M <= 16.
//
// With so few tokens the product is a stream of the weights through the SMs: the
// time is the bytes of W over the HBM bandwidth, and what matters is that every
// SM keeps enough loads in flight.  A CTA of 4, 8 or 16 warps owns 8 output rows (8 rows
// of W); each warp takes a contiguous share of K, loads 16 bytes of a weight row
// per lane straight from global memory into the operand registers of
// mma.sync.m16n8k16 (tokens are the 16-row side, the 8 weight rows the 8-column
// side), and the warps' partial tiles are added in warp order through shared memory,
// so the sum does not depend on timing.  With `swiglu` the CTA also streams the
// matching 8 rows of the "up" half of a stacked [gate; up] matrix and writes
// silu(gate) * up, which is the reference's fused gate/up kernel
// (src/lfm25_gpu.cu:583-618); `accumulate` adds into the fp32 residual stream
// (its accum=true, src/lfm25_engine.c:380,405,419).
//
// The 16-byte loads give each lane 8 consecutive k of its row; the two MMAs per
// load pair use the k order (8t, 8t+1, 8t+2, 8t+3 | 8t+4 ..) for both operands,
// which is a permutation of k inside the 32-wide step and leaves the dot products
// unchanged.
#include "common.cuh"

namespace {
constexpr int ROWS = 8;        // output rows per CTA
constexpr int KSTEP = 32;      // k per warp step
constexpr int CHUNK = 8;       // steps whose weight loads are issued together

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// HI: tokens 8..15 exist.  SWIGLU: W is [2F, K], rows n and F+n are combined.
template <int WARPS, bool HI, bool SWIGLU, typename CT, bool ACCUM>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, CT* __restrict__ C,
                   int M, int N, int K, long long lda, long long ldw, long long ldc, int F) {
    __shared__ float red[SWIGLU ? 2 : 1][WARPS][16][ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int n_rows = SWIGLU ? F : N;                 // rows of the output
    const int row = n0 + g;
    const bool row_ok = row < n_rows;
    // this warp's K range, in whole steps
    const int steps = (K + KSTEP - 1) / KSTEP;
    const int per = (steps + WARPS - 1) / WARPS;
    const int s_begin = warp * per, s_end = min(steps, s_begin + per);

    const bf16* w_row = W + (size_t)(row_ok ? row : 0) * ldw;
    const bf16* u_row = SWIGLU ? W + (size_t)(row_ok ? row + F : 0) * ldw : nullptr;
    const bf16* x_lo = A + (size_t)(g < M ? g : 0) * lda;
    const bf16* x_hi = A + (size_t)(g + 8 < M ? g + 8 : 0) * lda;
    const bool lo_ok = g < M, hi_ok = HI && (g + 8 < M);

    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // The weight loads of a chunk of steps are all issued before the first is used, so that
    // every lane has CHUNK (or 2*CHUNK) 16-byte loads in flight: with matrices of a few
    // megabytes the whole matrix is on its way at once, and the time is one trip to HBM.
#pragma unroll 1
    for (int s0 = s_begin; s0 < s_end; s0 += CHUNK) {
        uint4 wv[CHUNK], uv[SWIGLU ? CHUNK : 1];
#pragma unroll
        for (int u = 0; u < CHUNK; ++u) {
            const int k = (s0 + u) * KSTEP + t * 8;
            const bool ok = row_ok && (s0 + u) < s_end && k < K;     // K % 8 == 0: a lane's 8 k are all in or all out
            wv[u] = ok ? ldg_stream(w_row + k) : zero;
            if (SWIGLU) uv[u] = ok ? ldg_stream(u_row + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < CHUNK; ++u) {
            const int k = (s0 + u) * KSTEP + t * 8;
            const bool ok = (s0 + u) < s_end && k < K;
            const uint4 xa = (lo_ok && ok) ? ldg_cached(x_lo + k) : zero;
            const uint4 xb = (hi_ok && ok) ? ldg_cached(x_hi + k) : zero;
            mma16816(acc, xa.x, xb.x, xa.y, xb.y, wv[u].x, wv[u].y);
            mma16816(acc, xa.z, xb.z, xa.w, xb.w, wv[u].z, wv[u].w);
            if (SWIGLU) {
                mma16816(acc_u, xa.x, xb.x, xa.y, xb.y, uv[u].x, uv[u].y);
                mma16816(acc_u, xa.z, xb.z, xa.w, xb.w, uv[u].z, uv[u].w);
            }
        }
    }
    // acc[0], acc[1]: token g, rows n0+2t, n0+2t+1; acc[2], acc[3]: token g+8
    red[0][warp][g][2 * t] = acc[0];
    red[0][warp][g][2 * t + 1] = acc[1];
    red[0][warp][g + 8][2 * t] = acc[2];
    red[0][warp][g + 8][2 * t + 1] = acc[3];
    if (SWIGLU) {
        red[1][warp][g][2 * t] = acc_u[0];
        red[1][warp][g][2 * t + 1] = acc_u[1];
        red[1][warp][g + 8][2 * t] = acc_u[2];
        red[1][warp][g + 8][2 * t + 1] = acc_u[3];
    }
    __syncthreads();
    const int tok = threadIdx.x >> 3, r = threadIdx.x & 7;      // the first 128 threads: 16 tokens x 8 rows
    if (threadIdx.x < 128 && tok < M && n0 + r < n_rows) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[0][w][tok][r];
        if (SWIGLU) {
            float u = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) u += red[1][w][tok][r];
            // the unfused path rounds gate and up to bf16 before the activation; so does this one
            const float gq = __bfloat162float(__float2bfloat16_rn(v)), uq = __bfloat162float(__float2bfloat16_rn(u));
            v = gq / (1.f + expf(-gq)) * uq;
        }
        CT* p = C + (size_t)tok * ldc + n0 + r;
        if (ACCUM) *p = from_f32<CT>(to_f32(*p) + v);
        else *p = from_f32<CT>(v);
    }
}
}  // namespace

// C[M,N] (=|+=) A[M,K] W[N,K]^T for M <= 16; A and W bf16 with K % 8 == 0, row strides % 8 == 0 and
// 16-byte aligned bases.  swiglu != 0: W is [2N, K] (gate rows then up rows) and C[M,N] = silu(gate)*up.
extern "C" int tuff_gemm_skinny(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K,
                                long long lda, long long ldw, long long ldc, int accumulate, int swiglu,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0) return TUFF_E_SIZE;
    if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TUFF_E_ALIGN;
    if (accumulate && (c_dtype != TUFF_F32 || swiglu)) return TUFF_E_DTYPE;
    dim3 grid(ceil_div(N, ROWS));
    const bf16* a = (const bf16*)A; const bf16* w = (const bf16*)W;
    // enough warps along K that a warp's share is about one chunk of steps
    const int steps = ceil_div(K, KSTEP);
    const int warps = steps <= 4 * CHUNK ? 4 : steps <= 8 * CHUNK ? 8 : 16;
#define GO3(WP, HI, SW, CT, ACC) gemm_skinny_kernel<WP, HI, SW, CT, ACC><<<grid, WP * 32, 0, stream>>>( \
        a, w, (CT*)C, M, N, K, lda, ldw, ldc, N)
#define GO(HI, SW, CT, ACC) do { if (warps == 4) GO3(4, HI, SW, CT, ACC); else if (warps == 8) GO3(8, HI, SW, CT, ACC); \
        else GO3(16, HI, SW, CT, ACC); } while (0)
    const bool hi = M > 8;
    if (swiglu) {
        if (c_dtype != TUFF_BF16) return TUFF_E_DTYPE;
        if (hi) GO(true, true, bf16, false); else GO(false, true, bf16, false);
    } else if (c_dtype == TUFF_BF16) {
        if (hi) GO(true, false, bf16, false); else GO(false, false, bf16, false);
    } else if (c_dtype == TUFF_F32) {
        if (accumulate) { if (hi) GO(true, false, float, true); else GO(false, false, float, true); }
        else { if (hi) GO(true, false, float, false); else GO(false, false, float, false); }
    } else {
        return TUFF_E_DTYPE;
    }
#undef GO
#undef GO3
    return launch_status();
}
