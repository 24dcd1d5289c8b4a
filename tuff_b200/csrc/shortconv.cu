// Gated short convolution over a batch of portions, continuing per-request state.
//
// Per channel c and token t of a request (reference: src/lfm25_gpu.cu:287-337 for
// one token, src/lfm25_gpu.cu:1046-1099 for consecutive tokens):
//   bcx = [B | C | x]  (three d-wide thirds of the in_proj output, in this order)
//   u_t = B_t * x_t
//   y_t = sum_{j=0..K-1} taps[c][j] * u_{t-(K-1)+j}      (tap K-1 meets the current token)
//   g_t = C_t * y_t
//   state after t = the last K-1 values of u, oldest first
// u before the request's first token is zero; u before the first token of this
// portion comes from the request's state slot.
//
// The reference walks a portion sequentially per channel.  Here every (token,
// channel) is computed independently from the K values of u it needs, so a long
// portion runs in parallel, and a second kernel rolls the state afterwards (the
// first one must only read it).  All arithmetic is fp32; the sum runs over the
// taps in ascending order whatever the portion's length, so cutting a prompt
// differently changes nothing.
#include "common.cuh"
#include "index.cuh"

namespace {

template <typename T>
__global__ void shortconv_fwd_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                     const float* __restrict__ state, const int* __restrict__ slot_of_row,
                                     const int* __restrict__ row_of_token, const int* __restrict__ cu_q,
                                     T* __restrict__ out, int n_tokens, int d, int K, Bounds bounds) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= d) return;
    const int r = row_of_token[t];
    if (!check_row(bounds, r) || !check_slot(bounds, slot_of_row[r])) return;
    const int i = t - cu_q[r];                 // index inside this portion
    const size_t ld = (size_t)3 * d;
    const float* st = state + slot_elem(slot_of_row[r], (size_t)(K - 1) * d);
    float y = 0.f;
    for (int j = 0; j < K; ++j) {
        const int back = (K - 1) - j;          // how many tokens before t
        float u;
        if (i - back >= 0) {
            const T* p = bcx + (size_t)(t - back) * ld;
            u = to_f32(p[c]) * to_f32(p[2 * d + c]);
        } else {
            u = st[(size_t)((K - 1) + (i - back)) * d + c];
        }
        y = fmaf(taps[(size_t)c * K + j], u, y);
    }
    out[(size_t)t * d + c] = from_f32<T>(to_f32(bcx[(size_t)t * ld + d + c]) * y);
}

// bf16, d % 8 == 0: a thread takes 8 neighbouring channels of one token with 16-byte loads.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__global__ void shortconv_fwd_vec_kernel(const bf16* __restrict__ bcx, const float* __restrict__ taps,
                                         const float* __restrict__ state, const int* __restrict__ slot_of_row,
                                         const int* __restrict__ row_of_token, const int* __restrict__ cu_q,
                                         bf16* __restrict__ out, int n_tokens, int d, int K, Bounds bounds) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int t = blockIdx.x;
    if (c >= d) return;
    const int r = row_of_token[t];
    if (!check_row(bounds, r) || !check_slot(bounds, slot_of_row[r])) return;
    const int i = t - cu_q[r];
    const size_t ld = (size_t)3 * d;
    const float* st = state + slot_elem(slot_of_row[r], (size_t)(K - 1) * d);
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = 0.f;
    for (int j = 0; j < K; ++j) {
        const int back = (K - 1) - j;
        float u[8];
        if (i - back >= 0) {
            const bf16* p = bcx + (size_t)(t - back) * ld;
            float b[8], x[8];
            unpack8(*reinterpret_cast<const uint4*>(p + c), b);
            unpack8(*reinterpret_cast<const uint4*>(p + 2 * d + c), x);
#pragma unroll
            for (int e = 0; e < 8; ++e) u[e] = b[e] * x[e];
        } else {
            const float* sp = st + (size_t)((K - 1) + (i - back)) * d + c;
            const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
            u[0] = s0.x; u[1] = s0.y; u[2] = s0.z; u[3] = s0.w; u[4] = s1.x; u[5] = s1.y; u[6] = s1.z; u[7] = s1.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fmaf(taps[(size_t)(c + e) * K + j], u[e], y[e]);
    }
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(bcx + (size_t)t * ld + d + c), g);
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 v = __floats2bfloat162_rn(g[2 * e] * y[2 * e], g[2 * e + 1] * y[2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * d + c) = make_uint4(w[0], w[1], w[2], w[3]);
}

// bf16, d % 8 == 0, K known at compile time: a thread takes 8 neighbouring channels of RUN
// consecutive tokens, keeps the last K-1 values of u in registers while it walks them, and so
// reads B, C and x of every token once (the kernel above reads B and x K times).  The history is
// rebuilt where a run starts and where a new request's portion starts inside it.  The taps are
// applied in the same ascending order, so the result is the same to the bit.
template <int K, int RUN>
__global__ void __launch_bounds__(128)
shortconv_fwd_run_kernel(const bf16* __restrict__ bcx, const float* __restrict__ taps,
                         const float* __restrict__ state, const int* __restrict__ slot_of_row,
                         const int* __restrict__ row_of_token, const int* __restrict__ cu_q,
                         bf16* __restrict__ out, int n_tokens, int d, Bounds bounds) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int t0 = blockIdx.x * RUN;
    pdl_wait();
    pdl_launch_dependents();
    if (c >= d) return;
    const size_t ld = (size_t)3 * d;
    float tap[K][8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int j = 0; j < K; ++j) tap[j][e] = taps[(size_t)(c + e) * K + j];
    float hist[K - 1][8];                              // u of the K-1 tokens before the current one, oldest first
    const int t1 = min(n_tokens, t0 + RUN);
    // the loads of the run's tokens are independent of one another: issue them four tokens at a time
    for (int tb = t0; tb < t1; tb += 4) {
        uint4 vb[4], vc[4], vx[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (tb + q < t1) {
                const bf16* p = bcx + (size_t)(tb + q) * ld + c;
                vb[q] = ld_act_u4(p);
                vc[q] = ld_act_u4(p + d);
                vx[q] = ld_act_u4(p + 2 * d);
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int t = tb + q;
            if (t >= t1) break;
            const int r = ld_act(row_of_token + t);
            if (!check_row(bounds, r) || !check_slot(bounds, ld_act(slot_of_row + r))) return;
            const int i = t - ld_act(cu_q + r);
            if (t == t0 || i == 0) {
                const float* st = state + slot_elem(ld_act(slot_of_row + r), (size_t)(K - 1) * d);
#pragma unroll
                for (int j = 0; j < K - 1; ++j) {
                    const int back = (K - 1) - j;
                    if (i - back >= 0) {
                        const bf16* p = bcx + (size_t)(t - back) * ld + c;
                        float b[8], x[8];
                        unpack8(ld_act_u4(p), b);
                        unpack8(ld_act_u4(p + 2 * d), x);
#pragma unroll
                        for (int e = 0; e < 8; ++e) hist[j][e] = b[e] * x[e];
                    } else {
                        const float* sp = st + (size_t)((K - 1) + (i - back)) * d + c;
                        const float4 s0 = __ldcg(reinterpret_cast<const float4*>(sp)), s1 = __ldcg(reinterpret_cast<const float4*>(sp + 4));
                        hist[j][0] = s0.x; hist[j][1] = s0.y; hist[j][2] = s0.z; hist[j][3] = s0.w;
                        hist[j][4] = s1.x; hist[j][5] = s1.y; hist[j][6] = s1.z; hist[j][7] = s1.w;
                    }
                }
            }
            float b[8], g[8], x[8], y[8];
            unpack8(vb[q], b); unpack8(vc[q], g); unpack8(vx[q], x);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float u = b[e] * x[e];
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < K - 1; ++j) acc = fmaf(tap[j][e], hist[j][e], acc);
                y[e] = fmaf(tap[K - 1][e], u, acc);
#pragma unroll
                for (int j = 0; j + 1 < K - 1; ++j) hist[j][e] = hist[j + 1][e];
                hist[K - 2][e] = u;
            }
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 v = __floats2bfloat162_rn(g[2 * e] * y[2 * e], g[2 * e + 1] * y[2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(out + (size_t)t * d + c) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// New state entry s (0 = oldest) is u at portion index n-(K-1)+s; if that is
// negative it is the old entry s+n.  Ascending s reads old entries before they
// are overwritten, since s+n > s.
template <typename T>
__global__ void shortconv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                       const int* __restrict__ slot_of_row, const int* __restrict__ cu_q,
                                       int d, int K, Bounds bounds) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int r = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();                     // the product that follows may set itself up meanwhile
    if (c >= d) return;
    const int q0 = ld_act(cu_q + r), n = ld_act(cu_q + r + 1) - q0;
    if (n <= 0) return;
    const size_t ld = (size_t)3 * d;
    if (!check_slot(bounds, ld_act(slot_of_row + r))) return;
    float* st = state + slot_elem(ld_act(slot_of_row + r), (size_t)(K - 1) * d);
    for (int s = 0; s < K - 1; ++s) {
        const int i = n - (K - 1) + s;
        float u;
        if (i >= 0) {
            const T* p = bcx + (size_t)(q0 + i) * ld;
            u = ld_act(p + c) * ld_act(p + 2 * d + c);
        } else {
            u = ld_act(st + (size_t)(s + n) * d + c);
        }
        st[(size_t)s * d + c] = u;
    }
}

// Every row brings exactly one token (decode): one thread per (row, channel) reads the state,
// computes the output and rolls the state, so one launch does both steps.
template <typename T>
__global__ void shortconv_single_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                        float* __restrict__ state, const int* __restrict__ slot_of_row,
                                        T* __restrict__ out, int d, int K, Bounds bounds) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int r = blockIdx.x;                       // row r's token is token r
    pdl_wait();
    pdl_launch_dependents();
    if (c >= d) return;
    const T* p = bcx + (size_t)r * 3 * d;
    const float u = ld_act(p + c) * ld_act(p + 2 * d + c);
    if (!check_slot(bounds, ld_act(slot_of_row + r))) return;
    float* st = state + slot_elem(ld_act(slot_of_row + r), (size_t)(K - 1) * d);
    float y = 0.f;
    for (int j = 0; j < K - 1; ++j) {
        const float s = ld_act(st + (size_t)j * d + c);
        y = fmaf(taps[(size_t)c * K + j], s, y);
        if (j > 0) st[(size_t)(j - 1) * d + c] = s;
    }
    y = fmaf(taps[(size_t)c * K + K - 1], u, y);
    st[(size_t)(K - 2) * d + c] = u;
    out[(size_t)r * d + c] = from_f32<T>(ld_act(p + d + c) * y);
}
}  // namespace

// bcx [n_tokens, 3d], taps [d, K] fp32, state [n_slots, K-1, d] fp32, out [n_tokens, d].
extern "C" int tuff_shortconv(const void* bcx, void* out, int dtype, const float* taps, float* state,
                              const int* slot_of_row, const int* row_of_token, const int* cu_q,
                              int n_tokens, int n_rows, int d, int K, int all_single, long long n_slots, int* status,
                              cudaStream_t stream) {
    if (n_tokens <= 0 || n_rows <= 0) return 0;
    if (K < 2) return TUFF_E_SIZE;
    const Bounds bounds{n_rows, n_slots, status};        // read by a checked build only
    const int threads = 128;
    if (all_single && n_tokens == n_rows) {
        dim3 g(n_rows, ceil_div(d, threads));
        if (dtype == TUFF_F32)
            return launch_pdl(shortconv_single_kernel<float>, g, dim3(threads), 0, stream, (const float*)bcx, taps, state, slot_of_row, (float*)out, d, K, bounds);
        else if (dtype == TUFF_BF16)
            return launch_pdl(shortconv_single_kernel<bf16>, g, dim3(threads), 0, stream, (const bf16*)bcx, taps, state, slot_of_row, (bf16*)out, d, K, bounds);
        return TUFF_E_DTYPE;
    }
    dim3 g1(n_tokens, ceil_div(d, threads)), g2(n_rows, ceil_div(d, threads));
    if (dtype == TUFF_F32) {
        shortconv_fwd_kernel<float><<<g1, threads, 0, stream>>>((const float*)bcx, taps, state, slot_of_row,
                                                                 row_of_token, cu_q, (float*)out, n_tokens, d, K, bounds);
        shortconv_state_kernel<float><<<g2, threads, 0, stream>>>((const float*)bcx, state, slot_of_row, cu_q, d, K, bounds);
    } else if (dtype == TUFF_BF16) {
        const bool vec = d % 8 == 0 && !((uintptr_t)bcx & 15) && !((uintptr_t)out & 15) && !((uintptr_t)state & 15);
        constexpr int RUN = 8;
        const dim3 gr(ceil_div(n_tokens, RUN), ceil_div(d / 8, threads));
        if (vec && n_tokens >= 4 * RUN && K == 3)
            launch_pdl(shortconv_fwd_run_kernel<3, RUN>, gr, dim3(threads), 0, stream, (const bf16*)bcx, taps, (const float*)state, slot_of_row,
                       row_of_token, cu_q, (bf16*)out, n_tokens, d, bounds);
        else if (vec && n_tokens >= 4 * RUN && K == 2)
            launch_pdl(shortconv_fwd_run_kernel<2, RUN>, gr, dim3(threads), 0, stream, (const bf16*)bcx, taps, (const float*)state, slot_of_row,
                       row_of_token, cu_q, (bf16*)out, n_tokens, d, bounds);
        else if (vec && n_tokens >= 4 * RUN && K == 4)
            launch_pdl(shortconv_fwd_run_kernel<4, RUN>, gr, dim3(threads), 0, stream, (const bf16*)bcx, taps, (const float*)state, slot_of_row,
                       row_of_token, cu_q, (bf16*)out, n_tokens, d, bounds);
        else if (vec)
            shortconv_fwd_vec_kernel<<<dim3(n_tokens, ceil_div(d / 8, threads)), threads, 0, stream>>>(
                (const bf16*)bcx, taps, state, slot_of_row, row_of_token, cu_q, (bf16*)out, n_tokens, d, K, bounds);
        else
            shortconv_fwd_kernel<bf16><<<g1, threads, 0, stream>>>((const bf16*)bcx, taps, state, slot_of_row,
                                                                    row_of_token, cu_q, (bf16*)out, n_tokens, d, K, bounds);
        launch_pdl(shortconv_state_kernel<bf16>, g2, dim3(threads), 0, stream, (const bf16*)bcx, state, slot_of_row, cu_q, d, K, bounds);
    } else {
        return TUFF_E_DTYPE;
    }
    return launch_status();
}
