// The decode-step matrix products: C[M,N] = A[M,K] * W[N,K]^T for M <= 16 tokens, with what
// surrounds them in a layer fused in, so that a layer is a few launches instead of a dozen.
//
// With so few tokens a product is a stream of W through the SMs; its time is the bytes of W
// over the HBM bandwidth plus what it costs to start and stop a kernel.  So each kernel here
//   * keeps many 16-byte weight loads in flight per lane all the time (a CTA of 8 warps splits K
//     eight ways; a warp streams its share of a few groups of 8 rows straight into the operand
//     registers of mma.sync.m16n8k16, tokens on the 16-row side; CTAs are persistent and the
//     loads of the next blocks, also of the next work item, are issued before a block is used),
//   * does the neighbouring small operations itself:
//       prologue  RMSNorm of the fp32 residual rows (each CTA norms the M rows it needs into
//                 shared memory: reference src/lfm25_gpu.cu:207-262),
//       epilogue  plain store / add into the fp32 residual (reference accum=true,
//                 src/lfm25_engine.c:380,405,419) / silu(gate)*up over a stacked [gate; up]
//                 matrix (src/lfm25_gpu.cu:583-618) / the gated short convolution over a
//                 stacked [B; C; x] projection with the state roll (src/lfm25_gpu.cu:344-415,
//                 which fuses the same way for one token).
// The warps' partial sums are added in warp order through shared memory, so results do not
// depend on timing.  Inside a 32-wide K step the k order is permuted identically for both
// operands (a lane's 16 bytes are 8 consecutive k), which leaves dot products unchanged.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int KSTEP = 32;
constexpr int NORM_BLOCKS = 2;     // the fused RMSNorm holds rows of up to NORM_BLOCKS * 1024 columns in registers

enum : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_CONV = 3 };

struct DecodeGemm {
    const void* a;            // activations: bf16 [M, K] (lda), or fp32 residual [M, K] when norm_w is set
    const float* norm_w;      // RMSNorm weight [K] or null
    const bf16* w;            // [rows, K] (ldw)
    void* out;                // [M, ldc]
    long long lda, ldw, ldc;
    int M, N, K;              // N: output columns (for swiglu the width F, for conv the channels d)
    int set_block;            // rows of one set that lie together in W: N (sets stacked whole) or a block size
    float eps;
    // convolution epilogue
    const float* taps;        // [d, L]
    float* state;             // [slots, L-1, d]
    const int* slot_of_row;
    int L;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// A CTA is persistent: it takes work items blockIdx.x, blockIdx.x + gridDim.x, ...  An item is GPS
// groups of 8 output columns, i.e. NG = GPS * SETS groups of 8 weight rows (SETS = 1 for a plain
// product, 2 for [gate; up], 3 for [B; C; x]), over all of K.  Each warp owns a fixed share of K
// (`per` steps of 32) and walks it in blocks of D steps.  The loads of the next B blocks, across item
// boundaries, are always in flight in a ring of registers: a block is refilled as soon as it has
// been used, before the item's partial sums are added up, so the stream from HBM never drains.
template <int NG, int D, bool HI, bool NORM, int EPI, typename CT>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_decode_kernel(DecodeGemm p) {
    constexpr int B = 2;                                                      // blocks in flight per lane
    constexpr int SETS = EPI == EPI_SWIGLU ? 2 : EPI == EPI_CONV ? 3 : 1;     // row sets that are combined
    constexpr int GPS = NG / SETS;                                            // groups per set
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);                       // [WARPS][NG][16][8]
    bf16* hs = reinterpret_cast<bf16*>(smem + WARPS * NG * 128 * 4);    // NORM: [M_pad][K + 8] bf16
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K;
    const int steps = (K + KSTEP - 1) / KSTEP;
    const int per = (steps + WARPS - 1) / WARPS;
    const int s_begin = warp * per, s_end = min(steps, s_begin + per);
    const int nblk = (per + D - 1) / D;                                       // the same for every warp
    const int n_items = (p.N + GPS * 8 - 1) / (GPS * 8);
    const int my_items = blockIdx.x < n_items ? (n_items - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total = my_items * nblk;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const bool lo_ok = g < p.M, hi_ok = HI && (g + 8 < p.M);
    const int hs_ld = K + 8;                                   // padded row of the normed activations

    pdl_wait();
    if (NORM) {
        // RMSNorm of the M residual rows into shared memory as bf16, once per CTA.  All 256 threads
        // share each row: a thread holds one float4 of every row of a half (8 rows) per 1024 columns,
        // so all of a half's loads are in flight at once and the values stay in registers.
        const float* x = reinterpret_cast<const float*>(p.a);
        float* part = red;                                       // [8 rows][WARPS] partial sums
        for (int r0 = 0; r0 < p.M; r0 += 8) {
            float4 v[NORM_BLOCKS][8];
            float ss[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) ss[r] = 0.f;
#pragma unroll
            for (int cb = 0; cb < NORM_BLOCKS; ++cb) {
                const int k = cb * 1024 + threadIdx.x * 4;
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    v[cb][r] = (k < K && r0 + r < p.M) ? __ldcg(reinterpret_cast<const float4*>(x + (size_t)(r0 + r) * p.lda + k))
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int cb = 0; cb < NORM_BLOCKS; ++cb)
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float4 a = v[cb][r];
                    ss[r] = fmaf(a.x, a.x, ss[r]); ss[r] = fmaf(a.y, a.y, ss[r]);
                    ss[r] = fmaf(a.z, a.z, ss[r]); ss[r] = fmaf(a.w, a.w, ss[r]);
                }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float w = warp_sum(ss[r]);
                if (lane == 0) part[r * WARPS + warp] = w;
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) tot += part[r * WARPS + w];
                ss[r] = rsqrtf(tot / (float)K + p.eps);
            }
            __syncthreads();
#pragma unroll
            for (int cb = 0; cb < NORM_BLOCKS; ++cb) {
                const int k = cb * 1024 + threadIdx.x * 4;
                if (k < K) {
                    const float4 wn = *reinterpret_cast<const float4*>(p.norm_w + k);
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        if (r0 + r >= p.M) break;
                        const float4 a = v[cb][r];
                        __nv_bfloat162 lo2 = __floats2bfloat162_rn(a.x * ss[r] * wn.x, a.y * ss[r] * wn.y);
                        __nv_bfloat162 hi2 = __floats2bfloat162_rn(a.z * ss[r] * wn.z, a.w * ss[r] * wn.w);
                        *reinterpret_cast<uint2*>(hs + (size_t)(r0 + r) * hs_ld + k) =
                            make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
                    }
                }
            }
        }
        __syncthreads();
    }

    uint4 wr[B][D][NG];                       // the ring: weights of the next B blocks
    uint4 xr[B][D][HI ? 2 : 1];               // and, when the activations come from global memory, theirs
    const bf16* a_lo = reinterpret_cast<const bf16*>(p.a) + (size_t)(lo_ok ? g : 0) * p.lda;
    const bf16* a_hi = reinterpret_cast<const bf16*>(p.a) + (size_t)(hi_ok ? g + 8 : 0) * p.lda;

    // issues the loads of block `jj` of this warp's sequence into ring slot `bb`
    auto fetch = [&](int jj, int bb) {
        const bool live = jj < total;
        const int it = live ? jj / nblk : 0, blk = live ? jj - it * nblk : 0;
        const int n0 = (blockIdx.x + it * gridDim.x) * GPS * 8;
#pragma unroll
        for (int i = 0; i < NG; ++i) {
            const int col = n0 + (i % GPS) * 8 + g;
            const bool cok = live && col < p.N;
            // set s of output column c is row (c / sb) * sb * SETS + s * sb + c % sb of W
            const int sb = p.set_block;
            const int wr_row = SETS == 1 ? col : (col / sb) * sb * SETS + (i / GPS) * sb + col % sb;
            const bf16* wrow = p.w + (size_t)(cok ? wr_row : 0) * p.ldw;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const int s = s_begin + blk * D + d;
                const int k = s * KSTEP + t * 8;
                wr[bb][d][i] = (cok && s < s_end && k < K) ? ldg_stream(wrow + k) : zero;   // K % 8 == 0
            }
        }
        if (!NORM) {
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const int s = s_begin + blk * D + d;
                const int k = s * KSTEP + t * 8;
                const bool ok = live && s < s_end && k < K;
                xr[bb][d][0] = (ok && lo_ok) ? ld_act_u4(a_lo + k) : zero;
                if (HI) xr[bb][d][HI ? 1 : 0] = (ok && hi_ok) ? ld_act_u4(a_hi + k) : zero;
            }
        }
    };

    float acc[NG][4];
#pragma unroll
    for (int i = 0; i < NG; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
    for (int bb = 0; bb < B; ++bb) fetch(bb, bb);

#pragma unroll 1
    for (int j0 = 0; j0 < total; j0 += B) {
#pragma unroll
        for (int bb = 0; bb < B; ++bb) {
            const int jj = j0 + bb;
            if (jj >= total) break;                              // the same for every thread of the CTA
            const int it = jj / nblk, blk = jj - it * nblk;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                uint4 xa = zero, xb = zero;
                if (NORM) {
                    const int s = s_begin + blk * D + d;
                    const int k = s * KSTEP + t * 8;
                    const bool ok = s < s_end && k < K;
                    if (lo_ok && ok) xa = *reinterpret_cast<const uint4*>(hs + (size_t)g * hs_ld + k);
                    if (hi_ok && ok) xb = *reinterpret_cast<const uint4*>(hs + (size_t)(g + 8) * hs_ld + k);
                } else {
                    xa = xr[bb][d][0];
                    if (HI) xb = xr[bb][d][HI ? 1 : 0];
                }
#pragma unroll
                for (int i = 0; i < NG; ++i) {
                    mma16816(acc[i], xa.x, xb.x, xa.y, xb.y, wr[bb][d][i].x, wr[bb][d][i].y);
                    mma16816(acc[i], xa.z, xb.z, xa.w, xb.w, wr[bb][d][i].z, wr[bb][d][i].w);
                }
            }
            fetch(jj + B, bb);                                   // refill the slot at once
            if (blk != nblk - 1) continue;
            // ---- the item is complete: add the warps' partial tiles in warp order and write out
            // acc[i][0..1]: token g, columns 2t, 2t+1 of group i; acc[i][2..3]: token g + 8
#pragma unroll
            for (int i = 0; i < NG; ++i) {
                float* r = red + ((size_t)(warp * NG + i) * 16) * 8;
                r[g * 8 + 2 * t] = acc[i][0];
                r[g * 8 + 2 * t + 1] = acc[i][1];
                r[(g + 8) * 8 + 2 * t] = acc[i][2];
                r[(g + 8) * 8 + 2 * t + 1] = acc[i][3];
                acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            }
            __syncthreads();
            const int n0 = (blockIdx.x + it * gridDim.x) * GPS * 8;
            for (int idx = threadIdx.x; idx < GPS * 128; idx += WARPS * 32) {
                const int grp = idx >> 7, tok = (idx >> 3) & 15, c = idx & 7;
                const int col = n0 + grp * 8 + c;
                if (tok >= p.M || col >= p.N) continue;
                float v[SETS];
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    float a = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) a += red[((size_t)(w * NG + s * GPS + grp) * 16 + tok) * 8 + c];
                    v[s] = a;
                }
                CT* op = reinterpret_cast<CT*>(p.out) + (size_t)tok * p.ldc + col;
                if (EPI == EPI_STORE) {
                    *op = from_f32<CT>(v[0]);
                } else if (EPI == EPI_ACCUM) {
                    *op = from_f32<CT>(ld_act(op) + v[0]);
                } else if (EPI == EPI_SWIGLU) {
                    // gate and up rounded to bf16 first, as a separate projection would store them
                    const float gq = bf16_round(v[0]), uq = bf16_round(v[SETS > 1 ? 1 : 0]);
                    *op = from_f32<CT>(gq / (1.f + expf(-gq)) * uq);
                } else {
                    // gated short convolution of one token per row; this CTA alone owns these channels
                    const float b = bf16_round(v[0]), cg = bf16_round(v[SETS > 1 ? 1 : 0]), xg = bf16_round(v[SETS > 2 ? 2 : 0]);
                    const float u = b * xg;
                    const int L = p.L, d = p.N;
                    float* st = p.state + (size_t)ld_act(p.slot_of_row + tok) * (L - 1) * d;
                    float y = 0.f;
                    for (int j = 0; j < L - 1; ++j) {
                        const float sv = ld_act(st + (size_t)j * d + col);
                        y = fmaf(p.taps[(size_t)col * L + j], sv, y);
                        if (j > 0) st[(size_t)(j - 1) * d + col] = sv;
                    }
                    y = fmaf(p.taps[(size_t)col * L + L - 1], u, y);
                    st[(size_t)(L - 2) * d + col] = u;
                    *op = from_f32<CT>(cg * y);
                }
            }
            __syncthreads();                                     // `red` is reused by the next item
        }
    }
    pdl_launch_dependents();
}

template <int NG, int D, bool NORM, int EPI, typename CT>
int launch(const DecodeGemm& p, cudaStream_t stream) {
    constexpr int SETS = EPI == EPI_SWIGLU ? 2 : EPI == EPI_CONV ? 3 : 1;
    constexpr int GPS = NG / SETS;
    const int m_pad = p.M > 8 ? 16 : 8;
    size_t smem = (size_t)WARPS * NG * 128 * 4 + (NORM ? (size_t)m_pad * (p.K + 8) * 2 : 0);
    // as many CTAs as stay resident (two per SM), each with the same number of items
    const int n_items = ceil_div(p.N, GPS * 8);
    const int rounds = ceil_div(n_items, 2 * 148);
    dim3 grid(ceil_div(n_items, rounds));
    if (p.M > 8) {
        auto k = gemm_decode_kernel<NG, D, true, NORM, EPI, CT>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(k, grid, dim3(WARPS * 32), smem, stream, p);
    }
    auto k = gemm_decode_kernel<NG, D, false, NORM, EPI, CT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(k, grid, dim3(WARPS * 32), smem, stream, p);
}

}  // namespace

// epilogue: 0 store, 1 add into fp32 C, 2 swiglu (W is [2N, K]: gate rows then up rows), 3 gated
// short convolution (W is [3N, K]: B, C, x rows; one token per row of A; taps [N, L], state
// [slots, L-1, N], slot_of_row [M]).  norm_w: if not null, A is the fp32 residual [M, K] and is
// RMS-normed with this weight and eps first; else A is bf16 [M, K].
// Requirements: M <= 16, K % 8 == 0, ldw % 8 == 0, 16-byte aligned bases; bf16 A: lda % 8 == 0;
// fp32 A: lda % 4 == 0.  C is bf16 or fp32 (fp32 only for epilogue 1).
// set_block: for epilogues 2 and 3, how the row sets lie in W: 0 = stacked whole ([gate; up]), else
// blocks of that many rows of each set in turn (a multiple of 8).
extern "C" int tuff_gemm_decode(const void* A, const float* norm_w, float eps, const void* W, void* C, int c_dtype,
                                int M, int N, int K, long long lda, long long ldw, long long ldc, int epilogue,
                                const float* taps, float* state, const int* slot_of_row, int L, int set_block,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || epilogue < 0 || epilogue > 3) return TUFF_E_SIZE;
    if ((K % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TUFF_E_ALIGN;
    if (norm_w ? (lda % 4 != 0 || ((uintptr_t)norm_w & 15)) : (lda % 8 != 0)) return TUFF_E_ALIGN;
    if (epilogue == EPI_ACCUM && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if ((epilogue == EPI_SWIGLU || epilogue == EPI_CONV) && c_dtype != TUFF_BF16) return TUFF_E_DTYPE;
    if (epilogue == EPI_CONV && (L < 2 || !taps || !state || !slot_of_row)) return TUFF_E_SIZE;
    if (norm_w && K > NORM_BLOCKS * 1024) return TUFF_E_SIZE;      // a normed row must fit the prologue's registers
    DecodeGemm p{};
    p.a = A; p.norm_w = norm_w; p.w = (const bf16*)W; p.out = C; p.lda = lda; p.ldw = ldw; p.ldc = ldc;
    if (set_block < 0 || (set_block % 8)) return TUFF_E_SIZE;
    p.set_block = set_block ? set_block : N;
    p.M = M; p.N = N; p.K = K; p.eps = eps; p.taps = taps; p.state = state; p.slot_of_row = slot_of_row; p.L = L;
    const bool norm = norm_w != nullptr;
#define PICK(NGV, DV, EPI, CT) (norm ? launch<NGV, DV, true, EPI, CT>(p, stream) : launch<NGV, DV, false, EPI, CT>(p, stream))
    // two groups of 8 columns per item when that still leaves every resident CTA an item
    const bool wide = ceil_div(N, 16) >= 2 * 148;
    int rc;
    if (epilogue == EPI_SWIGLU) {
        rc = PICK(2, 4, EPI_SWIGLU, bf16);
    } else if (epilogue == EPI_CONV) {
        rc = PICK(3, 2, EPI_CONV, bf16);
    } else if (epilogue == EPI_ACCUM) {
        rc = wide ? PICK(2, 4, EPI_ACCUM, float) : PICK(1, 4, EPI_ACCUM, float);
    } else if (c_dtype == TUFF_BF16) {
        rc = wide ? PICK(2, 4, EPI_STORE, bf16) : PICK(1, 4, EPI_STORE, bf16);
    } else if (c_dtype == TUFF_F32) {
        rc = wide ? PICK(2, 4, EPI_STORE, float) : PICK(1, 4, EPI_STORE, float);
    } else {
        return TUFF_E_DTYPE;
    }
#undef PICK
    return rc ? rc : launch_status();
}
