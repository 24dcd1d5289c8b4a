// bf16 matrix product on the Blackwell tensor cores:  C[M,N] (=|+=) A[M,K] * W[N,K]^T.
//
// Both operands are K-major ([rows, K] with K contiguous), which is how the
// activations and the checkpoints' [out, in] matrices lie in memory.  One CTA
// computes a 128 x BN tile: a producer thread streams 128x64 and BNx64 bf16
// tiles into a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte
// swizzle), one thread issues tcgen05.mma (M=128, N=BN, K=16, fp32 accumulation in
// tensor memory), and four warps read the accumulator back with tcgen05.ld and
// write the result.  No cluster multicast is used anywhere.
//
// Which operand is the 128-row side is the launcher's choice:
//   many tokens (prefill)   rows of A (tokens) x BN rows of W
//   few tokens (decode)     rows of W (outputs) x BN >= tokens ("swapped"): the
//                           weights stream through the 128-row side once, and the
//                           K range is split over blockIdx.z so that all SMs pull on
//                           HBM.  Partial sums go to a workspace and are added in a
//                           fixed order by a second kernel, so the result does not
//                           depend on timing.
// The reference computes these products with per-row matrix-vector kernels on
// quantised weights (src/lfm25_gpu.cu:148-202, 860-934); accumulation into the
// residual is its accum=true (src/lfm25_engine.c:380,405,419).
//
// Every wait on an mbarrier is bounded: if it runs out, the kernel records a code
// in *status, lets its copies in flight land, frees its tensor memory and returns.
#include "sm100.cuh"
#include <algorithm>

namespace {

constexpr int BM = 128;            // rows of the 128-row operand per CTA (UMMA M)
constexpr int BK = 64;             // K elements per stage: 128 bytes of bf16, one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;   // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..5: epilogue

enum : int { OUT_STORE = 0, OUT_ACCUM = 1, OUT_PARTIAL = 2, OUT_SWIGLU = 3 };

struct GemmParams {
    void* out;            // [rows_of_tokens, ld] bf16 or fp32
    float* partial;       // [splits, rows_of_tokens, n_out] fp32 (OUT_PARTIAL)
    int* status;
    long long ld;         // row stride of out, in elements
    int a_rows, b_rows;   // rows of the 128-row operand and of the BN-row operand
    int k_blocks;         // ceil(K / 64)
    int kb_per_split;
    int mode;             // OUT_*
    int out_dtype;        // TUFF_F32 / TUFF_BF16
    int swapped;          // 1: the 128-row operand is W, so D is [out, token]
    int splits;           // parts the K range is cut into
};

// Instruction descriptor: fp32 accumulator, bf16 x bf16, both K-major, M=128, N=BN.
template <int BN> __device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Two accumulators of BN columns each, so that one is read out while the other is filled.
template <int BN> constexpr int tmem_cols() { return 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512; }

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int TILES = STAGES * (A_BYTES + B_BYTES);
    static constexpr int BARS = TILES;                       // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    static constexpr int TMEM_SLOT = BARS + (2 * STAGES + 4) * 8;
    static constexpr int OUT_STAGE = TMEM_SLOT + 16;         // 4 epilogue warps x 2 KB, 16-byte aligned
    static constexpr int TOTAL = OUT_STAGE + 4 * 2048 + 1024;   // + room to align the base to 1024 bytes
};

// Writes 16 consecutive accumulator columns of one row: `row`/`col` index the 128-row and the
// BN-row operand.  Not swapped: the 16 values are consecutive in the output row (vector stores
// when aligned); swapped: they belong to 16 different tokens, and the warp's lanes hold
// consecutive outputs, so each store of the warp is one contiguous run.
__device__ __forceinline__ void store16(const GemmParams& p, int split, int row, int col0, const uint32_t (&r)[16]) {
    const int n_out = p.swapped ? p.a_rows : p.b_rows;
    const int n_tok = p.swapped ? p.b_rows : p.a_rows;
    const int n_valid = min(16, p.b_rows - col0);
    if (!p.swapped) {
        if (p.mode == OUT_PARTIAL) {
            float* dst = p.partial + ((size_t)split * n_tok + row) * n_out + col0;
#pragma unroll
            for (int j = 0; j < 16; ++j) if (j < n_valid) dst[j] = __uint_as_float(r[j]);
            return;
        }
        const size_t idx = (size_t)row * p.ld + col0;
        if (p.out_dtype == TUFF_BF16) {
            bf16* dst = (bf16*)p.out + idx;
            if (n_valid == 16 && (((uintptr_t)dst) & 15) == 0) {
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                    w[j] = *reinterpret_cast<uint32_t*>(&v);
                }
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) if (j < n_valid) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
        } else {
            float* dst = (float*)p.out + idx;
            if (n_valid == 16 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    if (p.mode == OUT_ACCUM) {
                        const float4 o = reinterpret_cast<float4*>(dst)[j];
                        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    }
                    reinterpret_cast<float4*>(dst)[j] = v;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) if (j < n_valid) dst[j] = (p.mode == OUT_ACCUM ? dst[j] : 0.f) + __uint_as_float(r[j]);
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (j >= n_valid) break;
        const int tok = col0 + j;
        const float v = __uint_as_float(r[j]);
        if (p.mode == OUT_PARTIAL) {
            p.partial[((size_t)split * n_tok + tok) * n_out + row] = v;
        } else {
            const size_t idx = (size_t)tok * p.ld + row;
            if (p.out_dtype == TUFF_F32) {
                float* op = (float*)p.out + idx;
                *op = p.mode == OUT_ACCUM ? *op + v : v;
            } else {
                ((bf16*)p.out)[idx] = __float2bfloat16_rn(v);
            }
        }
    }
}

// The same 16 columns of 32 rows (one epilogue warp's rows), written so that every store of the warp
// covers whole 32-byte sectors: the warp's values go through a 2 KB staging tile in shared memory
// (16-byte slots XOR-swizzled by the row so that neither side has bank conflicts), and come back
// with four lanes per row (fp32) or two lanes per row (bf16).  Only for a full, aligned chunk of
// the unswapped form; every lane of the warp must call it.
// Residual values (fp32 out, OUT_ACCUM) that store16_rows will add for the chunk at col0: loaded
// ahead of time so that their latency is not paid chunk by chunk.
__device__ __forceinline__ void load_residual(const GemmParams& p, int row0, int col0, int lane, float4 (&o)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = (lane >> 2) + 8 * i;
        o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.mode == OUT_ACCUM && row0 + rr < p.a_rows)
            o[i] = __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)(row0 + rr) * p.ld + col0) + (lane & 3));
    }
}

__device__ __forceinline__ void store16_rows(const GemmParams& p, uint8_t* stage, int row0, int col0, int lane,
                                             const uint32_t (&r)[16], const float4 (&o)[4]) {
    if (p.out_dtype == TUFF_F32) {
        uint4* st = reinterpret_cast<uint4*>(stage);                    // [32 rows][4 slots]
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int q = 0; q < 4; ++q) st[lane * 4 + (q ^ sw)] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        __syncwarp();
        const int c4 = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = (lane >> 2) + 8 * i;
            const uint4 u = st[rr * 4 + (c4 ^ ((rr >> 1) & 3))];
            if (row0 + rr < p.a_rows)
                *(reinterpret_cast<float4*>((float*)p.out + (size_t)(row0 + rr) * p.ld + col0) + c4) =
                    make_float4(__uint_as_float(u.x) + o[i].x, __uint_as_float(u.y) + o[i].y,
                                __uint_as_float(u.z) + o[i].z, __uint_as_float(u.w) + o[i].w);
        }
    } else {
        uint4* st = reinterpret_cast<uint4*>(stage);                    // [32 rows][2 slots]
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            w[j] = *reinterpret_cast<uint32_t*>(&v);
        }
        const int sw = (lane >> 2) & 1;
        st[lane * 2 + (0 ^ sw)] = make_uint4(w[0], w[1], w[2], w[3]);
        st[lane * 2 + (1 ^ sw)] = make_uint4(w[4], w[5], w[6], w[7]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int rr = (lane >> 1) + 16 * i, h = lane & 1;
            const uint4 u = st[rr * 2 + (h ^ ((rr >> 2) & 1))];
            if (row0 + rr < p.a_rows)
                *(reinterpret_cast<uint4*>((bf16*)p.out + (size_t)(row0 + rr) * p.ld + col0) + h) = u;
        }
    }
    __syncwarp();
}

// One epilogue warp's part of a finished tile: the 32 accumulator rows of TMEM lane quarter
// `quad`, all BN columns, read with tcgen05.ld from `taddr` and written as the mode says.  `m0` is
// the first row of this CTA's 128 rows, `stage` the warp's 2 KB staging tile.
template <int BN>
__device__ __forceinline__ void write_tile(const GemmParams& p, uint8_t* stage, uint32_t taddr, int m0, int n0, int split,
                                           int quad, int lane) {
    const int row = m0 + quad * 32 + lane;          // row of the 128-row operand
    if (BN == 256 && p.mode == OUT_SWIGLU) {
        // W is [gate block; up block] per 256 rows: columns c and c + 128 of the accumulator
        // are gate and up of output column n0/2 + c.  Both are rounded to bf16 first, as a
        // separate projection would store them.
        bf16* orow = (bf16*)p.out + (size_t)row * p.ld + (n0 >> 1);
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 16) {
            uint32_t gq[16], uq[16];
            tmem_ld16(taddr + (uint32_t)c0, gq);
            tmem_ld16(taddr + (uint32_t)(c0 + 128), uq);
            if (row < p.a_rows) {
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gq[2 * j])));
                    float a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gq[2 * j + 1])));
                    const float u0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uq[2 * j])));
                    const float u1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uq[2 * j + 1])));
                    a0 = a0 / (1.f + expf(-a0)) * u0;
                    a1 = a1 / (1.f + expf(-a1)) * u1;
                    __nv_bfloat162 v = __floats2bfloat162_rn(a0, a1);
                    w[j] = *reinterpret_cast<uint32_t*>(&v);
                }
                reinterpret_cast<uint4*>(orow + c0)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(orow + c0)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
    } else {
        // whole, aligned chunks of the unswapped form go out as full sectors through shared memory
        const int esz = p.out_dtype == TUFF_F32 ? 4 : 2;
        const bool rows_ok = !p.swapped && p.mode != OUT_PARTIAL && ((p.ld * esz) % 16 == 0) &&
                             ((((uintptr_t)p.out) + (size_t)n0 * esz) % 16 == 0);
        
        const bool resid = rows_ok && p.mode == OUT_ACCUM && p.out_dtype == TUFF_F32;
#pragma unroll 1
        for (int g0 = 0; g0 < BN; g0 += 64) {
            if (n0 + g0 >= p.b_rows) break;             // uniform over the warp
            // the residual values of up to four chunks, all in flight at once
            float4 o[4][4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int c0 = g0 + cc * 16;
                if (resid && c0 < BN && n0 + c0 + 16 <= p.b_rows) load_residual(p, m0 + quad * 32, n0 + c0, lane, o[cc]);
                else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[cc][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int c0 = g0 + cc * 16;
                if (c0 >= BN || n0 + c0 >= p.b_rows) break;
                uint32_t r[16];
                tmem_ld16(taddr + (uint32_t)c0, r);
                if (rows_ok && n0 + c0 + 16 <= p.b_rows) store16_rows(p, stage, m0 + quad * 32, n0 + c0, lane, r, o[cc]);
                else if (row < p.a_rows) store16(p, split, row, n0 + c0, r);
            }
        }
    }
}

// Persistent: each CTA walks the work items (128-row block, BN-row block, K split) that fall to
// it, blockIdx.x, blockIdx.x + gridDim.x, ...; the 128-row block index runs fastest, so CTAs that
// run together share the BN-row operand's tile in L2.
template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_tiles = base, b_tiles = base + STAGES * L::A_BYTES;
    const uint32_t bars = base + L::BARS;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::TMEM_SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = (p.a_rows + BM - 1) / BM, nt = (p.b_rows + BN - 1) / BN;
    const int n_work = mt * nt * p.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + (uint32_t)L::TMEM_SLOT), "r"((uint32_t)tmem_cols<BN>()) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    // Everything above touched nothing that another kernel writes: with programmatic dependent launch it
    // runs beside the tail of the kernel before.  From here on activations are read and outputs written.
    pdl_wait();
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                                  // k-block counter over all of this CTA's work
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
                const int m0 = (w % mt) * BM, n0 = ((w / mt) % nt) * BN, split = w / (mt * nt);
                const int kb0 = split * p.kb_per_split;
                const int nkb = min(p.kb_per_split, p.k_blocks - kb0);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, p.status, 1)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), L::A_BYTES + L::B_BYTES);
                    const int k = (kb0 + i) * BK;
                    tma_load_2d(a_tiles + s * L::A_BYTES, &map_a, full_bar(s), k, m0);
                    tma_load_2d(b_tiles + s * L::B_BYTES, &map_b, full_bar(s), k, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<BN>();
            uint32_t it = 0, tile = 0;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++tile) {
                const int split = w / (mt * nt);
                const int nkb = min(p.kb_per_split, p.k_blocks - split * p.kb_per_split);
                const uint32_t buf = tile & 1u;
                // the epilogue must have emptied this accumulator (two tiles ago)
                if (!mbar_wait(acc_empty(buf), ((tile >> 1) & 1u) ^ 1u, p.status, 4)) { ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * BN;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, p.status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a = a_tiles + s * L::A_BYTES, b = b_tiles + s * L::B_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(acc, smem_desc_k_major(a + k * UMMA_K * 2), smem_desc_k_major(b + k * UMMA_K * 2), idesc,
                             (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));      // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full(buf)); // the accumulator is complete once all MMAs retire
            }
        }
    } else {
        const int quad = warp & 3;                          // the 32 tensor-memory lanes this warp may read
        uint32_t tile = 0;
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++tile) {
            const int m0 = (w % mt) * BM, n0 = ((w / mt) % nt) * BN, split = w / (mt * nt);
            const uint32_t buf = tile & 1u;
            if (!mbar_wait(acc_full(buf), (tile >> 1) & 1u, p.status, 3)) { ok = false; break; }
            tc_fence_after();
            write_tile<BN>(p, base_ptr + L::OUT_STAGE + (warp - 2) * 2048, tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN,
                           m0, n0, split, quad, lane);
            // this warp has read its part of the accumulator: hand it back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
        }
    }
    if (!ok) {
        // A wait ran out.  Give copies that may still be in flight time to land before the
        // shared memory is released.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)tmem_cols<BN>()) : "memory");
    }
}

// Adds the split-K partial sums in split order and writes them out.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, long long ld,
                                     int n_tok, int n_out, int splits, int mode, int out_dtype) {
    const size_t total = (size_t)n_tok * n_out;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * total + i];
        const size_t t = i / n_out, o = i - t * n_out;
        const size_t idx = t * ld + o;
        if (out_dtype == TUFF_F32) {
            float* op = (float*)out + idx;
            *op = mode == OUT_ACCUM ? *op + acc : acc;
        } else {
            ((bf16*)out)[idx] = __float2bfloat16_rn(acc);
        }
    }
}

// ------------------------------------------------------------------ host side
template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int rc = launch_pdl(gemm_tc_kernel<BN, STAGES>, grid, dim3(NUM_THREADS), L::TOTAL, stream, ma, mb, p);
    return rc ? rc : launch_status();
}

}  // namespace

// Bytes of workspace that tuff_gemm_tc may need for a product with this many tokens and outputs.
extern "C" long long tuff_gemm_tc_workspace_bytes(int m_tokens, int n_out, int k) {
    if (m_tokens > 128) return 0;
    const int kb = (k + BK - 1) / BK;
    const int splits = kb < 16 ? kb : 16;
    return (long long)splits * m_tokens * n_out * 4;
}

// C[M,N] (=|+=) A[M,K] W[N,K]^T with bf16 A and W.  C is bf16 (store only) or fp32.
// Requirements: K % 8 == 0, lda % 8 == 0, ldw % 8 == 0, A and W 16-byte aligned (TMA strides).
// `workspace` (fp32) is used when the K range is split; `status` is a device int that
// receives a non-zero code if a bounded wait ran out.
// accumulate == 2: W is [2F, K] laid out as blocks of 128 gate rows followed by their 128 up rows
// (N = 2F, a multiple of 256), and C [M, F] (bf16, ldc % 8 == 0, 16-byte aligned) receives
// silu(gate) * up; only for M > 128.
extern "C" int tuff_gemm_tc(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K,
                            long long lda, long long ldw, long long ldc, int accumulate,
                            float* workspace, long long workspace_bytes, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return TUFF_E_SIZE;
    const bool swiglu = accumulate == 2;
    if (swiglu) {
        if (M <= 128 || (N % 256) || c_dtype != TUFF_BF16) return TUFF_E_SIZE;
        if ((ldc % 8) || ((uintptr_t)C & 15)) return TUFF_E_ALIGN;
        accumulate = 0;
    }
    if (accumulate && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TUFF_E_ALIGN;
    const int k_blocks = ceil_div(K, BK);
    const bool swapped = M <= 128;
    const int sms = sm_count();
    GemmParams p{};
    p.out = C; p.partial = workspace; p.status = status; p.ld = ldc; p.k_blocks = k_blocks;
    p.out_dtype = c_dtype; p.swapped = swapped ? 1 : 0;
    p.mode = swiglu ? OUT_SWIGLU : accumulate ? OUT_ACCUM : OUT_STORE;
    CUtensorMap ma, mb;
    int bn, splits = 1;
    if (swapped) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        p.a_rows = N; p.b_rows = M;
        const int tiles = ceil_div(N, BM);
        if (tiles < sms && k_blocks > 1) {
            splits = sms / tiles > 0 ? sms / tiles : 1;     // one wave of work items: fewer, larger items
            if (splits > 16) splits = 16;
            if (splits > k_blocks) splits = k_blocks;
            const long long need = (long long)splits * M * N * 4;
            if (!workspace || need > workspace_bytes) splits = 1;
        }
        if (!tensor_map(&ma, W, N, K, ldw, BM) || !tensor_map(&mb, A, M, K, lda, bn)) return TUFF_E_ALIGN;
    } else {
        bn = N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : 256;     // swiglu: N % 256 == 0, so 256
        // Few tiles (a few hundred tokens against a narrow matrix) leave SMs idle and make every CTA walk a
        // whole K range for one wide tile: narrower tiles put more SMs to work on shorter K loops.  Measured
        // at 544 x 2,048 x 2,048: 30.7 us with 128 x 256 tiles (40 of them), 22.5 us with 128 x 128.
        if (bn == 256 && !swiglu) {
            const int rows = ceil_div(M, BM);
            if (rows * ceil_div(N, 256) <= sms / 2) bn = 128;
            else if (ceil_div(rows * ceil_div(N, 192), sms) * 192 < ceil_div(rows * ceil_div(N, 256), sms) * 256) bn = 192;
            // 192-wide tiles when they fill the rounds of the SMs better: 2,048 x 3,072 takes two rounds either
            // way (192 tiles of 256 columns, 256 of 192), and two rounds of narrower tiles are shorter
        }
        p.a_rows = M; p.b_rows = N;
        if (!tensor_map(&ma, A, M, K, lda, BM) || !tensor_map(&mb, W, N, K, ldw, bn)) return TUFF_E_ALIGN;
    }
    p.kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, p.kb_per_split);
    const int user_mode = p.mode;
    if (splits > 1) p.mode = OUT_PARTIAL;
    p.splits = splits;
    const int n_work = ceil_div(p.a_rows, BM) * ceil_div(p.b_rows, bn) * splits;
    dim3 grid(n_work < sms ? n_work : sms);
    int rc;
    switch (bn) {
        case 16: rc = launch<16, 8>(ma, mb, p, grid, stream); break;
        case 32: rc = launch<32, 8>(ma, mb, p, grid, stream); break;
        case 64: rc = launch<64, 6>(ma, mb, p, grid, stream); break;
        case 128: rc = launch<128, 5>(ma, mb, p, grid, stream); break;
        case 192: rc = launch<192, 5>(ma, mb, p, grid, stream); break;
        default: rc = launch<256, 4>(ma, mb, p, grid, stream); break;
    }
    if (rc != 0 || splits == 1) return rc;
    const size_t total = (size_t)M * N;
    const int threads = 256;
    const int blocks = (int)std::min((total + threads - 1) / threads, (size_t)sms * 8);
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(workspace, C, ldc, M, N, splits, user_mode, c_dtype);
    return launch_status();
}
