// The matrix products of a step with 17 to 128 tokens (many requests decoding together, or a
// short portion of a prompt):  C[M,N] (=|+=) A[M,K] * W[N,K]^T, bf16 operands, fp32 accumulation.
//
// The weights are the only large operand, so they take the 128-row side of tcgen05.mma: a CTA owns
// a tile of 128 rows of W (128 output columns) and all tokens (BN = 32, 64 or 128 accumulator
// columns in tensor memory).  A matrix has few such tiles (16 for 2,048 outputs), far fewer than
// the GPU has SMs, so the K range of a tile is cut over the CTAs of a thread-block cluster: each
// streams its K slice of the tile through a TMA ring, and the partial sums meet in distributed
// shared memory.  CTA r of the cluster owns a share of the tile's rows (whole groups of four).
// Every CTA reads its accumulator from tensor memory and stores each row straight into the shared
// memory of the row's owner (st.shared::cluster: the stores are not waited for), into a slot of its
// own; after one cluster barrier every owner adds the S slots in CTA order from its own shared
// memory and writes its slice of the result.  No partial sum goes through global memory, no second
// kernel adds them, and the order of the additions is fixed, so the result does not depend on
// timing.
//
// What follows the product is done where the sums meet:
//   store     C = sum (bf16 or fp32)
//   accum     C += sum (the residual; fp32).  With `emit_w` the kernel also writes what the RMSNorm
//             after this addition needs: bf16(C * emit_w) and, per CTA and token, the sum of squares
//             of the CTA's slice of the row (the consumer adds the parts in CTA order).
//   swiglu    W holds gate and up rows in alternating blocks of 128; the CTA keeps two accumulators
//             and writes silu(gate) * up (both rounded to bf16 first, as separate products would
//             store them).
// `scale_part`: the rows of A are bf16(x * norm weight) of such an emit; every token's result is
// multiplied by rsqrt(mean of squares + eps), which the epilogue warps work out from the parts
// while the main loop runs.
//
// The weights of the first stages are requested before griddepcontrol.wait (no kernel writes
// them), so with programmatic dependent launch the first trip to HBM runs under the tail of the
// kernel before.  No load is multicast.  Every wait on an mbarrier is bounded; a CTA whose wait ran
// out records a code, sends zeros and still arrives at the cluster barrier, so its peers never
// wait for it in vain.
//
// The reference computes these products row by row with matrix-vector kernels on quantised
// weights (src/lfm25_gpu.cu:148-202, 860-934) and has no batch of this size on its LFM path.
#include "sm100.cuh"
#include <algorithm>

namespace {

constexpr int BM = 128;            // rows of W per tile (UMMA M)
constexpr int BK = 64;             // K elements per stage: one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;   // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..5: epilogue
constexpr int MAX_SPLITS = 8;      // the portable cluster size

// Ring depths (stages of 64 K elements): what fits beside the memory that the peers write into.
#ifndef SKINNY_STAGES
#define SKINNY_STAGES 7
#endif
#ifndef SKINNY_STAGES_128
#define SKINNY_STAGES_128 4
#endif
#ifndef SKINNY_PAIR_STAGES_32
#define SKINNY_PAIR_STAGES_32 5
#endif
#ifndef SKINNY_PAIR_STAGES_64
#define SKINNY_PAIR_STAGES_64 3
#endif
#ifndef SKINNY_CH
#define SKINNY_CH 16               // accumulator columns read from tensor memory and sent to their owners at a time
#endif

enum : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

struct SkinnyParams {
    void* out;                 // [M, ldc] bf16 or fp32
    long long ldc;
    int out_dtype;
    int M, n_out;              // tokens; columns of `out`
    int k_blocks, kb_per_split, splits;
    int epi;
    const float* emit_w;       // accum only, may be null: [n_out]
    bf16* emit_xw;             // [M, n_out]
    float* emit_part;          // [CTAs, part_stride]
    int part_stride;
    const float* scale_part;   // may be null: [scale_parts, scale_stride]
    int scale_parts, scale_stride;
    float scale_eps;
    int K;
    int* status;
    long long* trace;          // null, or 8 time stamps per CTA of this launch (tuff_gemm_skinny_trace)
};

template <int BN> __device__ __forceinline__ constexpr uint32_t instr_desc() {
    // fp32 accumulator, bf16 x bf16, both K-major, M = 128, N = BN
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <int BN, bool PAIR, int STAGES>
struct Layout {
    static constexpr int NW = PAIR ? 2 : 1;
    static constexpr int W_BYTES = BM * BK * 2;
    static constexpr int A_BYTES = BN * BK * 2;
    static constexpr int STAGE = NW * W_BYTES + A_BYTES;
    static constexpr int RING = STAGES * STAGE;
    static constexpr int SQ = BN * (BM / 4) * 4;              // squares of an emit: a float per token and group of four rows (in the ring's memory, after the main loop)
    static_assert(SQ <= RING, "the ring must hold what the epilogue puts there");
    // What the peers send: S slots of [token][rows of this CTA's share] fp32 per accumulator.  A share has at
    // most 4 * ceil(32 / S) rows, so S shares have at most 128 + 4 * (S - 1) rows together.
    static constexpr int RECV_ROWS = BM + 4 * (MAX_SPLITS - 1);
    static constexpr int RECV = NW * BN * RECV_ROWS * 4;      // memory of its own: peers write it while this CTA's main loop still runs
    static constexpr int BARS = RING + RECV;                  // full[STAGES], empty[STAGES], acc_full
    static constexpr int TMEM_SLOT = BARS + (2 * STAGES + 1) * 8;
    static constexpr int SCALE = TMEM_SLOT + 16;              // [BN] floats
    static constexpr int TOTAL = SCALE + BN * 4 + 1024;       // + room to align the base to 1024 bytes
    static_assert(TOTAL <= 227 * 1024, "more shared memory than a CTA may have");
    static constexpr uint32_t TMEM_COLS = NW * BN <= 32 ? 32 : NW * BN <= 64 ? 64 : NW * BN <= 128 ? 128 : 256;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Every thread of every CTA of the cluster arrives; what it stored before, also into a peer's shared
// memory, is visible to the peers once they have waited.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// The address, in the cluster's shared window, of `local_addr` in the shared memory of CTA `rank`.
__device__ __forceinline__ uint32_t peer_addr(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_peer(uint32_t remote, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// First group of four rows of rank r's share of a 128-row tile split over S CTAs.
__device__ __forceinline__ int share_lo(uint32_t r, uint32_t S) { return (int)(r * (BM / 4) / S); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int BN, bool PAIR, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, SkinnyParams p) {
    using L = Layout<BN, PAIR, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BARS;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t acc_full = bars + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::TMEM_SLOT);
    float* scale_s = reinterpret_cast<float*>(base_ptr + L::SCALE);
    const uint32_t recv = base + L::RING;                                  // [NW][S slots][BN tokens][rows of this CTA's share]
    const float* recv_s = reinterpret_cast<const float*>(base_ptr + L::RING);
    float* sq_s = reinterpret_cast<float*>(base_ptr);                      // [tokens * row groups of this CTA's share]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t S = (uint32_t)p.splits, rank = cluster_rank();
    const int tile = blockIdx.x / (int)S;
    const int kb0 = (int)rank * p.kb_per_split;
    const int nkb = max(0, min(p.kb_per_split, p.k_blocks - kb0));
    const int w_row0 = tile * BM * L::NW;                                  // first row of W of this tile (pair: gate block, then up block)
    long long* trace = p.trace ? p.trace + (size_t)blockIdx.x * 8 : nullptr;
    if (trace && threadIdx.x == 0) trace[0] = global_ns();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + (uint32_t)L::TMEM_SLOT), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    if (trace && threadIdx.x == 0) trace[1] = global_ns();
    // A store into a peer's shared memory needs the peer to have started.  Every thread arrives here, and waits
    // (long after, so never in earnest) before the first such store.
    cluster_arrive();

    if (warp == 0) {
        if (lane == 0) {
            auto load_w = [&](int i) {
                const int s = i % STAGES;
                const uint32_t dst = base + (uint32_t)(s * L::STAGE);
                mbar_expect_tx(full_bar(s), L::STAGE);
                tma_load_2d(dst, &map_w, full_bar(s), (kb0 + i) * BK, w_row0);
                if (PAIR) tma_load_2d(dst + L::W_BYTES, &map_w, full_bar(s), (kb0 + i) * BK, w_row0 + BM);
            };
            auto load_a = [&](int i) {
                const int s = i % STAGES;
                tma_load_2d(base + (uint32_t)(s * L::STAGE + L::NW * L::W_BYTES), &map_a, full_bar(s), (kb0 + i) * BK, 0);
            };
            const int pre = min(nkb, STAGES);
            for (int i = 0; i < pre; ++i) load_w(i);           // weights: written by no kernel, so not ordered after one
            pdl_wait();
            pdl_launch_dependents();
            if (trace) trace[2] = global_ns();
            for (int i = 0; i < pre; ++i) load_a(i);
            for (int i = pre; i < nkb; ++i) {
                if (!mbar_wait(empty_bar(i % STAGES), ((i / STAGES) & 1u) ^ 1u, p.status, 51)) { ok = false; break; }
                load_w(i);
                load_a(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<BN>();
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(full_bar(s), (i / STAGES) & 1u, p.status, 52)) { ok = false; break; }
                if (trace && i == 0) trace[3] = global_ns();
                tc_fence_after();
                const uint32_t w = base + (uint32_t)(s * L::STAGE), a = w + L::NW * L::W_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    umma(tmem_base, smem_desc_k_major(w + k * UMMA_K * 2), smem_desc_k_major(a + k * UMMA_K * 2), idesc,
                         (i > 0 || k > 0) ? 1u : 0u);
                    if (PAIR)
                        umma(tmem_base + BN, smem_desc_k_major(w + L::W_BYTES + k * UMMA_K * 2),
                             smem_desc_k_major(a + k * UMMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));
            }
            if (ok) umma_commit(acc_full);          // arrives once every MMA above has retired (at once if there was none)
        }
    } else {
        // ---- epilogue warps, part one: row scales; then this CTA's accumulator, row by row, to the rows' owners
        const int t = threadIdx.x - 64;                        // 0..127
        const int quad = warp & 3;                             // the 32 tensor-memory lanes this warp may read
        const int row = quad * 32 + lane;                      // row of the tile
        pdl_wait();
        if (t < BN) {
            float sc = 1.f;
            if (p.scale_part && t < p.M) {
                float ss = 0.f;
                for (int q = 0; q < p.scale_parts; ++q) ss += ld_act(p.scale_part + (size_t)q * p.scale_stride + t);
                sc = rsqrtf(ss / (float)p.K + p.scale_eps);
            }
            scale_s[t] = sc;
        }
        // the owner of this thread's row, and where the row lies in the owner's slot for this CTA
        uint32_t owner = 0;
        while (owner + 1 < S && share_lo(owner + 1, S) * 4 <= row) ++owner;
        const int o_rows = (share_lo(owner + 1, S) - share_lo(owner, S)) * 4;
        const uint32_t dst0 = peer_addr(recv, owner) + (uint32_t)((rank * BN * o_rows + (row - share_lo(owner, S) * 4)) * 4);
        if (!mbar_wait(acc_full, 0, p.status, 53)) ok = false;
        ok = __all_sync(0xffffffffu, ok);                      // tcgen05.ld below is a warp-wide instruction
        cluster_wait();                                        // every CTA of the cluster runs (see above)
        if (trace && t == 0) trace[4] = global_ns();
        tc_fence_after();
        constexpr int CH = SKINNY_CH < BN ? SKINNY_CH : BN;    // columns read from tensor memory at a time
#pragma unroll 1
        for (int h = 0; h < L::NW; ++h) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t r[CH];
                if (ok && nkb > 0) {
                    const uint32_t ta = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * BN + c0);
                    if constexpr (CH == 64) tmem_ld64(ta, r); else if constexpr (CH == 32) tmem_ld32(ta, r); else tmem_ld16(ta, r);
                } else {
#pragma unroll
                    for (int j = 0; j < CH; ++j) r[j] = 0u;
                }
                // slot layout at the owner: [accumulator h][CTA][token][row of the share]
                const uint32_t d = dst0 + (uint32_t)((h * (int)S * BN + c0) * o_rows * 4);
#pragma unroll
                for (int j = 0; j < CH; ++j) st_peer(d + (uint32_t)(j * o_rows * 4), __uint_as_float(r[j]));
            }
        }
        tc_fence_before();
    }
    __syncwarp();
    if (warp < 2) cluster_wait();                              // the first phase of the cluster barrier, for these warps
    cluster_arrive();
    // ---- part two (all warps): this CTA's share of the tile's rows, added over the slots in CTA order
    const int t2 = threadIdx.x;
    const int q_lo = share_lo(rank, S), nq = share_lo(rank + 1, S) - q_lo, my_rows = nq * 4;
    const int n_tok = min(BN, p.M);
    const int total = n_tok * nq;                              // items: a token and a group of four rows
    const int col0 = tile * BM;                                // first column of `out` of this tile
    const int esz = p.out_dtype == TUFF_F32 ? 4 : 2;
    const bool vec = ((uintptr_t)p.out % (4 * esz) == 0) && (p.ldc % 4 == 0) && (p.n_out % 4 == 0) &&
                     (!p.emit_w || ((uintptr_t)p.emit_xw % 8 == 0 && (uintptr_t)p.emit_w % 16 == 0));
    // the residual values of this thread's first items do not depend on the peers: ask for them before waiting
    constexpr int PRE = 4;
    float4 old[PRE];
    if (!PAIR && p.epi == EPI_ACCUM && vec) {
#pragma unroll
        for (int i = 0; i < PRE; ++i) {
            const int idx = t2 + i * NUM_THREADS;
            old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < total) {
                const int tok = idx / nq, col = col0 + (q_lo + idx - tok * nq) * 4;
                if (col + 4 <= p.n_out) old[i] = __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)tok * p.ldc + col));
            }
        }
    }
    cluster_wait();                     // every CTA's rows have arrived at their owners
    if (trace && threadIdx.x == 64) trace[5] = global_ns();

    // Two items at a time, their loads first: with so few warps on the SM nothing else hides a latency.
    for (int idx0 = t2, it = 0; idx0 < total; idx0 += 2 * NUM_THREADS, it += 2) {
        int tok[2], col[2];
        bool live[2];
        float v[2][4], u[2][4], ew[2][4], sc[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int idx = idx0 + k * NUM_THREADS;
            live[k] = idx < total;
            tok[k] = live[k] ? idx / nq : 0;
            const int ql = live[k] ? idx - tok[k] * nq : 0;
            col[k] = col0 + (q_lo + ql) * 4;
            const float* at = recv_s + (size_t)tok[k] * my_rows + ql * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[k][j] = 0.f; u[k][j] = 0.f; ew[k][j] = 0.f; }
#pragma unroll
            for (uint32_t s2 = 0; s2 < (uint32_t)MAX_SPLITS; ++s2) {
                if (s2 < S) {
                    const float4 pv = *reinterpret_cast<const float4*>(at + (size_t)s2 * BN * my_rows);
                    v[k][0] += pv.x; v[k][1] += pv.y; v[k][2] += pv.z; v[k][3] += pv.w;
                    if (PAIR) {
                        const float4 pu = *reinterpret_cast<const float4*>(at + (size_t)(S + s2) * BN * my_rows);
                        u[k][0] += pu.x; u[k][1] += pu.y; u[k][2] += pu.z; u[k][3] += pu.w;
                    }
                }
            }
            sc[k] = scale_s[tok[k]];
            if (!PAIR && p.emit_w && live[k]) {
                if (vec && col[k] + 4 <= p.n_out) {
                    const float4 w4 = __ldg(reinterpret_cast<const float4*>(p.emit_w + col[k]));
                    ew[k][0] = w4.x; ew[k][1] = w4.y; ew[k][2] = w4.z; ew[k][3] = w4.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) if (col[k] + j < p.n_out) ew[k][j] = __ldg(p.emit_w + col[k] + j);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (!live[k]) continue;
            float sq = 0.f;
            if (col[k] < p.n_out) {
                const size_t o = (size_t)tok[k] * p.ldc + col[k];
                const bool whole = vec && col[k] + 4 <= p.n_out;
                float r[4];
                if (PAIR) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float gq = bf16_round(v[k][j] * sc[k]), uq = bf16_round(u[k][j] * sc[k]);
                        r[j] = gq / (1.f + __expf(-gq)) * uq;
                    }
                } else if (p.epi == EPI_ACCUM) {
                    float x[4];
                    if (whole) {
                        float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        bool have = false;
#pragma unroll
                        for (int i = 0; i < PRE; ++i) if (it + k == i) { w4 = old[i]; have = true; }
                        if (!have) w4 = __ldcg(reinterpret_cast<const float4*>((const float*)p.out + o));
                        x[0] = w4.x; x[1] = w4.y; x[2] = w4.z; x[3] = w4.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) x[j] = col[k] + j < p.n_out ? ld_act((const float*)p.out + o + j) : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) r[j] = x[j] + v[k][j] * sc[k];
                    if (p.emit_w) {
                        float e[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool in = col[k] + j < p.n_out;
                            e[j] = in ? r[j] * ew[k][j] : 0.f;
                            sq += in ? r[j] * r[j] : 0.f;
                        }
                        bf16* xw = p.emit_xw + (size_t)tok[k] * p.n_out + col[k];
                        if (whole) {
                            *reinterpret_cast<uint2*>(xw) = make_uint2(pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) if (col[k] + j < p.n_out) xw[j] = __float2bfloat16_rn(e[j]);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) r[j] = v[k][j] * sc[k];
                }
                if (p.out_dtype == TUFF_F32) {
                    float* op = (float*)p.out + o;
                    if (whole) {
                        *reinterpret_cast<float4*>(op) = make_float4(r[0], r[1], r[2], r[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) if (col[k] + j < p.n_out) op[j] = r[j];
                    }
                } else {
                    bf16* op = (bf16*)p.out + o;
                    if (whole) {
                        *reinterpret_cast<uint2*>(op) = make_uint2(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) if (col[k] + j < p.n_out) op[j] = __float2bfloat16_rn(r[j]);
                    }
                }
            }
            if (!PAIR && p.emit_w) sq_s[idx0 + k * NUM_THREADS] = sq;
        }
    }
    if (!PAIR && p.emit_w) {
        __syncthreads();
        // a token's squares over this CTA's rows, added in row order
        if (t2 < p.part_stride) {
            float ss = 0.f;
            if (t2 < n_tok)
                for (int ql = 0; ql < nq; ++ql) ss += sq_s[t2 * nq + ql];
            p.emit_part[(size_t)blockIdx.x * p.part_stride + t2] = ss;
        }
    }
    if (trace && threadIdx.x == 64) trace[6] = global_ns();
    if (!ok) {
        // A wait ran out.  Give copies that may still be in flight time to land before the
        // shared memory is released.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    if (trace && threadIdx.x == 64) trace[7] = global_ns();
    // (after the barrier no CTA touches a peer's shared memory, so a CTA may leave before its peers)
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
long long* g_trace = nullptr;
int g_trace_launches = 0, g_trace_capacity = 0;

struct Plan { int tiles, splits, kb_per_split, bn; bool ok; };

template <int BN, bool PAIR, int STAGES>
int max_clusters(int splits) {
    // how many clusters of `splits` CTAs of this kernel the device holds at once (asked once per size)
    using L = Layout<BN, PAIR, STAGES>;
    static int cached[MAX_SPLITS + 1] = {0};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[splits]) return cached[splits];
    if (cudaFuncSetAttribute(gemm_skinny_kernel<BN, PAIR, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
        return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits * 64); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = L::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_skinny_kernel<BN, PAIR, STAGES>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    cached[splits] = n > 0 ? n : -1;
    return cached[splits];
}

template <int BN, bool PAIR, int STAGES>
Plan plan_for(int w_rows, int K) {
    Plan pl{};
    pl.bn = BN;
    pl.tiles = PAIR ? w_rows / (2 * BM) : ceil_div(w_rows, BM);
    const int k_blocks = ceil_div(K, BK), sms = sm_count();
    if (pl.tiles >= sms) { pl.ok = false; return pl; }          // enough tiles for every SM: the persistent product does these
    int s = std::min({MAX_SPLITS, sms / pl.tiles, std::max(1, k_blocks / 2)});
    if (const char* e = getenv("TUFF_SKINNY_SPLITS")) { const int v = atoi(e); if (v >= 1 && v <= MAX_SPLITS) s = std::min(v, k_blocks); }
    // All clusters of the product must run at once, and with room to spare: a cluster needs its SMs free in one
    // GPC, and while the CTAs of the kernel before still leave theirs, a count that only just fits is placed in
    // two rounds (seen: 44 clusters of 3, of 45 that fit an idle GPU, took twice the time).
    int slack = 90;
    if (const char* e = getenv("TUFF_SKINNY_SLACK")) { const int v = atoi(e); if (v >= 10 && v <= 100) slack = v; }
    while (s > 1 && max_clusters<BN, PAIR, STAGES>(s) * slack < pl.tiles * 100) --s;
    if (max_clusters<BN, PAIR, STAGES>(s) < 1) { pl.ok = false; return pl; }
    pl.kb_per_split = ceil_div(k_blocks, s);
    pl.splits = ceil_div(k_blocks, pl.kb_per_split);
    pl.ok = true;
    return pl;
}

Plan plan(int M, int w_rows, int K, bool pair) {
    if (M <= 32) return pair ? plan_for<32, true, SKINNY_PAIR_STAGES_32>(w_rows, K) : plan_for<32, false, SKINNY_STAGES>(w_rows, K);
    if (M <= 64) return pair ? plan_for<64, true, SKINNY_PAIR_STAGES_64>(w_rows, K) : plan_for<64, false, SKINNY_STAGES>(w_rows, K);
    if (pair) { Plan no{}; return no; }        // two accumulators of 128 tokens leave no room for a ring: the caller runs the activation by itself
    return plan_for<128, false, SKINNY_STAGES_128>(w_rows, K);
}

template <int BN, bool PAIR, int STAGES>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const SkinnyParams& p, int grid, cudaStream_t stream) {
    using L = Layout<BN, PAIR, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<BN, PAIR, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    const int rc = (int)cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<BN, PAIR, STAGES>, mw, ma, p);
    return rc ? rc : launch_status();
}

}  // namespace

// CTAs (= parts of an emit) of the product with these sizes, or 0 if this kernel does not take it
// (more tiles than SMs, or sizes it refuses): the caller then uses another product.
// w_rows: rows of W (for swiglu the stacked gate and up rows).
extern "C" int tuff_gemm_skinny_ctas(int M, int w_rows, int K, int epilogue) {
    if (M <= 0 || M > 128 || w_rows <= 0 || K <= 0 || (K % 8)) return 0;
    if (epilogue == EPI_SWIGLU && (w_rows % (2 * BM))) return 0;
    const Plan pl = plan(M, w_rows, K, epilogue == EPI_SWIGLU);
    return pl.ok ? pl.tiles * pl.splits : 0;
}

// C[M, n_out] (=|+=) A[M,K] W[w_rows,K]^T for M <= 128; bf16 A and W.  epilogue 0: store (C bf16 or
// fp32, n_out = w_rows); 1: C += (fp32); 2 (M <= 64): W = gate and up rows in alternating blocks of 128, C bf16
// [M, w_rows / 2] = silu(gate) * up.  emit_w / emit_xw / emit_part (epilogue 1, may be null): see the
// head of this file; emit_part has tuff_gemm_skinny_ctas rows of part_stride >= M floats.
// scale_part (may be null): [scale_parts, scale_stride] sums of squares of the rows of A's source.
// Requirements: K % 8 == 0, lda % 8 == 0, ldw % 8 == 0, A and W 16-byte aligned.
extern "C" int tuff_gemm_skinny(const void* A, const void* W, void* C, int c_dtype, int M, int w_rows, int K,
                                long long lda, long long ldw, long long ldc, int epilogue,
                                const float* emit_w, void* emit_xw, float* emit_part, int part_stride,
                                const float* scale_part, int scale_parts, int scale_stride, float scale_eps,
                                int* status, cudaStream_t stream) {
    if (M <= 0 || w_rows <= 0) return 0;
    if (M > 128 || K <= 0 || epilogue < 0 || epilogue > 2 || !status) return TUFF_E_SIZE;
    if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TUFF_E_ALIGN;
    const bool pair = epilogue == EPI_SWIGLU;
    if (pair && ((w_rows % (2 * BM)) || c_dtype != TUFF_BF16)) return TUFF_E_SIZE;
    if (epilogue == EPI_ACCUM && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if (c_dtype != TUFF_F32 && c_dtype != TUFF_BF16) return TUFF_E_DTYPE;
    if (emit_w && (epilogue != EPI_ACCUM || !emit_xw || !emit_part || part_stride < M)) return TUFF_E_SIZE;
    if (scale_part && (scale_parts <= 0 || scale_stride < M)) return TUFF_E_SIZE;
    const Plan pl = plan(M, w_rows, K, pair);
    if (!pl.ok) return TUFF_E_SIZE;
    SkinnyParams p{};
    p.out = C; p.ldc = ldc; p.out_dtype = c_dtype; p.M = M; p.n_out = pair ? w_rows / 2 : w_rows;
    p.k_blocks = ceil_div(K, BK); p.kb_per_split = pl.kb_per_split; p.splits = pl.splits; p.epi = epilogue;
    p.emit_w = emit_w; p.emit_xw = (bf16*)emit_xw; p.emit_part = emit_part; p.part_stride = part_stride;
    p.scale_part = scale_part; p.scale_parts = scale_parts; p.scale_stride = scale_stride; p.scale_eps = scale_eps;
    p.K = K; p.status = status;
    const int n_ctas = pl.tiles * pl.splits;
    if (g_trace && g_trace_launches < g_trace_capacity && n_ctas <= 256) p.trace = g_trace + (size_t)(g_trace_launches++) * 256 * 8;
    CUtensorMap mw, ma;
    if (!tensor_map(&mw, W, w_rows, K, ldw, BM) || !tensor_map(&ma, A, M, K, lda, pl.bn)) return TUFF_E_ALIGN;
    const int grid = pl.tiles * pl.splits;
    if (pl.bn == 32)
        return pair ? launch<32, true, SKINNY_PAIR_STAGES_32>(mw, ma, p, grid, stream) : launch<32, false, SKINNY_STAGES>(mw, ma, p, grid, stream);
    if (pl.bn == 64)
        return pair ? launch<64, true, SKINNY_PAIR_STAGES_64>(mw, ma, p, grid, stream) : launch<64, false, SKINNY_STAGES>(mw, ma, p, grid, stream);
    return launch<128, false, SKINNY_STAGES_128>(mw, ma, p, grid, stream);
}

// How many clusters of `splits` CTAs of the kernel for up to `m` tokens the device holds at once (0: none, or
// sizes that the kernel does not take).
extern "C" int tuff_gemm_skinny_max_clusters(int m, int pair, int splits) {
    if (splits < 1 || splits > MAX_SPLITS || m < 1 || m > 128 || (pair && m > 64)) return 0;
    int n;
    if (m <= 32) n = pair ? max_clusters<32, true, SKINNY_PAIR_STAGES_32>(splits) : max_clusters<32, false, SKINNY_STAGES>(splits);
    else if (m <= 64) n = pair ? max_clusters<64, true, SKINNY_PAIR_STAGES_64>(splits) : max_clusters<64, false, SKINNY_STAGES>(splits);
    else n = max_clusters<128, false, SKINNY_STAGES_128>(splits);
    return n > 0 ? n : 0;
}

// Sets (or, with null, clears) a trace buffer: room for `launches` launches of up to 256 CTAs, 8 time
// stamps (ns of the global timer) each: CTA start, set up, predecessor finished, first stage arrived,
// accumulator complete, partial tiles exchanged, slice written, peers done.  Returns the launches traced
// since the last call.  A diagnostic: stamps cost a few hundred ns per CTA.
extern "C" int tuff_gemm_skinny_trace(long long* buf, int launches) {
    const int n = g_trace_launches;
    g_trace = buf; g_trace_capacity = buf ? launches : 0; g_trace_launches = 0;
    return n;
}
