// The matrix products of a step with 17 to 128 tokens (many requests decoding together, or a
// short portion of a prompt):  C[M,N] (=|+=) A[M,K] * W[N,K]^T, bf16 operands, fp32 accumulation.
//
// The weights are the only large operand, so they take the 128-row side of tcgen05.mma: a CTA owns
// a tile of 128 rows of W (128 output columns) and all tokens (BN = 32, 64 or 128 accumulator
// columns in tensor memory).  A matrix has few such tiles (16 for 2,048 outputs), far fewer than
// the GPU has SMs, so the K range of a tile is cut over the CTAs of a thread-block cluster: each
// streams its K slice of the tile through a TMA ring, and the partial sums meet in distributed
// shared memory.  Every CTA copies its accumulator to its own shared memory; after a cluster
// barrier CTA r adds, in CTA order, its share of the rows (whole groups of four) of all S partial tiles, which
// it reads from its peers with ld.shared::cluster, and writes that slice of the result.  No
// partial sum goes through global memory, no second kernel adds them, and the order of the
// additions is fixed, so the result does not depend on timing.
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
// out records a code, skips its work and still arrives at both cluster barriers, so its peers
// never wait for it in vain.
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
    static constexpr int PARTIAL = NW * BN * BM * 4;          // this CTA's accumulator(s), [token][row] fp32, in the ring's memory
    static constexpr int SQ = BN * BM * 4;                    // squares of an emit, behind the partials
    static_assert(PARTIAL + (PAIR ? 0 : SQ) <= RING, "the ring must hold what the epilogue puts there");
    static constexpr int BARS = RING;                         // full[STAGES], empty[STAGES], acc_full
    static constexpr int TMEM_SLOT = BARS + (2 * STAGES + 1) * 8;
    static constexpr int SCALE = TMEM_SLOT + 16;              // [BN] floats
    static constexpr int TOTAL = SCALE + BN * 4 + 1024;       // + room to align the base to 1024 bytes
    static constexpr uint32_t TMEM_COLS = NW * BN <= 32 ? 32 : NW * BN <= 64 ? 64 : NW * BN <= 128 ? 128 : 256;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Every thread of every CTA of the cluster arrives and waits; shared-memory writes before it are
// visible to the peers after it.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Four consecutive floats at `local_addr` (16-byte aligned) of the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ float4 ld_peer4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
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
    float* partial_s = reinterpret_cast<float*>(base_ptr);                 // [NW][BN][BM]
    float* sq_s = reinterpret_cast<float*>(base_ptr + L::PARTIAL);         // [tokens * row groups of this CTA's slice]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t S = (uint32_t)p.splits, rank = cluster_rank();
    const int tile = blockIdx.x / (int)S;
    const int kb0 = (int)rank * p.kb_per_split;
    const int nkb = max(0, min(p.kb_per_split, p.k_blocks - kb0));
    const int w_row0 = tile * BM * L::NW;                                  // first row of W of this tile (pair: gate block, then up block)

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
        // ---- epilogue warps, part one: row scales, then this CTA's accumulator into its shared memory
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
        if (!mbar_wait(acc_full, 0, p.status, 53)) ok = false;
        ok = __all_sync(0xffffffffu, ok);                      // tcgen05.ld below is a warp-wide instruction
        tc_fence_after();
#pragma unroll 1
        for (int h = 0; h < L::NW; ++h) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                if (ok && nkb > 0) {
                    tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * BN + c0), r);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) partial_s[(size_t)(h * BN + c0 + j) * BM + row] = __uint_as_float(r[j]);
            }
        }
        tc_fence_before();
    }
    __syncwarp();
    cluster_sync_all();                 // every CTA's partial tile is in its shared memory

    if (warp >= 2) {
        // ---- part two: this CTA's rows of the tile (whole groups of four), added over the cluster in CTA order
        const int t = threadIdx.x - 64;
        const int q_lo = (int)(rank * (BM / 4) / S), q_hi = (int)((rank + 1) * (BM / 4) / S), nq = q_hi - q_lo;
        const int n_tok = min(BN, p.M);
        const int total = n_tok * nq;
        const int col0 = tile * BM;                            // first column of `out` of this tile
        const int esz = p.out_dtype == TUFF_F32 ? 4 : 2;
        const bool vec = ((uintptr_t)p.out % (4 * esz) == 0) && (p.ldc % 4 == 0) && (p.n_out % 4 == 0) &&
                         (!p.emit_w || ((uintptr_t)p.emit_xw % 8 == 0 && (uintptr_t)p.emit_w % 16 == 0));
        for (int idx = t; idx < total; idx += 128) {
            const int tok = idx / nq, ql = idx - tok * nq, row = (q_lo + ql) * 4, col = col0 + row;
            const uint32_t at = base + (uint32_t)((tok * BM + row) * 4);
            float4 pv[MAX_SPLITS], pu[MAX_SPLITS];
#pragma unroll
            for (uint32_t s = 0; s < (uint32_t)MAX_SPLITS; ++s) {         // all peers' loads in flight together
                pv[s] = s < S ? ld_peer4(at, s) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (PAIR) pu[s] = s < S ? ld_peer4(at + (uint32_t)(BN * BM * 4), s) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float v[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (uint32_t s = 0; s < (uint32_t)MAX_SPLITS; ++s) {
                if (s < S) {
                    v[0] += pv[s].x; v[1] += pv[s].y; v[2] += pv[s].z; v[3] += pv[s].w;
                    if (PAIR) { u[0] += pu[s].x; u[1] += pu[s].y; u[2] += pu[s].z; u[3] += pu[s].w; }
                }
            }
            const float sc = scale_s[tok];
            float sq = 0.f;
            if (col < p.n_out) {
                const size_t o = (size_t)tok * p.ldc + col;
                const bool whole = vec && col + 4 <= p.n_out;
                float r[4];
                if (PAIR) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float gq = bf16_round(v[j] * sc), uq = bf16_round(u[j] * sc);
                        r[j] = gq / (1.f + expf(-gq)) * uq;
                    }
                } else if (p.epi == EPI_ACCUM) {
                    float x[4];
                    if (whole) {
                        const float4 old = __ldcg(reinterpret_cast<const float4*>((const float*)p.out + o));
                        x[0] = old.x; x[1] = old.y; x[2] = old.z; x[3] = old.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) x[j] = col + j < p.n_out ? ld_act((const float*)p.out + o + j) : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) r[j] = x[j] + v[j] * sc;
                    if (p.emit_w) {
                        float e[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool in = col + j < p.n_out;
                            e[j] = in ? r[j] * p.emit_w[col + j] : 0.f;
                            sq += in ? r[j] * r[j] : 0.f;
                        }
                        bf16* xw = p.emit_xw + (size_t)tok * p.n_out + col;
                        if (whole) {
                            *reinterpret_cast<uint2*>(xw) = make_uint2(pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) if (col + j < p.n_out) xw[j] = __float2bfloat16_rn(e[j]);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) r[j] = v[j] * sc;
                }
                if (p.out_dtype == TUFF_F32) {
                    float* op = (float*)p.out + o;
                    if (whole) {
                        *reinterpret_cast<float4*>(op) = make_float4(r[0], r[1], r[2], r[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) if (col + j < p.n_out) op[j] = r[j];
                    }
                } else {
                    bf16* op = (bf16*)p.out + o;
                    if (whole) {
                        *reinterpret_cast<uint2*>(op) = make_uint2(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) if (col + j < p.n_out) op[j] = __float2bfloat16_rn(r[j]);
                    }
                }
            }
            if (!PAIR && p.emit_w) sq_s[idx] = sq;
        }
        if (!PAIR && p.emit_w) {
            epilogue_bar();
            // a token's squares over this CTA's rows, added in row order
            if (t < p.part_stride) {
                float ss = 0.f;
                if (t < n_tok)
                    for (int ql = 0; ql < nq; ++ql) ss += sq_s[t * nq + ql];
                p.emit_part[(size_t)blockIdx.x * p.part_stride + t] = ss;
            }
        }
    }
    if (!ok) {
        // A wait ran out.  Give copies that may still be in flight time to land before the
        // shared memory is released.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncwarp();
    cluster_sync_all();                 // no CTA leaves while a peer may still read its shared memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
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
    while (s > 1 && max_clusters<BN, PAIR, STAGES>(s) < pl.tiles) --s;     // all clusters of the product run at once
    if (max_clusters<BN, PAIR, STAGES>(s) < 1) { pl.ok = false; return pl; }
    pl.kb_per_split = ceil_div(k_blocks, s);
    pl.splits = ceil_div(k_blocks, pl.kb_per_split);
    pl.ok = true;
    return pl;
}

Plan plan(int M, int w_rows, int K, bool pair) {
    if (M <= 32) return pair ? plan_for<32, true, 6>(w_rows, K) : plan_for<32, false, 8>(w_rows, K);
    if (M <= 64) return pair ? plan_for<64, true, 5>(w_rows, K) : plan_for<64, false, 8>(w_rows, K);
    return pair ? plan_for<128, true, 4>(w_rows, K) : plan_for<128, false, 6>(w_rows, K);
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
// fp32, n_out = w_rows); 1: C += (fp32); 2: W = gate and up rows in alternating blocks of 128, C bf16
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
    CUtensorMap mw, ma;
    if (!tensor_map(&mw, W, w_rows, K, ldw, BM) || !tensor_map(&ma, A, M, K, lda, pl.bn)) return TUFF_E_ALIGN;
    const int grid = pl.tiles * pl.splits;
    if (pl.bn == 32) return pair ? launch<32, true, 6>(mw, ma, p, grid, stream) : launch<32, false, 8>(mw, ma, p, grid, stream);
    if (pl.bn == 64) return pair ? launch<64, true, 5>(mw, ma, p, grid, stream) : launch<64, false, 8>(mw, ma, p, grid, stream);
    return pair ? launch<128, true, 4>(mw, ma, p, grid, stream) : launch<128, false, 6>(mw, ma, p, grid, stream);
}
