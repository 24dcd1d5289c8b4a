// Causal attention of prompt portions over the paged cache on the Blackwell tensor cores
// (tcgen05.mma, accumulators in tensor memory), head size 64.
//
// One CTA takes 128 consecutive query tokens of one request and one query head and walks the
// 64-key tiles its tokens can see.  Per tile:
//     S  = Q K^T          tcgen05.mma, M=128 (query rows) x N=64 (keys) x K=head size, into TMEM
//     P  = softmax part   four warps, one thread per query row (= one TMEM lane): tcgen05.ld of
//                         the row's 64 scores, mask, exp2 against the row's reference maximum,
//                         bf16 P written back to tensor memory (tcgen05.st, two keys a column)
//     O += P V            tcgen05.mma with the A operand (P) read from tensor memory, M=128 x
//                         N=head size x K=64 keys, accumulated in TMEM over all tiles; V is used
//                         as it lies in the cache page ([key][dim], dim contiguous), i.e. as an
//                         MN-major shared-memory operand
// P never passes through shared memory, whose bandwidth (Q, K and V are read from it by every
// tile's MMAs, and TMA fills it) is the scarce resource of this kernel.
// The exponentials of a row are taken against a reference maximum that is raised only when the
// row's true maximum has grown by more than 2^8 beyond it (so no term exceeds 256); only then is
// the accumulated O of that row rescaled, by a read-modify-write of its TMEM lane, and that is
// rare after a row's first tiles.  Sum and output use the same reference, so the quotient is exact
// whatever the reference was.
// K and V tiles arrive through cp.async.bulk.tensor (one box per cache page, 128-byte swizzle)
// in a ring of stages; a producer warp runs ahead.  S and P are double-buffered, and the MMA
// thread issues S of tile j+1 before P V of tile j, so the tensor cores work on the next scores
// while the softmax warps are busy with the current ones.  Two CTAs fit on an SM (256 of the 512
// TMEM columns each: S twice 64, O 64, P twice 32).
//
// Online softmax as in the reference's kernel (src/lfm25_gpu.cu:506-558: scale 1/sqrt(hd) :520,
// head-to-group map :518, causal bound :531), which handles one key at a time per block.
//
// Keys outside a token's range never reach the result: their scores are replaced before the
// maximum, and the value rows of keys beyond the CTA's last position, which may never have been
// written, are zeroed in shared memory before P V (0 x NaN would otherwise spoil the row).
// Rows of the 128 that lie beyond the request's portion are computed on zero queries and not
// stored.  Every wait is bounded; a wait that runs out records a code in *status, and the CTA
// still frees its tensor memory.
#include "sm100.cuh"
#include "index.cuh"

namespace {
constexpr int TILE = 64;                 // keys per tile
constexpr int QROWS = 128;               // query tokens per CTA (UMMA M)
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;         // warps 0..3: softmax (TMEM lane quarter = warp), 4: TMA, 5: MMA + TMEM

struct TcAttnParams {
    const bf16* q; long long q_stride;
    const int* block_table; int max_blocks;
    long long n_pages;            // pages in the pool (read by a checked build only)
    const int* positions; const int* cu_q;
    bf16* out;
    int* status;
    int n_rows, H, G, page_size, window, n_blocks;
    float scale_log2;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Descriptor of V as the B operand of P V: [key][64 dims] with the dims (the N side) contiguous,
// i.e. MN-major, 128-byte swizzle: a key's row is 128 bytes, groups of 8 keys are 1024 bytes
// apart (the stride offset); the leading offset would separate 64-dim column blocks (one here).
// A K step of 16 keys moves the start address by 2048 bytes.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((TILE * 128) >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptors: fp32 accumulator, bf16 operands, M = 128.
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TILE >> 3) << 17) | ((uint32_t)(QROWS >> 4) << 24);
template <int HD> __host__ __device__ constexpr uint32_t idesc_pv() {          // B (V) is MN-major: bit 16
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QROWS >> 4) << 24);
}
template <int HD> struct Smem {
    static constexpr int Q = 0;                               // [128][64] bf16
    static constexpr int KV = Q + QROWS * 128;                // STAGES x (K tile, V tile)
    static constexpr int STAGE_BYTES = 2 * TILE * HD * 2;
    static constexpr int BARS = KV + STAGES * STAGE_BYTES;
    static constexpr int N_BARS = 1 + 2 * STAGES + 8;
    static constexpr int TMEM_SLOT = BARS + N_BARS * 8;
    static constexpr int TOTAL = TMEM_SLOT + 16 + 1024;       // + room to align the base to 1024 bytes
};

// Writes 64 bf16 (as 32 packed words) as row `row` of a [128][64] K-major swizzled tile.
__device__ __forceinline__ void store_row_swizzled(uint8_t* tile, int row, const uint32_t (&w)[32]) {
#pragma unroll
    for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(tile + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv, TcAttnParams p) {
    static_assert(HD == 64, "head size 64 only");
    using L = Smem<HD>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BARS;
    const uint32_t q_ready = bars;
    auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bars + 8u * (1 + STAGES + s); };
    auto s_full = [&](int b) { return bars + 8u * (1 + 2 * STAGES + b); };
    auto s_empty = [&](int b) { return bars + 8u * (1 + 2 * STAGES + 2 + b); };
    auto p_full = [&](int b) { return bars + 8u * (1 + 2 * STAGES + 4 + b); };
    auto pv_full = [&](int b) { return bars + 8u * (1 + 2 * STAGES + 6 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L::TMEM_SLOT);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which request, which block of its tokens, which head: heads run fastest, and later blocks
    // of a request (which see more keys) come first, so the long ones do not trail
    const int h = blockIdx.x % p.H;
    int blk = p.n_blocks - 1 - (int)(blockIdx.x / p.H);
    int row = -1, q0 = 0, q1 = 0;
    for (int r = 0; r < p.n_rows; ++r) {
        const int a = ld_act(p.cu_q + r), b = ld_act(p.cu_q + r + 1);    // written by a copy, not by the kernel before
        const int nb = (b - a + QROWS - 1) / QROWS;
        if (blk < nb) { row = r; q0 = a + blk * QROWS; q1 = b; break; }
        blk -= nb;
    }
    if (row < 0) return;                           // uniform over the CTA, before anything is allocated
    const int g = h / (p.H / p.G);
    const int n_here = min(QROWS, q1 - q0);
    const int pos0 = ld_act(p.positions + q0);     // positions of a request's tokens are consecutive
    const int pos_last = pos0 + n_here - 1;
    const int lo_cta = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int tile_lo = lo_cta / TILE, tile_hi = pos_last / TILE;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int* bt = p.block_table + (size_t)row * p.max_blocks;

    if (threadIdx.x == 0) {
        mbar_init(q_ready, 4);
        for (int s = 0; s < STAGES; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full(b), 1); mbar_init(s_empty(b), 4); mbar_init(p_full(b), 4);
            mbar_init(pv_full(b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    constexpr uint32_t TMEM_COLS = 256;                        // S twice (128), O (64), P twice (32 each)
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + (uint32_t)L::TMEM_SLOT), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * TILE, tmem_p = tmem_o + HD;
    bool ok = true;
    pdl_wait();                    // barriers and tensor memory are set up; queries, tables and pages are read from here on
    pdl_launch_dependents();

    if (warp == 4) {
        // ---------------- producer: K and V tiles through the block table
        if (lane == 0) {
            const int pages = TILE / p.page_size;
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % STAGES;
                if (!mbar_wait(kv_empty(s), ((j / STAGES) & 1) ^ 1, p.status, 31)) { ok = false; break; }
                const uint32_t sK = base + L::KV + s * L::STAGE_BYTES, sV = sK + TILE * HD * 2;
                mbar_expect_tx(kv_full(s), L::STAGE_BYTES);
                for (int i = 0; i < pages; ++i) {
                    const int bi = (tile_lo + j) * pages + i;
                    int page = bi < p.max_blocks ? ld_act(bt + bi) : -1;            // beyond the table: no page
                    if (TUFF_CHECKED && page != -1 && !page_ok(page, p.n_pages)) {  // (a load outside the tensor reads zeros)
                        bounds_fault(Bounds{0, p.n_pages, p.status}, TUFF_BOUNDS_PAGE);
                        page = -1;
                    }
                    const int y = (page * p.G + g) * p.page_size;                   // a missing page lies outside the tensor: zero fill
                    const uint32_t off = (uint32_t)(i * p.page_size) * 128;
                    tma_load_2d(sK + off, &mk, kv_full(s), 0, y);
                    tma_load_2d(sV + off, &mv, kv_full(s), 0, y);
                }
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issue: S of tile j, then P V of tile j-1
        if (lane == 0) {
            if (!mbar_wait(q_ready, 0, p.status, 32)) ok = false;
            const uint32_t sQ = base + L::Q;
            for (int j = 0; j <= n_tiles && ok; ++j) {
                if (j < n_tiles) {
                    const int s = j % STAGES, b = j & 1;
                    if (!mbar_wait(kv_full(s), (j / STAGES) & 1, p.status, 33)) { ok = false; break; }
                    if (!mbar_wait(s_empty(b), ((j >> 1) & 1) ^ 1, p.status, 34)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sK = base + L::KV + s * L::STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        umma(tmem_s + b * TILE, smem_desc_k_major(sQ + k * 32), smem_desc_k_major(sK + k * 32), IDESC_S, k > 0 ? 1u : 0u);
                    umma_commit(s_full(b));
                }
                if (j > 0) {
                    const int jj = j - 1, s = jj % STAGES, b = jj & 1;
                    if (!mbar_wait(p_full(b), (jj >> 1) & 1, p.status, 35)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sV = base + L::KV + s * L::STAGE_BYTES + TILE * HD * 2;
#pragma unroll
                    for (int k = 0; k < TILE / 16; ++k)
                        umma_ts(tmem_o, tmem_p + b * (TILE / 2) + k * 8, desc_mn_major(sV + k * 2048), idesc_pv<HD>(), (jj > 0 || k > 0) ? 1u : 0u);
                    umma_commit(pv_full(b));
                    umma_commit(kv_empty(s));          // K and V of the stage have been read once these retire
                }
            }
        }
    } else {
        // ---------------- softmax: thread r owns query row r
        const int r = threadIdx.x;                 // 0..127 = TMEM lane
        const bool valid = r < n_here;
        const int pos_r = pos0 + r;
        const int hi_r = valid ? pos_r : -1;
        const int lo_r = (p.window > 0 && pos_r - p.window + 1 > 0) ? pos_r - p.window + 1 : 0;
        const int w_first = pos0 + warp * 32, w_last = min(pos_last, w_first + 31);
        const int warp_lo = (p.window > 0 && w_first - p.window + 1 > 0) ? w_first - p.window + 1 : 0;
        const bool warp_valid = warp * 32 < n_here;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        {   // this row of Q into shared memory (zeros beyond the portion)
            uint32_t w[32];
            const bf16* qrow = p.q + (size_t)(q0 + (valid ? r : 0)) * p.q_stride + (size_t)h * HD;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 v = valid ? ld_act_u4(qrow + 8 * c) : make_uint4(0u, 0u, 0u, 0u);
                w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
            }
            store_row_swizzled(base_ptr + L::Q, r, w);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        float m_ref = -INFINITY, l = 0.f;          // reference maximum (raw score units) and sum of exp2 against it
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int b = j & 1, s = j % STAGES;
            const int key0 = (tile_lo + j) * TILE;
            const bool live = warp_valid && key0 <= w_last && key0 + TILE - 1 >= warp_lo;
            if (!mbar_wait(s_full(b), (j >> 1) & 1, p.status, 37)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[64];
            if (live) tmem_ld64(tmem_s + lane_addr + b * TILE, sr);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b));
            if (key0 + TILE - 1 > pos_last) {
                // the last tile: value rows of keys that no token of this CTA sees may never have been written
                if (!mbar_wait(kv_full(s), (j / STAGES) & 1, p.status, 38)) { ok = false; break; }
                uint8_t* sV = base_ptr + L::KV + s * L::STAGE_BYTES + TILE * HD * 2;
                const int first = pos_last + 1 - key0;                              // 1..63
                for (int i = first * 8 + r; i < TILE * 8; i += QROWS)
                    *reinterpret_cast<uint4*>(sV + i * 16) = make_uint4(0u, 0u, 0u, 0u);
                fence_async_smem();                                                 // before the MMA reads them
            }
            float mx = -INFINITY;
            if (live) {
                const bool need_mask = key0 + TILE - 1 > w_first || (p.window > 0 && key0 < w_first + 31 - p.window + 1) ||
                                       warp * 32 + 31 >= n_here;
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains, not one of 64
                if (need_mask) {                                                    // uniform over the warp
                    const int c_lo = lo_r - key0, c_hi = hi_r - key0;               // visible columns of this row
#pragma unroll
                    for (int c = 0; c < TILE; ++c) {
                        const float v = (c >= c_lo && c <= c_hi) ? __uint_as_float(sr[c]) : -INFINITY;
                        sr[c] = __float_as_uint(v);
                        mx4[c & 3] = fmaxf(mx4[c & 3], v);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < TILE; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
                }
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            }
            // raise the reference only when the maximum has outgrown it by more than 2^8
            const bool raise = mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * p.scale_log2 > 8.f);
            float corr = 1.f;
            if (raise) {
                corr = m_ref == -INFINITY ? 0.f : ex2((m_ref - mx) * p.scale_log2);
                l *= corr;
                m_ref = mx;
            }
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // O holds the tiles before this one: wait for the last of them, then rescale this lane
                if (!mbar_wait(pv_full((j - 1) & 1), ((j - 1) >> 1) & 1, p.status, 39)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int d0 = 0; d0 < HD; d0 += 32) {
                    uint32_t orow[32];
                    tmem_ld32(tmem_o + lane_addr + d0, orow);
#pragma unroll
                    for (int d = 0; d < 32; ++d) orow[d] = __float_as_uint(__uint_as_float(orow[d]) * corr);
                    tmem_st32(tmem_o + lane_addr + d0, orow);
                }
                tc_fence_before();
            }
            // P of two tiles ago has been read once its P V has retired
            if (j >= 2 && !mbar_wait(pv_full(b), ((j - 2) >> 1) & 1, p.status, 40)) { ok = false; break; }
            tc_fence_after();
            uint32_t w[32];                                                         // the row's P, two keys a word
            if (live) {
                const float nb = m_ref == -INFINITY ? 0.f : -m_ref * p.scale_log2;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < TILE; c += 2) {
                    const float e0 = ex2(fmaf(__uint_as_float(sr[c]), p.scale_log2, nb));
                    const float e1 = ex2(fmaf(__uint_as_float(sr[c + 1]), p.scale_log2, nb));
                    sum4[(c >> 1) & 3] += e0 + e1;
                    w[c >> 1] = pack_bf16(e0, e1);
                }
                l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) w[c] = 0u;
            }
            tmem_st32(tmem_p + lane_addr + b * (TILE / 2), w);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(b));
        }
        if (ok && !mbar_wait(pv_full((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, p.status, 41)) ok = false;
        tc_fence_after();
        if (ok && warp_valid) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = p.out + ((size_t)(q0 + r) * p.H + h) * HD;
#pragma unroll
            for (int d0 = 0; d0 < HD; d0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_o + lane_addr + d0, o);
                if (valid) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(o[8 * c]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + d0 + 8 * c) = v;
                    }
                }
            }
        }
    }
    if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(1000);    // copies in flight may still land
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
bool supported(int H, int G, int hd, int page_size) {
    if (hd != 64) return false;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return false;
    return G >= 1 && H % G == 0;
}
}  // namespace

extern "C" int tuff_attention_prefill_tc_supported(int H, int G, int hd, int page_size) {
    return supported(H, G, hd, page_size) ? 1 : 0;
}

// q: [n_tokens, H, hd] bf16 with row stride q_stride (elements; rows 16-byte aligned);
// k_pages/v_pages: [num_pages, G, page_size, hd] bf16; cu_q: [n_rows + 1] first token of each
// request's portion; positions: [n_tokens]; out: [n_tokens, H*hd] bf16.
extern "C" int tuff_attention_prefill_tc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                         long long num_pages, const int* block_table, int max_blocks, const int* positions,
                                         const int* cu_q, void* out, int* status, int n_tokens, int n_rows, int H, int G,
                                         int hd, int page_size, float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!supported(H, G, hd, page_size)) return TUFF_E_SIZE;
    if (((uintptr_t)q & 15) || (q_stride & 7) || ((uintptr_t)out & 15) || ((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127))
        return TUFF_E_ALIGN;
    CUtensorMap mk, mv;
    const long long rows = num_pages * G * page_size;
    if (!pool_map(&mk, k_pages, rows, hd, page_size) || !pool_map(&mv, v_pages, rows, hd, page_size)) return TUFF_E_ALIGN;
    TcAttnParams p{};
    p.q = (const bf16*)q; p.q_stride = q_stride; p.block_table = block_table; p.max_blocks = max_blocks; p.n_pages = num_pages;
    p.positions = positions; p.cu_q = cu_q; p.out = (bf16*)out; p.status = status;
    p.n_rows = n_rows; p.H = H; p.G = G; p.page_size = page_size; p.window = window;
    p.n_blocks = (n_tokens + QROWS - 1) / QROWS + n_rows;      // an upper bound on the blocks of all requests
    p.scale_log2 = scale * 1.4426950408889634f;
    const int smem = Smem<64>::TOTAL;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const int rc = launch_pdl(attn_prefill_tc_kernel<64>, dim3((unsigned)(p.n_blocks * H)), dim3(NUM_THREADS), smem, stream, mk, mv, p);
    return rc ? rc : launch_status();
}
