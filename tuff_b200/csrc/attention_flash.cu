// bf16 attention over the paged cache on the tensor cores, fed by TMA.
//
//   tuff_attention_decode   few query tokens, long contexts: one CTA per (token, key/value
//                           head, slice of the keys); the query heads that share the
//                           key/value head form the 16-row side of mma.sync.m16n8k16, the
//                           CTA's warps take the key tiles of the slice in turn, and the
//                           slices' partial results (max, sum, weighted values) are merged
//                           by tuff_attention_combine in slice order.
//   tuff_attention_prefill  portions of prompts: one CTA per (block of query tokens,
//                           key/value head); each warp owns 16 tokens of one query head and
//                           all warps walk the same key tiles, causally bounded per row.
// Both read 64-key tiles of K and V through cp.async.bulk.tensor (one box per cache page,
// 128-byte swizzle) into a ring of shared-memory stages guarded by mbarriers; a producer
// warp runs ahead of the consumers.  Scores, the running maximum and sum and the output
// accumulate in fp32 (online softmax as in the reference's kernel, src/lfm25_gpu.cu:506-558;
// scale 1/sqrt(hd) :520, head-to-group map :518, causal bound :531).  The reference walks
// one contiguous fp32 cache with one block per head and one key at a time.
//
// Supported here: head size 64 or 128, pages of 8, 16, 32 or 64 tokens, up to 8 query heads
// per key/value head; the launchers refuse anything else (TUFF_E_SIZE) and the caller uses
// the plain kernel.  Keys outside a token's range (beyond its position, before its window)
// never reach the result: their scores are replaced, and their values zeroed, before use,
// so stale or never-written cache contents (even NaN) are harmless.
// Every mbarrier wait is bounded; a wait that runs out records a code in *status.
#include "sm100.cuh"
#include "index.cuh"

namespace {
constexpr int TILE = 64;                 // keys per tile

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Address of 16-byte chunk `chunk` (8 dims) of key row `row` in a tile stored by TMA with
// 128-byte swizzle: per 64-dim half, rows are 128 bytes apart and chunk c of row r sits at
// c ^ (r & 7).  Halves (head size 128) are TILE*128 bytes apart.
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)(chunk >> 3) * (TILE * 128) + (uint32_t)row * 128 + (uint32_t)(((chunk & 7) ^ (row & 7)) << 4);
}

template <int HD> struct Frag {
    static constexpr int KS = HD / 16;       // k-steps over the head size
    static constexpr int DT = HD / 8;        // 8-dim output tiles
};

// One warp, one 64-key tile: S = Q K^T (scaled), masks, online softmax update, O += P V.
//   key0          absolute index of the tile's first key
//   lo_a/hi_a     visible key range of the row held in c[0], c[1] (row `g`); lo_b/hi_b for row g+8
//   v_hi          keys beyond it have their values zeroed (they may never have been written)
template <int HD>
__device__ __forceinline__ void process_tile(uint32_t sK, uint32_t sV, const uint32_t (&qa)[Frag<HD>::KS][4],
                                             float (&o)[Frag<HD>::DT][4], float& m_a, float& m_b, float& l_a, float& l_b,
                                             int key0, int lo_a, int hi_a, int lo_b, int hi_b, int v_hi, float scale_log2,
                                             bool need_mask) {
    const int lane = threadIdx.x & 31, t = lane & 3;
    float s[TILE / 8][4];
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int q = 0; q < HD / 32; ++q) {
            uint32_t r[4];
            ldsm_x4(tile_addr(sK, nt * 8 + (lane & 7), 4 * q + (lane >> 3)), r);
            mma16816(s[nt], qa[2 * q], r[0], r[1]);
            mma16816(s[nt], qa[2 * q + 1], r[2], r[3]);
        }
    }
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = s[nt][e] * scale_log2;
            if (need_mask) {
                const int key = key0 + nt * 8 + 2 * t + (e & 1);
                const bool ok = (e < 2) ? (key >= lo_a && key <= hi_a) : (key >= lo_b && key <= hi_b);
                v = ok ? v : -INFINITY;
            }
            s[nt][e] = v;
        }
        mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float base_a = mn_a == -INFINITY ? 0.f : mn_a, base_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float corr_a = exp2f(m_a - base_a), corr_b = exp2f(m_b - base_b);     // exp2(-inf) = 0
    m_a = mn_a; m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t pa[TILE / 16][4];
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt) {
        const float p0 = exp2f(s[nt][0] - base_a), p1 = exp2f(s[nt][1] - base_a);
        const float p2 = exp2f(s[nt][2] - base_b), p3 = exp2f(s[nt][3] - base_b);
        sum_a += p0 + p1; sum_b += p2 + p3;
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int dt = 0; dt < Frag<HD>::DT; ++dt) {
        o[dt][0] *= corr_a; o[dt][1] *= corr_a; o[dt][2] *= corr_b; o[dt][3] *= corr_b;
    }
#pragma unroll
    for (int j = 0; j < TILE / 16; ++j) {
#pragma unroll
        for (int u = 0; u < Frag<HD>::DT / 2; ++u) {
            uint32_t r[4];
            const int m = lane >> 3;
            ldsm_x4_trans(tile_addr(sV, 16 * j + 8 * (m & 1) + (lane & 7), 2 * u + (m >> 1)), r);
            if (need_mask) {
                // r[0], r[2]: keys 16j+2t, 16j+2t+1 (low, high half); r[1], r[3]: keys 16j+8+2t, +1
                const int k0 = key0 + 16 * j + 2 * t;
                const uint32_t keep0 = (k0 <= v_hi ? 0x0000ffffu : 0u) | (k0 + 1 <= v_hi ? 0xffff0000u : 0u);
                const uint32_t keep1 = (k0 + 8 <= v_hi ? 0x0000ffffu : 0u) | (k0 + 9 <= v_hi ? 0xffff0000u : 0u);
                r[0] &= keep0; r[2] &= keep0; r[1] &= keep1; r[3] &= keep1;
            }
            mma16816(o[2 * u], pa[j], r[0], r[1]);
            mma16816(o[2 * u + 1], pa[j], r[2], r[3]);
        }
    }
}

struct AttnParams {
    const bf16* q; long long q_stride;
    const int* block_table; int max_blocks;
    long long n_pages;            // pages in the pool (read by a checked build only)
    const int* positions; const int* row_of_token; const int* cu_q;
    bf16* out;                       // [T, H*HD]
    float* part_o; float* part_ml;   // decode: [T, H, splits, HD] and [T, H, splits, 2]
    int* status;
    int n_tokens, n_rows, H, G, page_size, window, n_splits;
    float scale_log2;
};

// Loads one 64-key tile of K and V (its pages through the block table) into a stage.
template <int HD>
__device__ __forceinline__ void load_tile(const CUtensorMap* mk, const CUtensorMap* mv, uint32_t sK, uint32_t sV,
                                          uint32_t bar, const int* bt, int max_blocks, int tile, int g, int G,
                                          int page_size, long long n_pages, int* status) {
    mbar_expect_tx(bar, 2 * TILE * HD * 2);
    const int pages = TILE / page_size;
    for (int i = 0; i < pages; ++i) {
        const int blk = tile * pages + i;
        int page = blk < max_blocks ? ld_act(bt + blk) : -1;          // beyond the row's table: no page
        if (TUFF_CHECKED && page != -1 && !page_ok(page, n_pages)) {  // (a load outside the tensor is harmless: it reads zeros)
            bounds_fault(Bounds{0, n_pages, status}, TUFF_BOUNDS_PAGE);
            page = -1;
        }
        const int y = (page * G + g) * page_size;            // a missing page (-1) lies outside the tensor: zero fill
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
            const uint32_t off = (uint32_t)h * (TILE * 128) + (uint32_t)(i * page_size) * 128;
            tma_load_2d(sK + off, mk, bar, h * 64, y);
            tma_load_2d(sV + off, mv, bar, h * 64, y);
        }
    }
}

// ------------------------------------------------------------------ decode
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 4;
// Warp w takes tiles w, w + DEC_WARPS, ...: with as many stages as warps a stage always belongs to the same warp,
// which therefore never waits for a phase of its barrier two ahead of the one it last saw.
static_assert(DEC_STAGES == DEC_WARPS, "a stage must always be read by the same warp");

template <int HD>
__global__ void __launch_bounds__((DEC_WARPS + 1) * 32)
attn_decode_kernel(const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv, AttnParams p) {
    constexpr int STAGE_BYTES = 2 * TILE * HD * 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + DEC_STAGES * STAGE_BYTES;
    float* merge = reinterpret_cast<float*>(base_ptr + DEC_STAGES * STAGE_BYTES + 128);   // [warps][8 rows][HD + 2]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g_lane = lane >> 2, t = lane & 3;
    const int tok = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int HG = p.H / p.G;
    if (threadIdx.x == 0) {
        for (int s = 0; s < DEC_STAGES; ++s) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (DEC_STAGES + s), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_wait();                                   // everything below reads what earlier kernels wrote
    const int pos = ld_act(p.positions + tok);
    const int row = ld_act(p.row_of_token + tok);
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int tile_lo = lo / TILE, tile_hi = pos / TILE;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int per = (n_tiles + p.n_splits - 1) / p.n_splits;
    const int t_begin = tile_lo + split * per;
    const int n_local = max(0, min(per, tile_hi + 1 - t_begin));
    const int* bt = p.block_table + (size_t)row * p.max_blocks;
    __syncthreads();
    bool ok = true;
    float o[Frag<HD>::DT][4];
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
#pragma unroll
    for (int dt = 0; dt < Frag<HD>::DT; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

    if (warp == DEC_WARPS) {
        if (lane == 0) {
            for (int i = 0; i < n_local; ++i) {
                const int s = i % DEC_STAGES;
                if (!mbar_wait(bars + 8 * (DEC_STAGES + s), ((i / DEC_STAGES) & 1) ^ 1, p.status, 11)) { ok = false; break; }
                load_tile<HD>(&mk, &mv, base + s * STAGE_BYTES, base + s * STAGE_BYTES + TILE * HD * 2, bars + 8 * s, bt,
                              p.max_blocks, t_begin + i, g, p.G, p.page_size, p.n_pages, p.status);
            }
        }
    } else {
        // query fragments: rows 0..HG-1 are the group's heads, the rest of the 16 rows are zero
        uint32_t qa[Frag<HD>::KS][4];
        const bf16* qrow = p.q + (size_t)tok * p.q_stride + (size_t)(g * HG + g_lane) * HD;
#pragma unroll
        for (int kk = 0; kk < Frag<HD>::KS; ++kk) {
            qa[kk][0] = g_lane < HG ? ld_act_u32(qrow + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = g_lane < HG ? ld_act_u32(qrow + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][1] = 0u; qa[kk][3] = 0u;
        }
        for (int i = warp; i < n_local; i += DEC_WARPS) {
            const int s = i % DEC_STAGES;
            if (!mbar_wait(bars + 8 * s, (i / DEC_STAGES) & 1, p.status, 12)) { ok = false; break; }
            const int key0 = (t_begin + i) * TILE;
            const bool need_mask = key0 < lo || key0 + TILE - 1 > pos;
            process_tile<HD>(base + s * STAGE_BYTES, base + s * STAGE_BYTES + TILE * HD * 2, qa, o, m_a, m_b, l_a, l_b,
                             key0, lo, pos, lo, pos, pos, p.scale_log2, need_mask);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (DEC_STAGES + s));
        }
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        // rows 0..7 only (HG <= 8): m, l and the output row of this warp
        float* mine = merge + (size_t)(warp * 8 + g_lane) * (HD + 2);
#pragma unroll
        for (int dt = 0; dt < Frag<HD>::DT; ++dt) {
            mine[dt * 8 + 2 * t] = o[dt][0];
            mine[dt * 8 + 2 * t + 1] = o[dt][1];
        }
        if (t == 0) { mine[HD] = m_a; mine[HD + 1] = l_a; }
    }
    if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    pdl_launch_dependents();                      // the keys are read: the next kernel may start its prologue
    __syncthreads();
    // merge the warps' partial results in warp order
    for (int idx = threadIdx.x; idx < HG * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, merge[(size_t)(w * 8 + r) * (HD + 2) + HD]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* src = merge + (size_t)(w * 8 + r) * (HD + 2);
            const float f = src[HD] == -INFINITY ? 0.f : exp2f(src[HD] - M);
            L += src[HD + 1] * f;
            O += src[d] * f;
        }
        const int h = g * HG + r;
        if (p.n_splits == 1) {
            p.out[((size_t)tok * p.H + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            const size_t pi = ((size_t)tok * p.H + h) * p.n_splits + split;
            p.part_o[pi * HD + d] = O;
            if (d == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = L; }
        }
    }
}

template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int n_splits) {
    const size_t th = blockIdx.x;                      // token * H + head
    pdl_wait();
    pdl_launch_dependents();
    const float* ml = part_ml + th * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ld_act(ml + 2 * s));
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = ld_act(ml + 2 * s);
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
            L += ld_act(ml + 2 * s + 1) * f;
            O += ld_act(part_o + (th * n_splits + s) * HD + d) * f;
        }
        out[th * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
}

// ----------------------------------------------------------------- prefill
constexpr int PRE_WARPS = 8;
constexpr int PRE_STAGES = 3;

template <int HD>
__global__ void __launch_bounds__((PRE_WARPS + 1) * 32, HD <= 64 ? 2 : 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv, AttnParams p) {
    constexpr int STAGE_BYTES = 2 * TILE * HD * 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + PRE_STAGES * STAGE_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g_lane = lane >> 2, t = lane & 3;
    const int g = blockIdx.y;
    const int HG = p.H / p.G;
    const int QB = PRE_WARPS / HG;                // 16-token sub-blocks per CTA
    const int n_cons = HG * QB;                   // consumer warps that take part
    const int QTOK = 16 * QB;
    // which row and which block of its tokens is this CTA's?
    // later blocks of a row see more keys: they are started first, so the long ones do not trail
    int row = -1, blk = (int)gridDim.x - 1 - (int)blockIdx.x, q0 = 0, q1 = 0;
    for (int r = 0; r < p.n_rows; ++r) {
        const int a = p.cu_q[r], b = p.cu_q[r + 1];
        const int nb = (b - a + QTOK - 1) / QTOK;
        if (blk < nb) { row = r; q0 = a + blk * QTOK; q1 = b; break; }
        blk -= nb;
    }
    if (row < 0) return;                          // uniform over the CTA
    const int n_here = min(QTOK, q1 - q0);
    const int pos0 = p.positions[q0];             // positions of a row's tokens are consecutive
    const int pos_last = pos0 + n_here - 1;
    const int lo_cta = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int tile_lo = lo_cta / TILE, tile_hi = pos_last / TILE;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int* bt = p.block_table + (size_t)row * p.max_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PRE_STAGES; ++s) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (PRE_STAGES + s), n_cons); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool ok = true;
    if (warp == PRE_WARPS) {
        if (lane == 0) {
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i % PRE_STAGES;
                if (!mbar_wait(bars + 8 * (PRE_STAGES + s), ((i / PRE_STAGES) & 1) ^ 1, p.status, 21)) { ok = false; break; }
                load_tile<HD>(&mk, &mv, base + s * STAGE_BYTES, base + s * STAGE_BYTES + TILE * HD * 2, bars + 8 * s, bt,
                              p.max_blocks, tile_lo + i, g, p.G, p.page_size, p.n_pages, p.status);
            }
        }
    } else if (warp < n_cons) {
        const int hh = warp % HG, sub = warp / HG;
        const int h = g * HG + hh;
        const int tok_a = q0 + sub * 16 + g_lane, tok_b = tok_a + 8;       // the rows this lane's registers hold
        const bool va = tok_a < q1 && sub * 16 + g_lane < n_here, vb = tok_b < q1 && sub * 16 + g_lane + 8 < n_here;
        const int pos_a = pos0 + sub * 16 + g_lane, pos_b = pos_a + 8;
        const int hi_a = va ? pos_a : -1, hi_b = vb ? pos_b : -1;
        const int lo_a = (p.window > 0 && pos_a - p.window + 1 > 0) ? pos_a - p.window + 1 : 0;
        const int lo_b = (p.window > 0 && pos_b - p.window + 1 > 0) ? pos_b - p.window + 1 : 0;
        const int warp_hi = min(pos_last, pos0 + sub * 16 + 15);           // last key any row of this warp sees
        const int warp_lo = (p.window > 0 && pos0 + sub * 16 - p.window + 1 > 0) ? pos0 + sub * 16 - p.window + 1 : 0;
        const bool warp_live = sub * 16 < n_here;
        uint32_t qa[Frag<HD>::KS][4];
        const bf16* qa_row = p.q + (size_t)(va ? tok_a : q0) * p.q_stride + (size_t)h * HD;
        const bf16* qb_row = p.q + (size_t)(vb ? tok_b : q0) * p.q_stride + (size_t)h * HD;
#pragma unroll
        for (int kk = 0; kk < Frag<HD>::KS; ++kk) {
            qa[kk][0] = va ? *reinterpret_cast<const uint32_t*>(qa_row + 16 * kk + 2 * t) : 0u;
            qa[kk][1] = vb ? *reinterpret_cast<const uint32_t*>(qb_row + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = va ? *reinterpret_cast<const uint32_t*>(qa_row + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][3] = vb ? *reinterpret_cast<const uint32_t*>(qb_row + 16 * kk + 8 + 2 * t) : 0u;
        }
        float o[Frag<HD>::DT][4];
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
#pragma unroll
        for (int dt = 0; dt < Frag<HD>::DT; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i % PRE_STAGES;
            if (!mbar_wait(bars + 8 * s, (i / PRE_STAGES) & 1, p.status, 22)) { ok = false; break; }
            const int key0 = (tile_lo + i) * TILE;
            if (warp_live && key0 <= warp_hi && key0 + TILE - 1 >= warp_lo) {
                // masks are needed unless every row of the warp sees the whole tile
                const bool need_mask = key0 + TILE - 1 > pos0 + sub * 16 || (p.window > 0 && key0 < pos0 + sub * 16 + 15 - p.window + 1)
                                       || sub * 16 + 15 >= n_here;
                process_tile<HD>(base + s * STAGE_BYTES, base + s * STAGE_BYTES + TILE * HD * 2, qa, o, m_a, m_b, l_a, l_b,
                                 key0, lo_a, hi_a, lo_b, hi_b, pos_last, p.scale_log2, need_mask);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (PRE_STAGES + s));
        }
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (ok) {
            const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
            bf16* oa = p.out + ((size_t)tok_a * p.H + h) * HD;
            bf16* ob = p.out + ((size_t)tok_b * p.H + h) * HD;
#pragma unroll
            for (int dt = 0; dt < Frag<HD>::DT; ++dt) {
                if (va) *reinterpret_cast<uint32_t*>(oa + dt * 8 + 2 * t) = pack_bf16(o[dt][0] * ia, o[dt][1] * ia);
                if (vb) *reinterpret_cast<uint32_t*>(ob + dt * 8 + 2 * t) = pack_bf16(o[dt][2] * ib, o[dt][3] * ib);
            }
        }
    }
    if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();                               // no CTA leaves while copies may still land in its shared memory
}

// ------------------------------------------------------------------ host side
bool supported(int H, int G, int hd, int page_size) {
    if (hd != 64 && hd != 128) return false;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return false;
    if (G < 1 || H % G != 0 || H / G > 8) return false;
    return true;
}

template <typename K>
int set_smem(K kernel, int bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
}  // namespace

extern "C" int tuff_attention_flash_supported(int H, int G, int hd, int page_size) {
    return supported(H, G, hd, page_size) ? 1 : 0;
}

// How many key slices tuff_attention_decode uses for this batch, and the floats of workspace it
// needs (partial outputs, then maxima and sums).
extern "C" int tuff_attention_decode_splits(int n_tokens, int G, int max_seq_len) {
    const int tiles = (max_seq_len + TILE - 1) / TILE;
    if (const char* e = getenv("TUFF_ATTN_SPLITS")) { const int v = atoi(e); if (v > 0) return v < tiles ? v : tiles; }
    // Enough CTAs to cover the SMs twice; beyond what stays resident at once (three CTAs per SM),
    // a count that fills whole rounds: a last round that is nearly empty costs a full round.
    const int sms = sm_count();
    const int pairs = n_tokens * G, resident = 3 * sms;
    int want = (2 * sms + pairs - 1) / pairs;
    if (pairs * want > resident) {
        int best = want;
        double best_eff = 0.0;
        for (int s = want; s <= want + 1; ++s) {
            const int ctas = pairs * s, rounds = (ctas + resident - 1) / resident;
            const double eff = (double)ctas / ((double)rounds * resident);
            if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
        }
        want = best;
    }
    if (want > tiles) want = tiles;
    if (want > 16) want = 16;          // more slices than this only add merge work
    return want < 1 ? 1 : want;
}
extern "C" long long tuff_attention_decode_workspace_floats(int n_tokens, int H, int hd, int n_splits) {
    return n_splits <= 1 ? 0 : (long long)n_tokens * H * n_splits * (hd + 2);
}

// q: [n_tokens, H, hd] bf16 with row stride q_stride; k_pages/v_pages: [num_pages, G, page_size, hd] bf16;
// out: [n_tokens, H*hd] bf16.  workspace: floats as tuff_attention_decode_workspace_floats says.
extern "C" int tuff_attention_decode(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                     long long num_pages, const int* block_table, int max_blocks, const int* positions,
                                     const int* row_of_token, void* out, float* workspace, int n_splits, int* status,
                                     int n_tokens, int H, int G, int hd, int page_size, float scale, int window,
                                     cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!supported(H, G, hd, page_size) || n_splits < 1) return TUFF_E_SIZE;
    if (((uintptr_t)q & 3) || (q_stride & 1) || ((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return TUFF_E_ALIGN;
    CUtensorMap mk, mv;
    const long long rows = num_pages * G * page_size;
    if (!pool_map(&mk, k_pages, rows, hd, page_size) || !pool_map(&mv, v_pages, rows, hd, page_size)) return TUFF_E_ALIGN;
    AttnParams p{};
    p.q = (const bf16*)q; p.q_stride = q_stride; p.block_table = block_table; p.max_blocks = max_blocks; p.n_pages = num_pages;
    p.positions = positions; p.row_of_token = row_of_token; p.out = (bf16*)out; p.status = status;
    p.part_o = workspace; p.part_ml = workspace ? workspace + (size_t)n_tokens * H * n_splits * hd : nullptr;
    p.n_tokens = n_tokens; p.H = H; p.G = G; p.page_size = page_size; p.window = window; p.n_splits = n_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    if (n_splits > 1 && !workspace) return TUFF_E_SIZE;
    dim3 grid(n_tokens, G, n_splits);
    const int threads = (DEC_WARPS + 1) * 32;
    int rc;
    if (hd == 64) {
        const int smem = DEC_STAGES * 2 * TILE * 64 * 2 + 128 + DEC_WARPS * 8 * (64 + 2) * 4 + 1024;
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_decode_kernel<64>, smem))) return rc; set = true; }
        rc = launch_pdl(attn_decode_kernel<64>, grid, dim3(threads), smem, stream, mk, mv, p);
    } else {
        const int smem = DEC_STAGES * 2 * TILE * 128 * 2 + 128 + DEC_WARPS * 8 * (128 + 2) * 4 + 1024;
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_decode_kernel<128>, smem))) return rc; set = true; }
        rc = launch_pdl(attn_decode_kernel<128>, grid, dim3(threads), smem, stream, mk, mv, p);
    }
    if (rc || (rc = launch_status()) || n_splits == 1) return rc;
    if (hd == 64) rc = launch_pdl(attn_combine_kernel<64>, dim3(n_tokens * H), dim3(64), 0, stream, (const float*)p.part_o, (const float*)p.part_ml, p.out, n_splits);
    else rc = launch_pdl(attn_combine_kernel<128>, dim3(n_tokens * H), dim3(128), 0, stream, (const float*)p.part_o, (const float*)p.part_ml, p.out, n_splits);
    return rc ? rc : launch_status();
}

extern "C" int tuff_attention_prefill(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                      long long num_pages, const int* block_table, int max_blocks, const int* positions,
                                      const int* row_of_token, const int* cu_q, void* out, int* status, int n_tokens,
                                      int n_rows, int H, int G, int hd, int page_size, float scale, int window,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!supported(H, G, hd, page_size)) return TUFF_E_SIZE;
    if (((uintptr_t)q & 3) || (q_stride & 1) || ((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return TUFF_E_ALIGN;
    CUtensorMap mk, mv;
    const long long rows = num_pages * G * page_size;
    if (!pool_map(&mk, k_pages, rows, hd, page_size) || !pool_map(&mv, v_pages, rows, hd, page_size)) return TUFF_E_ALIGN;
    AttnParams p{};
    p.q = (const bf16*)q; p.q_stride = q_stride; p.block_table = block_table; p.max_blocks = max_blocks; p.n_pages = num_pages;
    p.positions = positions; p.row_of_token = row_of_token; p.cu_q = cu_q; p.out = (bf16*)out; p.status = status;
    p.n_tokens = n_tokens; p.n_rows = n_rows; p.H = H; p.G = G; p.page_size = page_size; p.window = window; p.n_splits = 1;
    p.scale_log2 = scale * 1.4426950408889634f;
    const int HG = H / G, QTOK = 16 * (PRE_WARPS / HG);
    dim3 grid((n_tokens + QTOK - 1) / QTOK + n_rows, G);       // an upper bound on the blocks of all rows
    const int threads = (PRE_WARPS + 1) * 32;
    int rc;
    if (hd == 64) {
        const int smem = PRE_STAGES * 2 * TILE * 64 * 2 + 128 + 1024;
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_prefill_kernel<64>, smem))) return rc; set = true; }
        attn_prefill_kernel<64><<<grid, threads, smem, stream>>>(mk, mv, p);
    } else {
        const int smem = PRE_STAGES * 2 * TILE * 128 * 2 + 128 + 1024;
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_prefill_kernel<128>, smem))) return rc; set = true; }
        attn_prefill_kernel<128><<<grid, threads, smem, stream>>>(mk, mv, p);
    }
    return launch_status();
}
