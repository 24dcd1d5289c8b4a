// The decode-step matrix products: C[M,N] = A[M,K] * W[N,K]^T for M <= 8 tokens, with what
// surrounds them in a layer fused in, so that a layer is a few launches instead of a dozen.
//
// With so few tokens a product is a stream of W through the SMs; its time is the bytes of W over
// the HBM bandwidth plus what it costs to start and stop a kernel, and a decode step is seventy
// such products.  The kernel is therefore built so that the stream does not stop between two
// kernels:
//   * one CTA per SM owns an equal share of W's rows (13 or 14 of 2,048, not a multiple of a tile)
//     and walks all of K once per pass of at most 64 rows;
//   * a producer thread streams the share through a ring of shared-memory stages with TMA tile
//     loads (cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers; never multicast), one
//     load per stage: all rows, several 64-wide K blocks.  What is in flight lives in shared
//     memory, not in registers, so a CTA (8 warps) is small enough for the CTA of the next kernel
//     in the stream to be resident beside it;
//   * the weights depend on no earlier kernel, so the producer starts before griddepcontrol.wait:
//     launched with programmatic dependent launch, the kernel fills its ring while its predecessor
//     is still running, and finds its first weights in shared memory when it may read activations;
//   * six consumer warps take the 16-wide K steps of a stage in turn (warp w: steps w, w+6, ...),
//     feed mma.sync.m16n8k16 from shared memory with ldmatrix, and add their partial sums in warp
//     order through shared memory, so results do not depend on timing.
// The neighbouring small operations are done here too:
//   prologue  RMSNorm of the fp32 residual rows (reference src/lfm25_gpu.cu:207-262), once per CTA,
//             into shared memory in the layout ldmatrix reads;
//   epilogue  plain store / add into the fp32 residual (reference accum=true,
//             src/lfm25_engine.c:380,405,419) / silu(gate)*up over a stacked [gate; up] matrix
//             (src/lfm25_gpu.cu:583-618) / the gated short convolution over a stacked [B; C; x]
//             projection with the state roll (src/lfm25_gpu.cu:344-415, which fuses the same way
//             for one token).
// A norm that follows a product can be split over the two products around it, so that no CTA
// has to read and norm whole residual rows before its first MMA: the product that adds into the
// residual also writes bf16(x * w_norm) and, per CTA, the sum of squares of its columns of every
// row ("emit"); the product that consumes the norm reads those bf16 rows as its activations and
// multiplies its sums by rsqrt(mean square + eps) of the row in its epilogue ("row scale").  The
// scale is a factor per token, so it commutes with the product; the sums of squares are added in
// CTA order.
// The weights are the 16-row operand of the MMA and the tokens its 8 columns.  (More tokens go to the
// product that splits K over a thread-block cluster, gemm_skinny.cu: it is ahead from 9 tokens on.)
//
// Every wait on an mbarrier is bounded: if it runs out, the kernel records a code in *status
// (61 producer, 63 consumers), stops waiting, and runs to its end.
#include "sm100.cuh"
#include "index.cuh"
#include <algorithm>

namespace {
constexpr int CWARPS = 6;                    // consumer warps
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = 256;                 // + warp 6: the producer thread; warp 7 helps with the norm only
constexpr int MAX_STAGES = 16;
constexpr int NORM_BLOCKS = 2;               // the fused RMSNorm holds rows of up to NORM_BLOCKS * 1024 columns in registers
constexpr int MAX_ROWS = 64;                 // weight rows (all sets) of one pass
constexpr int BK = 64;                       // K elements of one tile: 128 bytes, one swizzle row
constexpr int PART_STRIDE = 16;              // floats per CTA in the buffer of partial sums of squares
constexpr int MAX_TAPS = 4;                  // taps of the convolution whose state is fetched ahead

enum : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_CONV = 3 };

struct StreamGemm {
    const void* a;            // NORM: fp32 residual [M, K] (lda); else unused (the activations come by TMA)
    const float* norm_w;      // RMSNorm weight [K]
    void* out;                // [M, ldc]
    int* status;
    long long lda, ldc;
    int M, N, K;
    float eps;
    int epi, out_dtype;
    int sets, set_block;      // row sets that are combined (1, 2: gate/up, 3: B/C/x); rows of a set that lie together
    const float* taps;        // convolution epilogue: [N, L]
    float* state;             // [slots, L-1, N]
    const int* slot_of_row;
    long long n_slots;        // slots of `state` (read by a checked build only)
    int L;
    // emit (with EPI_ACCUM): the new residual times this norm weight as bf16, and sums of squares per CTA
    const float* emit_w;      // [N] or null
    bf16* emit_xw;            // [M, N]
    float* emit_part;         // [CTAs, PART_STRIDE]
    // row scale: sums of squares per CTA of the rows of A as another product emitted them
    const float* scale_part;  // [scale_parts, PART_STRIDE] or null
    int scale_parts;
    float scale_eps;
    int pass_cols;            // output columns of a full pass (the TMA box holds this many rows of each set)
    int tile_rows;            // rows of a shared-memory tile: sets * pass_cols rounded up to 16
    int n_kb;                 // ceil(K / 64)
    int kb_per_stage, stages;
    int a_bytes;              // bytes of the activation region (whole normed rows, or a ring beside the weights')
    int red_stride;           // floats per (warp, token) row of the reduction buffer
    int k_inner;              // 1: K is not a multiple of 64; stages are single K blocks cut from a [rows, K] view
    int a_kb;                 // a_resident: K blocks of a row in shared memory (n_kb rounded up to odd)
    int a_resident;           // 1: the bf16 activations are loaded once, whole, and stay for all passes (else a ring beside the weights')
    long long* trace;         // null, or 8 time stamps per CTA of this launch (tuff_gemm_stream_trace)
};

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }
// Address of the 16-byte chunk `chunk` of the 128-byte line `line` of a tile written with the 128-byte
// swizzle (the tile starts on a 1024-byte boundary).  A stage's tile holds, row after row, the row's
// kb_per_stage consecutive 64-wide K blocks: line = row * kb_per_stage + block.  kb_per_stage is odd,
// so the lines of 8 consecutive rows at one block fall on 8 different swizzle phases and ldmatrix
// reads them without bank conflicts.
__device__ __forceinline__ uint32_t swz(uint32_t tile, int line, int chunk) {
    return tile + (uint32_t)line * 128u + (uint32_t)((chunk ^ (line & 7)) << 4);
}

// The stages of a CTA in the order they stream: its columns [c_lo, c_hi) in passes of at most
// pass_cols, each pass walking K in stages of kb_per_stage 64-wide blocks.  When the rows of a set
// lie in blocks of set_block columns (a [gate; up] matrix stacked in blocks), no CTA's columns
// reach from one block into the next: the CTAs are dealt out over the blocks.
struct StageCursor {
    int c, c_hi, pc, sb, st, spp;
    __device__ StageCursor(const StreamGemm& p, int stages_per_pass) {
        pc = p.pass_cols; sb = p.set_block; st = 0; spp = stages_per_pass;
        const long long b = blockIdx.x, G = gridDim.x;
        const int nblk = p.N / sb;
        if (nblk == 1) {                       // one block: every CTA an equal share of the columns
            c = (int)(b * p.N / G);
            c_hi = (int)((b + 1) * p.N / G);
        } else if (nblk >= G) {                // more blocks than CTAs: whole blocks
            c = (int)(b * nblk / G) * sb;
            c_hi = (int)((b + 1) * nblk / G) * sb;
        } else {                               // several CTAs share a block and none reaches into the next
            const int k = (int)(b * nblk / G);
            const int first = (int)((k * G + nblk - 1) / nblk), next = (int)(((k + 1) * G + nblk - 1) / nblk);
            const int j = (int)b - first, n_in = next - first;
            c = k * sb + j * sb / n_in;
            c_hi = k * sb + (j + 1) * sb / n_in;
        }
    }
    __device__ bool valid() const { return c < c_hi; }
    __device__ int width() const { return min(min(pc, c_hi - c), sb - c % sb); }
    __device__ void next_pass() { c += width(); st = 0; }
    __device__ void next() { if (++st == spp) next_pass(); }
};

// MT: tokens the MMA tile holds (8); NORM: RMSNorm prologue; NGT: groups of 16 weight rows in a pass.
template <int MT, bool NORM, int NGT>
__global__ void __launch_bounds__(THREADS, 2)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, StreamGemm p) {
    constexpr int A_TILE = MT * 128;                       // one 64-wide K block of the activations
    constexpr int NH = MT / 8;                             // MMAs per group of 16 weight rows and K step
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const int jb = p.kb_per_stage;
    const int w_stage = jb * p.tile_rows * 128;
    const int a_stage = jb * A_TILE;
    const int S = p.stages;
    const uint32_t ring = base;
    const uint32_t a_region = ring + (uint32_t)(S * w_stage);
    const uint32_t red_off = (uint32_t)(S * w_stage) + (uint32_t)p.a_bytes;
    float* red = reinterpret_cast<float*>(base_ptr + red_off);                         // [CWARPS][MT][red_stride]
    float* sq = red + CWARPS * MT * p.red_stride;                                      // [MT][pass_cols]: squares of a pass's new residual
    float* row_scale = sq + MT * p.pass_cols;                                          // [MT]
    const uint32_t bars = base + red_off + (uint32_t)((CWARPS * MT * p.red_stride + MT * p.pass_cols + MT) * 4);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
    const uint32_t a_full = bars + 8u * (2 * MAX_STAGES);           // the whole of A has arrived (a_resident)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp == CWARPS && lane == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), CWARPS); }
        mbar_init(a_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    long long* trace = p.trace ? p.trace + (size_t)blockIdx.x * 8 : nullptr;
    if (trace && threadIdx.x == 0) trace[0] = global_ns();
    __syncthreads();
    const int spp = (p.n_kb + jb - 1) / jb;                               // stages per pass
    const uint32_t box_bytes = (uint32_t)(p.sets * p.pass_cols) * 128u;

    // ---- the producer's two walks over the same stages: loads of weights into the ring, and loads of
    // activations beside them (only after griddepcontrol.wait).  One load per stage each: all sets, all
    // rows, kb_per_stage K blocks (blocks past the end of K are filled with zeros).
    StageCursor w_cur(p, spp), a_cur(p, spp);
    uint32_t n_w = 0, n_a = 0, w_phase = 1;        // w_phase: parity of the empty barrier's phase that frees the next slot
    int w_slot = 0, a_slot = 0;
    auto issue_w = [&]() {
        const int s = w_slot, kb0 = w_cur.st * jb;
        const int blk = w_cur.c / p.set_block, ci = w_cur.c - blk * p.set_block;
        mbar_expect_tx(full_bar(s), (uint32_t)jb * (box_bytes + ((NORM || p.a_resident) ? 0u : (uint32_t)A_TILE)));
        tma_load_5d(ring + (uint32_t)(s * w_stage), &map_w, full_bar(s), p.k_inner ? kb0 * BK : 0, p.k_inner ? 0 : kb0, ci, 0, blk);
        w_cur.next(); ++n_w;
        if (++w_slot == S) { w_slot = 0; w_phase ^= 1u; }
    };
    auto issue_a = [&]() {
        const int s = a_slot, kb0 = a_cur.st * jb;
        tma_load_5d(a_region + (uint32_t)(s * a_stage), &map_a, full_bar(s), p.k_inner ? kb0 * BK : 0, p.k_inner ? 0 : kb0, 0, 0, 0);
        a_cur.next(); ++n_a;
        if (++a_slot == S) a_slot = 0;
    };
    if (producer) {
        // Weights depend on no earlier kernel: fill the ring before the wait.
        if (trace) trace[6] = global_ns();
        while ((int)n_w < S && w_cur.valid()) issue_w();
    }
    __syncwarp();
    pdl_wait();
    if (trace && threadIdx.x == 0) trace[1] = global_ns();
    if (producer && !NORM) {
        if (p.a_resident) {
            // all of A in one load: it stays for every pass (a_kb blocks a row, an odd number: see swz)
            mbar_expect_tx(a_full, (uint32_t)(p.a_kb * A_TILE));
            tma_load_5d(a_region, &map_a, a_full, 0, 0, 0, 0, 0);
        } else {
            while (n_a < n_w) issue_a();
        }
    }
    // The next kernel in the stream may be scheduled once every CTA's producer is here: it sets itself
    // up and fetches its own weights beside this kernel, and waits for this kernel's end before it reads
    // anything that this kernel writes.  Not earlier: the loads of an SM are served in order, and the
    // next kernel's first weights would stand in front of this kernel's activations.
    if (producer) pdl_launch_dependents();

    const int K = p.K;
    if (NORM) {
        // RMSNorm of the M residual rows into shared memory as bf16, in 64-wide swizzled K blocks.  All
        // 256 threads share each row: a thread holds one float4 of every row of a half (8 rows) per
        // 1024 columns, so all of a half's loads are in flight at once and the values stay in registers.
        const float* x = reinterpret_cast<const float*>(p.a);
        float* part = red;                                       // [8 rows][8 warps] partial sums
        const int kpad = p.n_kb * BK;
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
                if (lane == 0) part[r * 8 + warp] = w;
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < THREADS / 32; ++w) tot += part[r * 8 + w];
                ss[r] = rsqrtf(tot / (float)K + p.eps);
            }
            __syncthreads();
#pragma unroll
            for (int cb = 0; cb < NORM_BLOCKS; ++cb) {
                const int k = cb * 1024 + threadIdx.x * 4;
                if (k < kpad) {
                    const float4 wn = k < K ? *reinterpret_cast<const float4*>(p.norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const int kb = k >> 6, chunk = (k & 63) >> 3, half = (k >> 2) & 1;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        if (r0 + r >= p.M) break;
                        const float4 a = v[cb][r];
                        const uint32_t lo = pack_bf16(a.x * ss[r] * wn.x, a.y * ss[r] * wn.y);
                        const uint32_t hi = pack_bf16(a.z * ss[r] * wn.z, a.w * ss[r] * wn.w);
                        const uint32_t dst = swz(a_region + (uint32_t)(kb * A_TILE), r0 + r, chunk) + (uint32_t)(half * 8);
                        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(dst), "r"(lo), "r"(hi) : "memory");
                    }
                }
            }
        }
        __syncthreads();
    }
    if (trace && threadIdx.x == 0) trace[2] = global_ns();

    if (warp >= CWARPS) {
        if (producer) {
            bool p_ok = true;
            while (w_cur.valid() && p_ok) {
                if (!mbar_wait(empty_bar(w_slot), w_phase, p.status, 61)) { p_ok = false; break; }
                issue_w();
                if (!NORM && !p.a_resident) issue_a();
            }
            if (trace) trace[7] = global_ns();
        }
        return;
    }

    // ---- consumers
    const int g = lane >> 2, t = lane & 3;
    // The factor of each row, when the rows come without their 1/rms: the sums of squares that the CTAs
    // of the emitting product wrote, added in CTA order (a lane takes every 32nd, then the lanes are
    // added by a fixed tree).  Warp w does rows w, w + 6, ...; read by the epilogue, after a barrier.
    // The loads are issued here and added up when the first pass ends, so nobody waits for them.
    constexpr int SP_TOKS = (16 + CWARPS - 1) / CWARPS, SP_PER_LANE = 8;          // up to 256 CTAs' parts
    float sp[SP_TOKS][SP_PER_LANE];
    if (p.scale_part) {
#pragma unroll
        for (int j = 0; j < SP_TOKS; ++j) {
            const int tok = warp + j * CWARPS;
#pragma unroll
            for (int i = 0; i < SP_PER_LANE; ++i)
                sp[j][i] = (tok < p.M && lane + 32 * i < p.scale_parts) ? ld_act(p.scale_part + (size_t)(lane + 32 * i) * PART_STRIDE + tok) : 0.f;
        }
    }
    // What the first pass's epilogue will read from global memory, asked for now: the residual value
    // that this thread adds to, or its channel's convolution state and taps.
    StageCursor cur(p, spp);
    float pre_res = 0.f, pre_emit_w = 0.f, pre_state[MAX_TAPS - 1], pre_taps[MAX_TAPS];
    int pre_slot = 0;
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) { pre_taps[j] = 0.f; if (j < MAX_TAPS - 1) pre_state[j] = 0.f; }
    {
        const int n_cols = cur.valid() ? cur.width() : 0;
        const int idx = threadIdx.x;
        if (idx < p.M * n_cols) {
            const int tok = idx / n_cols, col = cur.c + (idx - tok * n_cols);
            if (p.epi == EPI_ACCUM) pre_res = ld_act(reinterpret_cast<const float*>(p.out) + (size_t)tok * p.ldc + col);
            if (p.emit_w) pre_emit_w = p.emit_w[col];
            if (p.epi == EPI_CONV && p.L <= MAX_TAPS) {
                pre_slot = ld_act(p.slot_of_row + tok);
                if (check_slot(Bounds{p.M, p.n_slots, p.status}, pre_slot)) {
                    const float* stt = p.state + slot_elem(pre_slot, (size_t)(p.L - 1) * p.N);
#pragma unroll
                    for (int j = 0; j < MAX_TAPS; ++j) {
                        if (j < p.L) pre_taps[j] = p.taps[(size_t)col * p.L + j];
                        if (j < p.L - 1) pre_state[j] = ld_act(stt + (size_t)j * p.N + col);
                    }
                }
            }
        }
    }
    // Two sets of accumulators (8 tokens; registers allow it): the K steps of an iteration alternate
    // between them, so an MMA does not wait for the one before it; the sets are added when a pass ends.
    static_assert(MT == 8, "the tokens are the 8 columns of the MMA");
    constexpr int NU = 2;
    // K steps of one iteration: all their fragments are loaded before the first MMA, and a warp's share
    // of a stage is one iteration where registers allow, because an iteration costs a fixed 200 clocks
    // (ldmatrix, then the MMA pipeline) on top of its MMAs
    constexpr int US = NGT == 1 ? 6 : NGT == 2 ? 4 : 2;
    float acc[NU][NGT][NH][4];
    float row_sq = 0.f;                                           // emit: this CTA's sum of squares of row threadIdx.x
    bool ok = true, first_pass = true;
    int s = 0;
    uint32_t phase = 0, it = 0;
    const int rs = p.red_stride;
    // This lane's part of the ldmatrix addresses.  Weights: row lane & 15 of a group, the
    // chunk pair lane >> 4; 8 tokens: row lane & 7, the chunk pair (lane >> 3) & 1.  Groups of 16 rows lie
    // 16 * jb lines apart, a multiple of 8, so all groups of a K step share one swizzle phase.
    const int w_line0 = (lane & 15) * jb, w_half = lane >> 4;
    const uint32_t w_group = (uint32_t)(2048 * jb);
    const int ja = NORM ? 1 : p.a_resident ? p.a_kb : jb;                // lines from one row of A to the next
    const int a_line0 = (lane & 7) * ja, a_half = (lane >> 3) & 1;
    if (!NORM && p.a_resident && !mbar_test(a_full, 0)) ok = mbar_wait(a_full, 0, p.status, 63);
    for (; cur.valid(); cur.next_pass(), first_pass = false) {
        const int n_cols = cur.width();
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
            for (int i = 0; i < NGT; ++i)
#pragma unroll
                for (int h = 0; h < NH; ++h) acc[u][i][h][0] = acc[u][i][h][1] = acc[u][i][h][2] = acc[u][i][h][3] = 0.f;
        for (int st = 0; st < spp; ++st, ++it) {
            if (ok && !mbar_test(full_bar(s), phase)) ok = mbar_wait(full_bar(s), phase, p.status, 63);
            if (trace && threadIdx.x == 0 && it == 0) trace[3] = global_ns();
            const int kb0 = st * jb, n_steps = min(jb, p.n_kb - kb0) * 4;
            const uint32_t wt = ring + (uint32_t)(s * w_stage);
            // the normed rows lie as one 8- or 16-row tile per K block; the loaded ones as the weights do
            const uint32_t at = NORM ? a_region + (uint32_t)(kb0 * A_TILE) : p.a_resident ? a_region : a_region + (uint32_t)(s * a_stage);
            for (int step = warp; step < n_steps; step += US * CWARPS) {
                uint32_t tf[US][2], wf[US][NGT][4];
#pragma unroll
                for (int u = 0; u < US; ++u) {
                    const int stp = min(step + u * CWARPS, n_steps - 1);         // past the end: loaded again, not used
                    const int q = stp >> 2, kk = stp & 3;
                    const int al = a_line0 + (NORM ? 0 : p.a_resident ? kb0 + q : q), wl = w_line0 + q;
                    const uint32_t aa = at + (NORM ? (uint32_t)(q * A_TILE) : 0u) + (uint32_t)(al * 128) + (uint32_t)(((2 * kk + a_half) ^ (al & 7)) << 4);
                    const uint32_t wa = wt + (uint32_t)(wl * 128) + (uint32_t)(((2 * kk + w_half) ^ (wl & 7)) << 4);
                    ldsm_x2(aa, tf[u][0], tf[u][1]);
#pragma unroll
                    for (int i = 0; i < NGT; ++i) ldsm_x4(wa + (uint32_t)i * w_group, wf[u][i][0], wf[u][i][1], wf[u][i][2], wf[u][i][3]);
                }
#pragma unroll
                for (int u = 0; u < US; ++u) {
                    if (step + u * CWARPS >= n_steps) break;
#pragma unroll
                    for (int i = 0; i < NGT; ++i)          // 16 weight rows x 8 tokens
                        mma16816(acc[u % NU][i][0], wf[u][i][0], wf[u][i][1], wf[u][i][2], wf[u][i][3], tf[u][0], tf[u][1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));              // this warp has read the stage
            if (++s == S) { s = 0; phase ^= 1u; }
        }
        if (trace && threadIdx.x == 0) trace[4] = global_ns();
        // ---- the pass is complete: add the warps' partial sums in warp order and write out
#pragma unroll
        for (int i = 0; i < NGT; ++i) {
            // acc[.][i][0][0..1]: weight row 16 i + g, tokens 2t, 2t+1;  [2..3]: weight row 16 i + g + 8
            float* r = red + (size_t)(warp * MT + 2 * t) * rs + i * 16 + g;
            r[0] = acc[0][i][0][0] + acc[NU - 1][i][0][0]; r[rs] = acc[0][i][0][1] + acc[NU - 1][i][0][1];
            r[8] = acc[0][i][0][2] + acc[NU - 1][i][0][2]; r[rs + 8] = acc[0][i][0][3] + acc[NU - 1][i][0][3];
        }
        if (first_pass && p.scale_part) {
#pragma unroll
            for (int j = 0; j < SP_TOKS; ++j) {
                const int tok = warp + j * CWARPS;
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < SP_PER_LANE; ++i) a += sp[j][i];
                a = warp_sum(a);
                if (lane == 0 && tok < p.M) row_scale[tok] = rsqrtf(a / (float)K + p.scale_eps);
            }
        }
        consumer_sync();
        const int pc = p.pass_cols;
        for (int idx = threadIdx.x; idx < p.M * n_cols; idx += CTHREADS) {
            const int tok = idx / n_cols, c = idx - tok * n_cols;
            const int col = cur.c + c;
            const bool fetched = first_pass && idx == (int)threadIdx.x;   // this element's global inputs were asked for at the start
            const float scale = p.scale_part ? row_scale[tok] : 1.f;
            float v[3];
#pragma unroll
            for (int e = 0; e < 3; ++e) {
                float a = 0.f;
                if (e < p.sets) {
#pragma unroll
                    for (int w = 0; w < CWARPS; ++w) a += red[(size_t)(w * MT + tok) * rs + e * pc + c];
                }
                v[e] = a * scale;
            }
            const size_t o = (size_t)tok * p.ldc + col;
            auto store_bf16 = [&](float val) { reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(val); };
            if (p.epi == EPI_STORE) {
                if (p.out_dtype == TUFF_F32) reinterpret_cast<float*>(p.out)[o] = v[0];
                else store_bf16(v[0]);
            } else if (p.epi == EPI_ACCUM) {
                float* op = reinterpret_cast<float*>(p.out) + o;
                const float x_new = (fetched ? pre_res : ld_act(op)) + v[0];
                *op = x_new;
                if (p.emit_w) {
                    p.emit_xw[(size_t)tok * p.N + col] = __float2bfloat16_rn(x_new * (fetched ? pre_emit_w : p.emit_w[col]));
                    sq[tok * pc + c] = x_new * x_new;
                }
            } else if (p.epi == EPI_SWIGLU) {
                // gate and up rounded to bf16 first, as a separate projection would store them
                const float gq = bf16_round(v[0]), uq = bf16_round(v[1]);
                store_bf16(gq / (1.f + expf(-gq)) * uq);
            } else {
                // gated short convolution of one token per row; this CTA alone owns these channels
                const float b = bf16_round(v[0]), cg = bf16_round(v[1]), xg = bf16_round(v[2]);
                const float u = b * xg;
                const int L = p.L, d = p.N;
                const int slot = (fetched && L <= MAX_TAPS) ? pre_slot : ld_act(p.slot_of_row + tok);
                if (!check_slot(Bounds{p.M, p.n_slots, p.status}, slot)) continue;      // a checked build leaves this row alone
                float* stt = p.state + slot_elem(slot, (size_t)(L - 1) * d);
                float y = 0.f;
                if (fetched && L <= MAX_TAPS) {
#pragma unroll
                    for (int j = 0; j < MAX_TAPS - 1; ++j) {
                        if (j < L - 1) {
                            y = fmaf(pre_taps[j], pre_state[j], y);
                            if (j > 0) stt[(size_t)(j - 1) * d + col] = pre_state[j];
                        }
                    }
#pragma unroll
                    for (int j = 1; j < MAX_TAPS; ++j) if (j == L - 1) y = fmaf(pre_taps[j], u, y);
                } else {
                    for (int j = 0; j < L - 1; ++j) {
                        const float sv = ld_act(stt + (size_t)j * d + col);
                        y = fmaf(p.taps[(size_t)col * L + j], sv, y);
                        if (j > 0) stt[(size_t)(j - 1) * d + col] = sv;
                    }
                    y = fmaf(p.taps[(size_t)col * L + L - 1], u, y);
                }
                stt[(size_t)(L - 2) * d + col] = u;
                store_bf16(cg * y);
            }
        }
        consumer_sync();                                           // `red` is reused by the next pass
        if (p.emit_w && (int)threadIdx.x < p.M) {
            // this CTA's squares of row threadIdx.x, added in column order (`sq` is next written after
            // the next pass's first barrier, which this thread reaches only after this loop)
            for (int c = 0; c < n_cols; ++c) row_sq += sq[threadIdx.x * pc + c];
        }
    }
    if (p.emit_w && (int)threadIdx.x < p.M) p.emit_part[(size_t)blockIdx.x * PART_STRIDE + threadIdx.x] = row_sq;
    if (trace && threadIdx.x == 0) trace[5] = global_ns();
    if (!ok) {
        // A wait ran out.  Give copies that may still be in flight time to land before the shared
        // memory is released.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
}

// ------------------------------------------------------------------ host side
struct MapKey {
    const void* ptr; long long d0, d1, d2, d3, ld; int b1, b2;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && ld == o.ld && b1 == o.b1 && b2 == o.b2;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        for (long long v : {k.d0, k.d1, k.d2, k.d3, k.ld, (long long)k.b1, (long long)k.b2}) h = h * 1000003u ^ std::hash<long long>()(v);
        return h;
    }
};

// A tensor map over a K-major bf16 matrix seen as [blocks][sets][rows][K / 64][64] (row stride ld
// elements, a set `rows` rows after the one before, a block `sets * rows` rows after the one before),
// boxes of box_sets x box_rows x box_kb x 64: one load brings box_kb consecutive 64-wide K blocks of
// every row.  When K is no multiple of 64 the K blocks are not a dimension of their own (the last
// would reach into the next row): the view is [blocks][sets][rows][1][K] with boxes of one block,
// cut (and zero-filled) at K.  Maps depend on the address, so they are cached.
bool stream_map(CUtensorMap* out, const void* ptr, long long K, long long rows, long long sets, long long blocks,
                long long ld, int box_kb, int box_rows, int box_sets) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, K, rows, sets, blocks * 1024 + box_kb, ld, box_rows, box_sets};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    PFN_cuTensorMapEncodeTiled enc = encode_fn();
    if (!enc) return false;
    const bool inner = (K % BK) != 0;
    cuuint64_t gdim[5] = {(cuuint64_t)(inner ? K : BK), (cuuint64_t)(inner ? 1 : K / BK), (cuuint64_t)rows, (cuuint64_t)sets, (cuuint64_t)blocks};
    cuuint64_t gstride[4] = {(cuuint64_t)BK * 2, (cuuint64_t)ld * 2, (cuuint64_t)rows * ld * 2, (cuuint64_t)sets * rows * ld * 2};
    cuuint32_t box[5] = {(cuuint32_t)BK, (cuuint32_t)box_kb, (cuuint32_t)box_rows, (cuuint32_t)box_sets, 1u};
    cuuint32_t estride[5] = {1, 1, 1, 1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(ptr), gdim, gstride, box, estride,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// Tracing: while a buffer is set, every launch writes 8 time stamps (ns, %globaltimer) per CTA at
// buf[(launch * 256 + cta) * 8 + i]: 0 entry, 1 after griddepcontrol.wait, 2 after the norm prologue,
// 3 first stage arrived, 4 last pass's K walk done, 5 end, 6 first / 7 last weight load issued.
long long* g_trace = nullptr;
int g_trace_launches = 0, g_trace_capacity = 0;

int smem_target() {
    // Shared memory a CTA aims to stay under, so that the next kernel's CTA fits the SM beside it
    // (227 KB per SM).  TUFF_STREAM_SMEM (in KB) overrides it for sweeps.
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("TUFF_STREAM_SMEM");
        v = e ? atoi(e) * 1024 : 140 * 1024;
        if (v < 32 * 1024) v = 32 * 1024;
        if (v > 220 * 1024) v = 220 * 1024;
    }
    return v;
}

int stream_grid(int N) { return std::min(sm_count(), ceil_div(N, 8)); }

template <int MT, bool NORM, int NGT>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const StreamGemm& p, int grid, size_t smem, cudaStream_t stream) {
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<MT, NORM, NGT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // all of the SM's configurable memory as shared memory: the CTA of the next kernel must fit beside this one
        e = cudaFuncSetAttribute(gemm_stream_kernel<MT, NORM, NGT>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int rc = launch_pdl(gemm_stream_kernel<MT, NORM, NGT>, dim3(grid), dim3(THREADS), smem, stream, mw, ma, p);
    return rc ? rc : launch_status();
}

}  // namespace

// Number of CTAs tuff_gemm_stream launches for N output columns: the rows of a buffer of partial sums.
extern "C" int tuff_gemm_stream_grid(int N) { return N > 0 ? stream_grid(N) : 0; }

// epilogue: 0 store, 1 add into fp32 C, 2 swiglu (W is [2N, K]: gate rows then up rows), 3 gated
// short convolution (W is [3N, K]: B, C, x rows; one token per row of A; taps [N, L], state
// [slots, L-1, N], slot_of_row [M]).  norm_w: if not null, A is the fp32 residual [M, K] and is
// RMS-normed with this weight and eps first; else A is bf16 [M, K].
// Requirements: M <= 8, K % 8 == 0, ldw % 8 == 0, 16-byte aligned bases; bf16 A: lda % 8 == 0;
// fp32 A: lda % 4 == 0 and K <= 2048.  C is bf16 or fp32 (fp32 only for epilogue 1).
// set_block: for epilogues 2 and 3, how the row sets lie in W: 0 = stacked whole ([gate; up]), else
// blocks of that many rows of each set in turn (N a multiple of it).
// `status` is a device int that receives a non-zero code if a bounded wait ran out.
// emit_w (epilogue 1 only; else null): a norm weight [N]; the product then also writes
// emit_xw [M, N] = bf16(C * emit_w) and emit_part [tuff_gemm_stream_grid(N), 16]: per CTA and row the
// sum of squares of the CTA's columns of C.  scale_part (A bf16 only; else null): such a buffer
// with scale_parts rows for the rows of A; every result row r is multiplied by
// rsqrt(sum over CTAs of scale_part[.][r] / K + scale_eps) before the epilogue.
extern "C" int tuff_gemm_stream(const void* A, const float* norm_w, float eps, const void* W, void* C, int c_dtype,
                                int M, int N, int K, long long lda, long long ldw, long long ldc, int epilogue,
                                const float* taps, float* state, const int* slot_of_row, long long n_slots, int L, int set_block,
                                const float* emit_w, void* emit_xw, float* emit_part,
                                const float* scale_part, int scale_parts, float scale_eps,
                                int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 8 || K <= 0 || epilogue < 0 || epilogue > 3 || !status) return TUFF_E_SIZE;
    if ((K % 8) || (ldw % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TUFF_E_ALIGN;
    if (norm_w ? (lda % 4 != 0 || ((uintptr_t)norm_w & 15)) : (lda % 8 != 0)) return TUFF_E_ALIGN;
    if (epilogue == EPI_ACCUM && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if ((epilogue == EPI_SWIGLU || epilogue == EPI_CONV) && c_dtype != TUFF_BF16) return TUFF_E_DTYPE;
    if (c_dtype != TUFF_F32 && c_dtype != TUFF_BF16) return TUFF_E_DTYPE;
    if (epilogue == EPI_CONV && (L < 2 || !taps || !state || !slot_of_row)) return TUFF_E_SIZE;
    if (norm_w && K > NORM_BLOCKS * 1024) return TUFF_E_SIZE;      // a normed row must fit the prologue's registers
    if (set_block < 0 || (set_block && N % set_block)) return TUFF_E_SIZE;
    if (emit_w && (epilogue != EPI_ACCUM || !emit_xw || !emit_part)) return TUFF_E_SIZE;
    if (scale_part && (norm_w || scale_parts <= 0 || scale_parts > 256)) return TUFF_E_SIZE;
    const bool norm = norm_w != nullptr;
    constexpr int MT = 8;
    StreamGemm p{};
    p.a = A; p.norm_w = norm_w; p.out = C; p.status = status; p.lda = lda; p.ldc = ldc;
    p.M = M; p.N = N; p.K = K; p.eps = eps; p.epi = epilogue; p.out_dtype = c_dtype;
    p.sets = epilogue == EPI_SWIGLU ? 2 : epilogue == EPI_CONV ? 3 : 1;
    p.set_block = (set_block && p.sets > 1) ? set_block : N;
    p.taps = taps; p.state = state; p.slot_of_row = slot_of_row; p.n_slots = n_slots; p.L = L;
    p.emit_w = emit_w; p.emit_xw = (bf16*)emit_xw; p.emit_part = emit_part;
    p.scale_part = scale_part; p.scale_parts = scale_parts; p.scale_eps = scale_eps;
    // every SM an equal share of the columns, in passes of at most MAX_ROWS weight rows
    const int grid = stream_grid(N);
    const int nblk = N / p.set_block;
    // the most columns a CTA gets (see StageCursor): an equal share of all columns, of whole blocks, or of one block
    const int cols_max = nblk == 1 ? ceil_div(N, grid) : nblk >= grid ? ceil_div(nblk, grid) * p.set_block
                                                                       : ceil_div(p.set_block, grid / nblk);
    const int cap = MAX_ROWS / p.sets;
    const int n_pass = ceil_div(cols_max, cap);
    p.pass_cols = std::min(ceil_div(cols_max, n_pass), p.set_block);
    p.tile_rows = ceil_div(p.sets * p.pass_cols, 16) * 16;
    p.n_kb = ceil_div(K, BK);
    const int a_tile = MT * 128, tile_bytes = p.tile_rows * 128;
    // bf16 activations of up to 40 KB are loaded once and stay; longer rows stream beside the weights
    p.a_resident = (!norm && !(K % BK) && (long long)(ceil_div(K, BK) | 1) * a_tile <= 40 * 1024) ? 1 : 0;
    const int per_kb = tile_bytes + ((norm || p.a_resident) ? 0 : a_tile);
    // A stage holds an odd number of 64-wide K blocks (see swz), up to 24 KB, and no more than K has
    // (rounded up to odd); a K that is no multiple of 64 goes one block at a time.
    p.k_inner = (K % BK) ? 1 : 0;
    int jb = std::max(1, 24576 / per_kb);
    if (!(jb & 1)) --jb;
    jb = std::min(jb, 9);
    jb = std::min(jb, p.n_kb | 1);
    p.kb_per_stage = p.k_inner ? 1 : jb;
    const int stage_bytes = p.kb_per_stage * per_kb;
    p.red_stride = p.tile_rows + 4;
    const int red_bytes = (CWARPS * MT * p.red_stride + MT * p.pass_cols + MT) * 4;
    p.a_kb = p.n_kb | 1;
    const int a_whole = norm ? p.n_kb * a_tile : p.a_resident ? p.a_kb * a_tile : 0;
    const int fixed = a_whole + red_bytes + (2 * MAX_STAGES + 1) * 8 + 1024;
    // a CTA that streams megabytes runs long enough to have the SM to itself; the others leave room
    const long long share = (long long)cols_max * p.sets * K * 2;
    const int budget = share > (1 << 20) ? 200 * 1024 : smem_target() + (norm ? 8 * 1024 : 0);
    int S = (budget - fixed) / stage_bytes;
    S = std::max(2, std::min(S, MAX_STAGES));
    p.stages = S;
    p.a_bytes = (norm || p.a_resident) ? a_whole : S * p.kb_per_stage * a_tile;
    const size_t smem = (size_t)fixed + (size_t)S * stage_bytes;
    if (smem > 227 * 1024) return TUFF_E_SIZE;
    if (g_trace && g_trace_launches < g_trace_capacity && grid <= 256) p.trace = g_trace + (size_t)(g_trace_launches++) * 256 * 8;
    CUtensorMap mw, ma;
    if (!stream_map(&mw, W, K, p.set_block, p.sets, N / p.set_block, ldw, p.kb_per_stage, p.pass_cols, p.sets)) return TUFF_E_ALIGN;
    if (norm) ma = mw;                                            // not used
    else if (!stream_map(&ma, A, K, M, 1, 1, lda, p.a_resident ? p.a_kb : p.kb_per_stage, MT, 1)) return TUFF_E_ALIGN;
    const int ngt = p.tile_rows / 16;
#define TUFF_PICK(NGV)                                                                                         \
    (norm ? launch<8, true, NGV>(mw, ma, p, grid, smem, stream) : launch<8, false, NGV>(mw, ma, p, grid, smem, stream))
    const int rc = ngt == 1 ? TUFF_PICK(1) : ngt == 2 ? TUFF_PICK(2) : ngt == 3 ? TUFF_PICK(3) : TUFF_PICK(4);
#undef TUFF_PICK
    return rc;
}

// Sets (or, with null, clears) the trace buffer: room for `launches` launches of up to 256 CTAs,
// 8 int64 each.  Returns how many launches the previous buffer recorded.
extern "C" int tuff_gemm_stream_trace(long long* buf, int launches) {
    const int n = g_trace_launches;
    g_trace = buf; g_trace_capacity = buf ? launches : 0; g_trace_launches = 0;
    return n;
}
