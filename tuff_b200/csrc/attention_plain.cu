// Attention over a paged key/value cache: the plain kernels.
//
//   tuff_qk_norm_rope_write   per-head RMSNorm of q and k, NeoX rotation at the
//                             token's absolute position, rotated K and raw V
//                             stored in the request's pages
//                             (reference: src/lfm25_gpu.cu:420-501)
//   tuff_paged_attention_plain  causal softmax(q.k/sqrt(hd)) v over the cached
//                             keys 0..p (or the last `window` of them), grouped
//                             query heads sharing a key/value head
//                             (reference: src/lfm25_gpu.cu:506-578)
//
// The reference keeps one contiguous fp32 cache per sequence and is written for
// head size 64; here the cache is paged ([page][kv_head][slot][hd], looked up
// through a block table per batch row), the head size is any value up to 256,
// and one launch covers a batch that mixes prompt portions and decode tokens.
// Scores, softmax and the weighted sum are fp32.  Which warp takes which key
// depends on the key's index alone, so a token's result does not depend on how
// the batch was cut.
#include "common.cuh"
#include "index.cuh"

namespace {
constexpr int MAX_HD = 256;
constexpr int QKV_WARPS = 4;

// One warp per head at a time.  A lane owns element pairs: pair j < rot_dim/2 is the rotation pair
// (j, j + rot_dim/2); the pairs after those cover the unrotated rest of the head two by two.  So the
// norm needs one warp reduction and the rotation no exchange between lanes; a warp works on
// several heads at once (independent loads), since it is latency that limits this kernel.
// PPL: element pairs per lane (head size <= 64 * PPL).
template <typename T, int PPL>
__global__ void __launch_bounds__(QKV_WARPS * 32)
qk_norm_rope_write_kernel(T* __restrict__ qkv, const float* __restrict__ q_norm_w,
                          const float* __restrict__ k_norm_w, const float* __restrict__ inv_freq,
                          const int* __restrict__ positions, const int* __restrict__ row_of_token,
                          const int* __restrict__ block_table, int max_blocks,
                          T* __restrict__ k_pages, T* __restrict__ v_pages,
                          int H, int G, int hd, int rot_dim, int page_size, float eps, int write_kv, Bounds bounds) {
    constexpr int UNROLL = 4;                        // heads in flight per warp
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_dependents();
    const int pos = ld_act(positions + t);
    const int r = ld_act(row_of_token + t);
    const int n_heads = H + 2 * G;
    const int half = rot_dim >> 1, n_pairs = hd >> 1;
    T* base = qkv + (size_t)t * n_heads * hd;
    size_t page_base = 0;
    int in_page = 0;
    if (write_kv) {
        long long page = -1;
        if (check_row(bounds, r) && check_entry(bounds, pos, page_size, max_blocks)) {
            page = ld_act(block_table + (size_t)r * max_blocks + page_entry(pos, page_size));
            if (!check_page(bounds, page)) page = -1;
        }
        if (TUFF_CHECKED && page < 0) {
            write_kv = 0;                            // a checked build leaves the pages alone and says so
        } else {
            in_page = page_offset(pos, page_size);
            page_base = (size_t)page * G;
        }
    }
    // this lane's pairs: element indices and rotation
    int e1[PPL], e2[PPL];
    float rc[PPL], rs[PPL], wq1[PPL], wq2[PPL], wk1[PPL], wk2[PPL];
#pragma unroll
    for (int i = 0; i < PPL; ++i) {
        const int j = lane + 32 * i;
        e1[i] = j < half ? j : rot_dim + 2 * (j - half);
        e2[i] = j < half ? j + half : e1[i] + 1;
        rc[i] = 1.f; rs[i] = 0.f;
        if (j < half) sincosf((float)pos * inv_freq[j], &rs[i], &rc[i]);
        const bool ok = j < n_pairs;
        wq1[i] = (ok && q_norm_w) ? q_norm_w[e1[i]] : 1.f; wq2[i] = (ok && q_norm_w) ? q_norm_w[e2[i]] : 1.f;
        wk1[i] = (ok && k_norm_w) ? k_norm_w[e1[i]] : 1.f; wk2[i] = (ok && k_norm_w) ? k_norm_w[e2[i]] : 1.f;
    }
    // heads are dealt to (block.y, warp) in turn, UNROLL at a time
    const int stride = QKV_WARPS * gridDim.y;
    for (int h0 = blockIdx.y * QKV_WARPS + warp; h0 < n_heads; h0 += stride * UNROLL) {
        float a[UNROLL][PPL], b[UNROLL][PPL], ss[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int head = h0 + u * stride;
            ss[u] = 0.f;
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const bool ok = head < n_heads && lane + 32 * i < n_pairs;
                a[u][i] = ok ? ld_act(base + (size_t)head * hd + e1[i]) : 0.f;
                b[u][i] = ok ? ld_act(base + (size_t)head * hd + e2[i]) : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int i = 0; i < PPL; ++i) ss[u] = fmaf(a[u][i], a[u][i], fmaf(b[u][i], b[u][i], ss[u]));
            ss[u] = warp_sum(ss[u]);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int head = h0 + u * stride;
            if (head >= n_heads) break;
            const bool is_q = head < H, is_k = !is_q && head < H + G;
            T* x = base + (size_t)head * hd;
            if (!is_q && !is_k) {          // value head: copy to its page
                if (write_kv) {
                    T* dst = v_pages + ((page_base + (head - H - G)) * page_size + in_page) * hd;
#pragma unroll
                    for (int i = 0; i < PPL; ++i)
                        if (lane + 32 * i < n_pairs) { dst[e1[i]] = from_f32<T>(a[u][i]); dst[e2[i]] = from_f32<T>(b[u][i]); }
                }
                continue;
            }
            const bool normed = is_q ? q_norm_w != nullptr : k_norm_w != nullptr;
            const float scale = normed ? rsqrtf(ss[u] / (float)hd + eps) : 1.f;
            T* dst = (is_k && write_kv) ? k_pages + ((page_base + (head - H)) * page_size + in_page) * hd : nullptr;
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                if (lane + 32 * i >= n_pairs) break;
                const float v1 = a[u][i] * scale * (is_q ? wq1[i] : wk1[i]);
                const float v2 = b[u][i] * scale * (is_q ? wq2[i] : wk2[i]);
                const float o1 = v1 * rc[i] - v2 * rs[i];          // identity for the unrotated pairs
                const float o2 = v1 * rs[i] + v2 * rc[i];
                x[e1[i]] = from_f32<T>(o1);
                x[e2[i]] = from_f32<T>(o2);
                if (dst) { dst[e1[i]] = from_f32<T>(o1); dst[e2[i]] = from_f32<T>(o2); }
            }
        }
    }
}

constexpr int ATT_WARPS = 4;
constexpr int MAX_PER_LANE = MAX_HD / 32;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_plain_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k_pages,
                             const T* __restrict__ v_pages, const int* __restrict__ block_table,
                             int max_blocks, const int* __restrict__ positions,
                             const int* __restrict__ row_of_token, T* __restrict__ out,
                             int H, int G, int hd, int page_size, float scale, int window, Bounds bounds) {
    __shared__ float sh_acc[ATT_WARPS][MAX_HD];
    __shared__ float sh_m[ATT_WARPS], sh_l[ATT_WARPS];
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (H / G);
    const int pos = positions[t];
    const int r = row_of_token[t];
    if (!check_row(bounds, r)) return;               // the same for the whole block
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* bt = block_table + (size_t)r * max_blocks;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        qv[i] = e < hd ? to_f32(qp[e]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += ATT_WARPS) {
        if (!check_entry(bounds, j, page_size, max_blocks)) continue;     // j is the same for the whole warp
        const int page = bt[page_entry(j, page_size)];
        if (!check_page(bounds, page)) continue;
        const size_t off = page_elem(page, g, page_offset(j, page_size), G, page_size, hd);
        const T* kp = k_pages + off;
        const T* vp = v_pages + off;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < hd) s = fmaf(qv[i], to_f32(kp[e]), s);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);     // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < hd) acc[i] = acc[i] * corr + p * to_f32(vp[e]);
        }
        m = m_new;
    }
    if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < hd) sh_acc[warp][e] = acc[i];
    }
    __syncthreads();
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) m_all = fmaxf(m_all, sh_m[w]);
    float l_all = 0.f;
    float f[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        f[w] = sh_l[w] > 0.f ? expf(sh_m[w] - m_all) : 0.f;
        l_all += sh_l[w] * f[w];
    }
    T* op = out + ((size_t)t * H + h) * hd;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += sh_acc[w][e] * f[w];
        op[e] = from_f32<T>(o / l_all);
    }
}
}  // namespace

// qkv [n_tokens, (H+2G)*hd] is updated in place: q heads normed and rotated, k
// heads too (and copied to the pages), v heads copied to the pages.
// q_norm_w / k_norm_w may be null (no norm); rot_dim = 0 means no rotation;
// write_kv = 0 leaves the pages alone.
extern "C" int tuff_qk_norm_rope_write(void* qkv, int dtype, const float* q_norm_w, const float* k_norm_w,
                                       const float* inv_freq, const int* positions, const int* row_of_token,
                                       const int* block_table, int max_blocks, void* k_pages, void* v_pages,
                                       int n_tokens, int H, int G, int hd, int rot_dim, int page_size,
                                       float eps, int write_kv, long long table_rows, long long n_pages, int* status,
                                       cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd < 2 || hd > MAX_HD || (hd & 1) || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || G < 0 || H < 0) return TUFF_E_SIZE;
    if (write_kv && page_size < 1) return TUFF_E_SIZE;
    // few tokens: spread a token's heads over several blocks so that the launch fills more SMs
    const int n_heads = H + 2 * G;
    int per_token = n_tokens >= 512 ? 1 : ceil_div(n_heads, QKV_WARPS);
    if (per_token > 65535) per_token = 65535;
    dim3 grid(n_tokens, per_token);
#define QK_GO(T, PPL) return launch_pdl(qk_norm_rope_write_kernel<T, PPL>, grid, dim3(QKV_WARPS * 32), 0, stream, \
        (T*)qkv, q_norm_w, k_norm_w, inv_freq, positions, row_of_token, block_table, max_blocks, \
        (T*)k_pages, (T*)v_pages, H, G, hd, rot_dim, page_size, eps, write_kv, Bounds{table_rows, n_pages, status})
    if (dtype == TUFF_F32) {
        if (hd <= 64) QK_GO(float, 1); else if (hd <= 128) QK_GO(float, 2); else QK_GO(float, 4);
    } else if (dtype == TUFF_BF16) {
        if (hd <= 64) QK_GO(bf16, 1); else if (hd <= 128) QK_GO(bf16, 2); else QK_GO(bf16, 4);
    }
#undef QK_GO
    return TUFF_E_DTYPE;
}

// q: [n_tokens, H, hd] with a row stride of q_stride elements; out: [n_tokens, H*hd].
extern "C" int tuff_paged_attention_plain(const void* q, long long q_stride, const void* k_pages,
                                          const void* v_pages, int dtype, const int* block_table, int max_blocks,
                                          const int* positions, const int* row_of_token, void* out,
                                          int n_tokens, int H, int G, int hd, int page_size, float scale,
                                          int window, long long table_rows, long long n_pages, int* status,
                                          cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd < 1 || hd > MAX_HD || G < 1 || H % G != 0 || page_size < 1 || H > 65535) return TUFF_E_SIZE;
    dim3 grid(n_tokens, H);
    if (dtype == TUFF_F32)
        paged_attention_plain_kernel<float><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table, max_blocks,
            positions, row_of_token, (float*)out, H, G, hd, page_size, scale, window, Bounds{table_rows, n_pages, status});
    else if (dtype == TUFF_BF16)
        paged_attention_plain_kernel<bf16><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const bf16*)q, q_stride, (const bf16*)k_pages, (const bf16*)v_pages, block_table, max_blocks,
            positions, row_of_token, (bf16*)out, H, G, hd, page_size, scale, window, Bounds{table_rows, n_pages, status});
    else
        return TUFF_E_DTYPE;
    return launch_status();
}
