// Token selection from fp32 logits, one thread block per row.
//
// The options and their order are those of the reference's host sampler
// (src/sampler.c:99-230, defaults src/sampler.c:8-18):
//   temp <= 0   greedy: the first maximum wins (also src/lfm25_gpu.cu:691-695,711)
//   otherwise   repetition penalty over the recent tokens (one application per
//               occurrence; positive logits divided, others multiplied)
//               -> maximum -> min-p on (l - max)/temp >= ln(min_p)
//               -> top-k -> softmax -> top-p with renormalisation -> one draw.
// The reference sorts candidates on the host and walks the sorted list; here
// the k-th value and the nucleus edge are found by bisection over the ordered
// bit patterns of the scaled logits, equal values are admitted lowest index
// first, and the draw walks the kept tokens in vocabulary order.  The random
// number is a counter-based hash of (seed, request key, token index), so a
// request's draws do not depend on what else is in the batch.
#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform number in [0,1) with 24 bits, from (seed, request key, token index).
__device__ __forceinline__ float draw_uniform(unsigned long long seed, unsigned long long request_key,
                                              unsigned long long token_index) {
    unsigned long long z = mix64(seed + 0x9E3779B97F4A7C15ull * (request_key + 1ull));
    z = mix64(z ^ (token_index * 0xD1B54A32D192ED03ull + 0x8CB92BA72F3D8DD7ull));
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

template <typename T> __device__ __forceinline__ T warp_incl_scan(T v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

// Exclusive prefix over the block's threads (in thread order); `total` gets the sum.
template <typename T>
__device__ __forceinline__ T block_excl_scan(T v, T* sh /* 33 entries */, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = blockDim.x >> 5;
    T incl = warp_incl_scan(v);
    __syncthreads();
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        T w = lane < nwarp ? sh[lane] : (T)0;
        T wi = warp_incl_scan(w);
        sh[lane] = wi - w;
        if (lane == 31) sh[32] = wi;
    }
    __syncthreads();
    *total = sh[32];
    return sh[warp] + incl - v;
}

__device__ __forceinline__ int block_sum_int(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int t = lane < nwarp ? sh[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ int block_argmax(const float* __restrict__ row, int V, float* shv, int* shi) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = ld_act(row + i);
        if (v > best.v) { best.v = v; best.i = i; }        // ascending i: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { shv[warp] = best.v; shi[warp] = best.i; }
    __syncthreads();
    ArgMax b2{lane < nwarp ? shv[lane] : -INFINITY, lane < nwarp ? shi[lane] : 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, b2.v, o), __shfl_xor_sync(0xffffffffu, b2.i, o)};
        b2 = better(b2, other);
    }
    return b2.i == 0x7fffffff ? 0 : b2.i;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float shv[32];
    __shared__ int shi[32];
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int best = block_argmax(logits + (size_t)r * V, V, shv, shi);
    if (threadIdx.x == 0) out[r] = best;
}

// Greedy choice over a wide vocabulary with few rows: the row is cut into `n_parts` pieces, one
// block each; the block that finishes last for a row (a counter tells) merges the pieces' maxima
// in piece order, which keeps the first maximum, and resets the counter for the next call.
// scratch: [n_rows][n_parts] (value, index) pairs, then n_rows counters that are zero between calls.
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int V, int n_parts, float* __restrict__ part_v,
                    int* __restrict__ part_i, unsigned* __restrict__ counters, int* __restrict__ out) {
    __shared__ float shv[32];
    __shared__ int shi[32];
    __shared__ bool last;
    const int r = blockIdx.x, part = blockIdx.y;
    pdl_wait();
    const int per = ((V + n_parts - 1) / n_parts + 3) & ~3;
    const int lo = part * per, hi = min(V, lo + per);
    const float* row = logits + (size_t)r * V;
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = ld_act(row + i);
        if (v > best.v) { best.v = v; best.i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) { shv[warp] = best.v; shi[warp] = best.i; }
    __syncthreads();
    if (warp == 0) {
        ArgMax b2{lane < nwarp ? shv[lane] : -INFINITY, lane < nwarp ? shi[lane] : 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other{__shfl_xor_sync(0xffffffffu, b2.v, o), __shfl_xor_sync(0xffffffffu, b2.i, o)};
            b2 = better(b2, other);
        }
        if (lane == 0) {
            part_v[(size_t)r * n_parts + part] = b2.v;
            part_i[(size_t)r * n_parts + part] = b2.i;
            __threadfence();
            last = atomicAdd(&counters[r], 1u) == (unsigned)(n_parts - 1);
        }
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
        __threadfence();
        ArgMax b{-INFINITY, 0x7fffffff};
        for (int q = 0; q < n_parts; ++q) {
            ArgMax o{__ldcg(part_v + (size_t)r * n_parts + q), __ldcg(part_i + (size_t)r * n_parts + q)};
            b = better(b, o);
        }
        out[r] = b.i == 0x7fffffff ? 0 : b.i;
        counters[r] = 0;
    }
}

struct SampleRow {       // one per logits row, 48 bytes
    float temp, top_p, min_p, repeat_penalty;
    int top_k, n_recent;
    unsigned long long seed, request_key, token_index;
};

// Keeps, of the entries of `w` (scaled logits, -inf = dropped), those above the
// threshold key and the first `need_ties` entries equal to it; drops the rest.
__device__ void apply_threshold(float* w, int V, unsigned thr, int need_ties, int* shi) {
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
    int ties = 0;
    for (int i = lo; i < hi; ++i) ties += ordered_key(w[i]) == thr;
    int total;
    int rank = block_excl_scan<int>(ties, shi, &total);
    for (int i = lo; i < hi; ++i) {
        const unsigned k = ordered_key(w[i]);
        if (k < thr) w[i] = -INFINITY;
        else if (k == thr) { if (rank >= need_ties) w[i] = -INFINITY; ++rank; }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const SampleRow* __restrict__ rows,
              const int* __restrict__ recent, int max_recent, float* __restrict__ work,
              int* __restrict__ out) {
    __shared__ float shf[33];
    __shared__ int shi[33];
    __shared__ int sh_choice;
    const int r = blockIdx.x;
    const SampleRow p = rows[r];
    const float* row = logits + (size_t)r * V;
    if (!(p.temp > 0.f)) {
        const int best = block_argmax(row, V, shf, shi);
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    float* w = work + (size_t)r * V;
    for (int i = threadIdx.x; i < V; i += blockDim.x) w[i] = row[i];
    __syncthreads();
    if (threadIdx.x == 0 && p.repeat_penalty > 1.f) {
        for (int k = 0; k < p.n_recent; ++k) {
            const int tok = recent[(size_t)r * max_recent + k];
            if (tok >= 0 && tok < V) {
                const float l = w[tok];
                w[tok] = l > 0.f ? l / p.repeat_penalty : l * p.repeat_penalty;
            }
        }
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, w[i]);
    mx = block_max(mx, shf);
    const float inv_temp = 1.f / p.temp;
    const float floor_scaled = (p.min_p > 0.f && p.min_p < 1.f) ? logf(p.min_p) : -INFINITY;
    int kept = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float s = (w[i] - mx) * inv_temp;
        if (!(s >= floor_scaled)) s = -INFINITY;     // also drops NaN
        kept += s > -INFINITY;
        w[i] = s;
    }
    kept = block_sum_int(kept, shi);
    __syncthreads();

    if (p.top_k > 0 && kept > p.top_k) {
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = thr | (1u << bit);
            int c = 0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) c += ordered_key(w[i]) >= cand;
            c = block_sum_int(c, shi);
            if (c >= p.top_k) thr = cand;
        }
        int above = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) above += ordered_key(w[i]) > thr;
        above = block_sum_int(above, shi);
        apply_threshold(w, V, thr, p.top_k - above, shi);
    }

    float total = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) total += expf(w[i]);   // exp(-inf) = 0
    total = block_sum(total, shf);

    if (p.top_p > 0.f && p.top_p < 1.f) {
        const float want = p.top_p * total;
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = thr | (1u << bit);
            float mass = 0.f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float s = w[i];
                if (ordered_key(s) >= cand) mass += expf(s);
            }
            mass = block_sum(mass, shf);
            if (mass >= want) thr = cand;
        }
        float mass_above = 0.f;
        int ties = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float s = w[i];
            const unsigned k = ordered_key(s);
            if (k > thr) mass_above += expf(s);
            ties += k == thr;
        }
        mass_above = block_sum(mass_above, shf);
        ties = block_sum_int(ties, shi);
        const float p_thr = expf(key_value(thr));
        int need = p_thr > 0.f ? (int)ceilf((want - mass_above) / p_thr) : ties;
        need = max(1, min(need, ties));
        apply_threshold(w, V, thr, need, shi);
        total = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) total += expf(w[i]);
        total = block_sum(total, shf);
    }

    // One draw; the chosen token is the first, in vocabulary order, whose
    // cumulative weight reaches u * total.
    const float u = draw_uniform(p.seed, p.request_key, p.token_index);
    const float target = u * total;
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
    float mine = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float e = expf(w[i]);
        mine += e;
        if (e > 0.f) last_kept = i;
    }
    float all;
    const float before = block_excl_scan<float>(mine, shf, &all);
    if (threadIdx.x == 0) sh_choice = 0x7fffffff;
    __syncthreads();
    if (mine > 0.f && target <= before + mine) {     // later chunks match too; the lowest index wins
        float cum = before;
        int pick = last_kept;
        for (int i = lo; i < hi; ++i) {
            const float e = expf(w[i]);
            if (e > 0.f) { cum += e; if (target <= cum) { pick = i; break; } }
        }
        atomicMin(&sh_choice, pick);
    }
    __syncthreads();
    if (sh_choice == 0x7fffffff) {
        // rounding left the target beyond every chunk: take the last kept token
        int lk = last_kept;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) shi[threadIdx.x >> 5] = lk;
        __syncthreads();
        if (threadIdx.x == 0) {
            int b = 0;
            for (int i = 0; i < (int)(blockDim.x >> 5); ++i) b = max(b, shi[i]);
            sh_choice = b;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[r] = sh_choice;
}
}  // namespace

constexpr int ARGMAX_PARTS = 32;

// Bytes of scratch that tuff_argmax wants for up to n_rows rows (it must be zero when first used).
extern "C" long long tuff_argmax_scratch_bytes(int n_rows) { return (long long)n_rows * (ARGMAX_PARTS * 8 + 4); }

// scratch: null, or tuff_argmax_scratch_bytes(n_rows) bytes, zeroed once; with it a wide row is
// searched by several blocks.
extern "C" int tuff_argmax(const float* logits, int n_rows, int V, int* out, void* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V < 1) return TUFF_E_SIZE;
    if (scratch && V >= 8192 && n_rows * 4 <= 2 * sm_count()) {
        float* pv = (float*)scratch;
        int* pi = (int*)(pv + (size_t)n_rows * ARGMAX_PARTS);
        unsigned* cnt = (unsigned*)(pi + (size_t)n_rows * ARGMAX_PARTS);
        return launch_pdl(argmax_split_kernel, dim3(n_rows, ARGMAX_PARTS), dim3(256), 0, stream, logits, V, ARGMAX_PARTS,
                          pv, pi, cnt, out);
    }
    return launch_pdl(argmax_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, V, out);
}

// rows: n_rows records of 48 bytes (see SampleRow); recent: [n_rows, max_recent]
// token ids; work: [n_rows, V] floats of scratch.
extern "C" int tuff_sample(const float* logits, int n_rows, int V, const void* rows, const int* recent,
                           int max_recent, float* work, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V < 1) return TUFF_E_SIZE;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, (const SampleRow*)rows, recent, max_recent,
                                                         work, out);
    return launch_status();
}

extern "C" int tuff_sample_row_bytes() { return (int)sizeof(SampleRow); }
