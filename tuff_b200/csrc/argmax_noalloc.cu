// Greedy token choice without any allocation: see argmax_noalloc.h for who needs this and the
// rules.  The kernel is the several-blocks-per-row argmax of sampling.cu (each row cut into
// pieces, the block that finishes last merges the pieces in order, so the first maximum wins);
// what differs is where its working memory lives: in `g_scratch` below, a file-scope device
// array, instead of a buffer the caller's framework allocates.
#include "argmax_noalloc.h"
#include <math.h>
#include <mutex>

namespace {
constexpr int PARTS = 32;                                    // pieces per row
constexpr int MAX_ROWS = TUFF_ARGMAX_NOALLOC_MAX_ROWS;
constexpr int MAX_DEVICES = 64;

struct Scratch {
    float value[MAX_ROWS * PARTS];        // each piece's maximum
    int index[MAX_ROWS * PARTS];          // and where it is
    unsigned done[MAX_ROWS];              // pieces finished per row; must be zero when a call starts
};

// The working memory of every call on this GPU.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) Scratch g_scratch;

struct Best { float v; int i; };
__device__ __forceinline__ Best pick(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__global__ void __launch_bounds__(256)
argmax_noalloc_kernel(const float* __restrict__ logits, int V, Scratch* __restrict__ s, int* __restrict__ out) {
    __shared__ float shv[8];
    __shared__ int shi[8];
    __shared__ bool last;
    const int r = blockIdx.x, part = blockIdx.y;
    const int per = ((V + PARTS - 1) / PARTS + 3) & ~3;
    const int lo = part * per, hi = min(V, lo + per);
    const float* row = logits + (size_t)r * V;
    Best best{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v) { best.v = v; best.i = i; }           // ascending i: the first maximum stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        best = pick(best, Best{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { shv[warp] = best.v; shi[warp] = best.i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        Best b{-INFINITY, 0x7fffffff};
        for (int w = 0; w < 8; ++w) b = pick(b, Best{shv[w], shi[w]});
        s->value[r * PARTS + part] = b.v;
        s->index[r * PARTS + part] = b.i;
        __threadfence();
        last = atomicAdd(&s->done[r], 1u) == (unsigned)(PARTS - 1);
        if (last) {
            __threadfence();
            Best m{-INFINITY, 0x7fffffff};
            for (int q = 0; q < PARTS; ++q)
                m = pick(m, Best{__ldcg(&s->value[r * PARTS + q]), __ldcg(&s->index[r * PARTS + q])});
            out[r] = m.i == 0x7fffffff ? 0 : m.i;
            s->done[r] = 0;                                   // ready for the next call
        }
    }
}

// Device address of g_scratch per device, looked up once with that device current.
Scratch* scratch_of_current_device(int* err) {
    static Scratch* addr[MAX_DEVICES] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *err = (int)e; return nullptr; }
    if (dev < 0 || dev >= MAX_DEVICES) { *err = (int)cudaErrorInvalidDevice; return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess || !p) { *err = e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol; return nullptr; }
        addr[dev] = static_cast<Scratch*>(p);
    }
    *err = 0;
    return addr[dev];
}
}  // namespace

extern "C" int tuff_argmax_noalloc_max_rows(void) { return MAX_ROWS; }

extern "C" const char* tuff_argmax_noalloc_message(int code) {
    switch (code) {
        case 0: return "ok";
        case TUFF_ARGMAX_NOALLOC_E_ROWS:
            return "tuff_argmax_noalloc: more rows than its fixed working array serves (256); split the call";
        case TUFF_ARGMAX_NOALLOC_E_ARG:
            return "tuff_argmax_noalloc: null logits or out pointer, or a vocabulary of less than one token";
        default: return "tuff_argmax_noalloc: a CUDA runtime error (the code is a cudaError_t)";
    }
}

extern "C" int tuff_argmax_noalloc(const float* logits, int n_rows, int V, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!logits || !out || V < 1) return TUFF_ARGMAX_NOALLOC_E_ARG;
    if (n_rows > MAX_ROWS) return TUFF_ARGMAX_NOALLOC_E_ROWS;
    int err = 0;
    Scratch* s = scratch_of_current_device(&err);      // first call on a device: not inside a stream capture
    if (!s) return err;
    // The counters are zero after every completed call; clear them anyway, in stream order, so
    // that a call that was cut short (a failed launch earlier in the stream) cannot poison this one.
    cudaError_t e = cudaMemsetAsync(s->done, 0, sizeof(unsigned) * n_rows, stream);
    if (e != cudaSuccess) return (int)e;
    argmax_noalloc_kernel<<<dim3(n_rows, PARTS), 256, 0, stream>>>(logits, V, s, out);
    return (int)cudaGetLastError();
}
