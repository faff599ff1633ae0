// Shared declarations of the kernel library: dtype codes, error reporting,
// conversions.  Every exported function is extern "C", takes raw device
// pointers, sizes and a CUDA stream, allocates nothing, and returns 0 or a
// non-zero code after storing a message that pl_last_error() returns.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define PL_EXPORT extern "C" __attribute__((visibility("default")))

enum PlDtype { PL_F32 = 0, PL_BF16 = 1 };

int pl_fail(const char* fmt, ...);

#define PL_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) return pl_fail(__VA_ARGS__); \
    } while (0)

#define PL_LAUNCHED(name)                                                        \
    do {                                                                         \
        cudaError_t e__ = cudaGetLastError();                                    \
        if (e__ != cudaSuccess) return pl_fail("%s: %s", name, cudaGetErrorString(e__)); \
    } while (0)

#define PL_CUDA(expr)                                                            \
    do {                                                                         \
        cudaError_t e__ = (expr);                                                \
        if (e__ != cudaSuccess) return pl_fail("%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum for up to 1024 threads; `red` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    t = red[0];
    __syncthreads();
    return t;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl may start
// while the kernel in front of it on the stream is still running; it must call
// pdl_wait() before it reads anything that kernel wrote and before it writes
// anything at all.  pdl_launch_dependents() lets the kernel behind start early.
// What a kernel does before pdl_wait() (fetching weights) overlaps the kernel in
// front.  Launched the ordinary way, both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool off = getenv("PAGED_LLM_B200_NO_PDL") != nullptr;     // ordinary launches, for measurements
    cfg.numAttrs = off ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Parameters of the paged attention kernels (both precisions).
struct AttnParams {
    const void* q;          // [T, q_stride] rows; head h of token t at t*q_stride + h*d
    const void* kv;         // one layer of a pool: [pages, 2, kv_heads, page_size, d]
    void* out;              // [T, out_stride]
    const int* block_table; // [S, bt_stride]
    const int* cu_q;        // [S+1]
    const int* k_lens;      // [S]
    const int4* work;       // items (request, tile | scratch base, split, splits); request < 0: none
    float* scratch;         // partial results of split items
    long long scratch_floats;
    int q_stride, out_stride, bt_stride;
    int n_work, max_splits;
    int nh, nkv, d, ps;
    int window;             // 0: none
    int is_small;           // items are (request, scratch base, split, splits), one tile per request
                            // (2: the same, and the items' key ranges are long: see the dispatch of the kernels)
    float scale;
    int ps_shift;           // log2(ps) if ps is a power of two, else -1
    unsigned int* counters; // [requests * kv_heads] zeros, or null: the block of a request's kv head that
                            // finishes last merges the splits itself (no separate merge kernel)
    int num_pages;          // pages in `kv` (0: unknown; kernels that need it step aside)
    int cluster;            // > 0: no work list; n_work requests of at most 16 rows each, every (request, kv head)
                            // is a thread-block cluster of this many blocks that split the keys between them
    // Score modifiers, both off by default (the Llama decoder uses neither).  With s = scale * q.k:
    float softcap;          // > 0: s = softcap * tanh(s / softcap)
    const float* slopes;    // [nh] or null: s += slopes[head] * (key position - query position), a bias that grows
                            // with the distance to the key; applied after the cap
    // Rotary positions inside the kernel (bfloat16 cluster form only; null: q, k, v are rotated and stored
    // already).  `q` then is the projection's output [T, (nh + 2 nkv) d] (q heads, k heads, v heads): queries
    // and the step's own keys are rotated over the whole head (pairs i, i + d/2) with the angles of this
    // table [rope_len, d/2] of (cos, sin), and the own keys and values are written to their page slots.
    const float2* rope_table;
    int rope_len;
    // A decode step padded to the size of its captured graph: rows [cu_q[pad_seqs], pad_to) of `out` belong to no
    // request (pad_seqs: the number of request slots, so cu_q[pad_seqs] is the number of real tokens, read on the
    // device because a replayed graph sees other lengths).  The first block of the split-context kernels zeroes
    // them, so that no fill kernel stands between two kernels of a layer.  pad_to == 0: nothing to do.
    int pad_seqs, pad_to;
};

// The score of one (query row, key) pair from the raw dot product, in natural-log units.
__device__ __forceinline__ float attn_score(const AttnParams& p, float dot, float slope, int key_pos, int query_pos) {
    float s = dot * p.scale;
    if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
    return s + slope * (float)(key_pos - query_pos);
}
