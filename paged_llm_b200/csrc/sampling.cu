// Sampling from float32 logits, one thread block per row: argmax, and the draw
// with temperature, top-k and top-p.
//
// The filter is the reference's (xiyiji/paged-llm pagedllm/sampler.py:17-29):
// logits / max(T, 1e-5); a token stays if fewer than top_k tokens are larger and
// if the probability mass of the larger tokens is <= top_p.  Instead of a sort,
// the two thresholds are found by a bit-wise search over the order-preserving
// integer image of the floats (32 counting passes each); tokens that tie with a
// threshold all stay.  The draw is argmax(logit/T + g), g = -log(-log u), which
// samples the softmax of the kept tokens; u comes from a counter-based stream
// u(seed, counter, token index) (splitmix64), so a request's draw does not
// depend on the rest of the batch.
#include "common.cuh"

__device__ __forceinline__ uint32_t ordered_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t counter, uint64_t i) {
    uint64_t x = seed + counter * 0x9E3779B97F4A7C15ull + i * 0xBF58476D1CE4E5B9ull;
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return ((float)(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

struct MaxIdx {
    float v;
    int i;
};
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ MaxIdx block_argmax(MaxIdx x, MaxIdx* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    if (lane == 0) red[warp] = x;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    MaxIdx t = threadIdx.x < nw ? red[threadIdx.x] : MaxIdx{-INFINITY, 0x7fffffff};
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx y;
            y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, y);
        }
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    t = red[0];
    __syncthreads();
    return t;
}

// A row is cut into ARGMAX_PARTS parts, one block each; a block packs its best (value, index)
// into 64 bits (order-preserving image of the float in the high word, ~index in the low word,
// so that of equal values the first index wins) and merges it with atomicMax.  The block of a
// row that finishes last unpacks the winner and leaves the cell and the counter zero.
constexpr int ARGMAX_PARTS = 16;

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, size_t row_stride,
                              unsigned long long* __restrict__ cells, unsigned int* __restrict__ counters) {
    __shared__ MaxIdx red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, part = blockIdx.y;
    const float* row = logits + (size_t)r * row_stride;
    const int per = ((V + ARGMAX_PARTS - 1) / ARGMAX_PARTS + 3) & ~3;
    const int lo = part * per, hi = min(V, lo + per);
    MaxIdx best{-INFINITY, 0x7fffffff};
    if ((row_stride & 3) == 0 && ((uintptr_t)logits & 15) == 0) {
#pragma unroll 2
        for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
            if (i + 3 < hi) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(row + i));
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (vv[e] > best.v || best.i == 0x7fffffff) best = MaxIdx{vv[e], i + e};
            } else {
                for (int e = 0; i + e < hi; ++e) {
                    const float v = __ldcg(row + i + e);
                    if (v > best.v || best.i == 0x7fffffff) best = MaxIdx{v, i + e};
                }
            }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float v = __ldcg(row + i);
            if (v > best.v || best.i == 0x7fffffff) best = MaxIdx{v, i};
        }
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) {
        if (best.i != 0x7fffffff) {
            const unsigned long long packed =
                ((unsigned long long)ordered_key(best.v) << 32) | (unsigned long long)(0xffffffffu - (unsigned)best.i);
            atomicMax(&cells[r], packed);
        }
        __threadfence();
        if (atomicAdd(&counters[r], 1u) == ARGMAX_PARTS - 1) {
            __threadfence();
            const unsigned long long w = atomicExch(&cells[r], 0ull);
            out[r] = w == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(w & 0xffffffffull));
            counters[r] = 0u;
        }
    }
}

// cells, counters: [rows] each, zero before the first call (the kernel leaves them zero).
PL_EXPORT int pl_argmax(const float* logits, int* out, int rows, int V, long long row_stride,
                        unsigned long long* cells, unsigned int* counters, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && V > 0 && row_stride >= V, "argmax: bad sizes rows=%d V=%d", rows, V);
    PL_CUDA(launch_pdl(argmax_kernel, dim3(rows, ARGMAX_PARTS), dim3(256), 0, stream, logits, out, V, (size_t)row_stride,
                       cells, counters));
    return 0;
}

__global__ void sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, size_t row_stride,
                              const float* __restrict__ temps, const int* __restrict__ top_ks,
                              const float* __restrict__ top_ps, const unsigned long long* __restrict__ seeds,
                              const unsigned long long* __restrict__ counters) {
    __shared__ MaxIdx red_mi[32];
    __shared__ float red_f[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temps[r];
    if (temp < 1e-5f) {                                       // greedy row in a mixed batch
        MaxIdx best{-INFINITY, 0x7fffffff};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > best.v || (v == best.v && i < best.i) || best.i == 0x7fffffff) best = MaxIdx{v, i};
        }
        best = block_argmax(best, red_mi);
        if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
        return;
    }
    const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
    const int top_k = top_ks[r];
    const float top_p = top_ps[r];
    uint32_t key_floor = 0;                                   // tokens with ordered_key >= key_floor stay

    if ((top_k > 0 && top_k < V) || top_p < 1.0f) {
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
        {
            MaxIdx m = block_argmax(MaxIdx{mx, (int)threadIdx.x}, red_mi);
            mx = m.v;
        }
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) z += expf(row[i] * inv_t - mx);
        z = block_sum(z, red_f);
        if (top_k > 0 && top_k < V) {
            uint32_t res = 0;                                 // largest key with count(key >= res) >= k
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t cand = res | (1u << bit);
                float cnt = 0.f;
                for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += ordered_key(row[i] * inv_t) >= cand ? 1.f : 0.f;
                cnt = block_sum(cnt, red_f);
                if (cnt >= (float)top_k) res = cand;
            }
            key_floor = res;
        }
        if (top_p < 1.0f) {
            uint32_t res = 0xFFFFFFFFu;                       // smallest key with mass above it <= top_p
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t cand = res & ~(1u << bit);
                float mass = 0.f;
                for (int i = threadIdx.x; i < V; i += blockDim.x) {
                    const float x = row[i] * inv_t;
                    if (ordered_key(x) > cand) mass += expf(x - mx);
                }
                mass = block_sum(mass, red_f);
                if (mass <= top_p * z) res = cand;
            }
            key_floor = max(key_floor, res);
        }
    }
    const uint64_t seed = seeds[r], counter = counters[r];
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = row[i] * inv_t;
        if (ordered_key(x) < key_floor) continue;
        const float u = uniform01(seed, counter, (uint64_t)i);
        const float score = x - logf(-logf(u));
        if (score > best.v || (score == best.v && i < best.i) || best.i == 0x7fffffff) best = MaxIdx{score, i};
    }
    best = block_argmax(best, red_mi);
    if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

PL_EXPORT int pl_sample(const float* logits, int* out, int rows, int V, long long row_stride, const float* temps,
                        const int* top_ks, const float* top_ps, const unsigned long long* seeds,
                        const unsigned long long* counters, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && V > 0 && row_stride >= V, "sample: bad sizes rows=%d V=%d", rows, V);
    sample_kernel<<<rows, 1024, 0, stream>>>(logits, out, V, (size_t)row_stride, temps, top_ks, top_ps, seeds, counters);
    PL_LAUNCHED("sample");
    return 0;
}
