// Sampling from float32 logits, one thread block per row: argmax, and the draw
// with temperature, top-k and top-p.
//
// The filter is the reference's (xiyiji/paged-llm pagedllm/sampler.py:17-29):
// logits / max(T, 1e-5); a token stays if fewer than top_k tokens are larger and
// if the probability mass of the larger tokens is <= top_p.  Instead of a sort,
// the two thresholds are found by a radix search over the order-preserving
// integer image of the floats: four passes of eight bits, each a histogram of the
// row (counts for top-k, probability mass for top-p) and a suffix sum over its 256
// bins; tokens that tie with a threshold all stay.  Mass is summed in fixed point
// (2^-40 units in 64-bit integers), so the sums do not depend on the order in
// which threads arrive.  The draw is argmax(logit/T + g), g = -log(-log u), which
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

// f(i, row[i]) for every token of a row, by all threads of the block; 16-byte loads where the row allows.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int V, bool vec, F f) {
    if (vec) {
        const int V4 = V & ~3;
#pragma unroll 2
        for (int i = threadIdx.x * 4; i < V4; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            f(i, v.x);
            f(i + 1, v.y);
            f(i + 2, v.z);
            f(i + 3, v.w);
        }
        for (int i = V4 + threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
    }
}

__global__ void sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, size_t row_stride,
                              const float* __restrict__ temps, const int* __restrict__ top_ks,
                              const float* __restrict__ top_ps, const unsigned long long* __restrict__ seeds,
                              const unsigned long long* __restrict__ counters) {
    __shared__ MaxIdx red_mi[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const bool vec = (row_stride & 3) == 0 && ((uintptr_t)logits & 15) == 0;
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

    const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.0f;
    if (use_k || use_p) {
        __shared__ unsigned int cnt[256], piece[3][256];
        __shared__ unsigned long long mass[256], total_mass;
        __shared__ unsigned int pick_k, pick_p, need_k, key_lo, key_hi;
        __shared__ unsigned long long above_p, limit_p;
        const int tid = threadIdx.x;
        if (tid == 0) {
            total_mass = 0ull;
            need_k = (unsigned)top_k;
            above_p = 0ull;
            key_lo = 0xFFFFFFFFu;
            key_hi = 0u;
        }
        __syncthreads();
        {
            uint32_t lo = 0xFFFFFFFFu, hi = 0u;
            for_each_logit(row, V, vec, [&](int, float v) {
                const uint32_t key = ordered_key(v * inv_t);
                lo = min(lo, key);
                hi = max(hi, key);
            });
            lo = __reduce_min_sync(0xffffffffu, lo);
            hi = __reduce_max_sync(0xffffffffu, hi);
            if ((tid & 31) == 0) {
                atomicMin(&key_lo, lo);
                atomicMax(&key_hi, hi);
            }
        }
        __syncthreads();
        // The search runs over a row's own span of keys: a key becomes its distance from the largest one, shifted
        // so that the span fills whole digits of eight bits, and turned around so that larger still means larger.
        // Its leading digit then spreads over the bins (the leading bits of the keys themselves are almost all alike).
        const uint32_t kmax = key_hi, span = key_hi - key_lo;
        const int bits = span == 0u ? 1 : 32 - __clz(span), digits = (bits + 7) / 8, lsh = 8 * digits - bits;
        const uint32_t full = digits == 4 ? 0xFFFFFFFFu : (1u << (8 * digits)) - 1u;
        auto spread = [&](uint32_t key) { return full - ((kmax - key) << lsh); };
        float mx;                                             // the float behind the largest key
        {
            const uint32_t bts = (kmax & 0x80000000u) ? (kmax & 0x7FFFFFFFu) : ~kmax;
            mx = __uint_as_float(bts);
        }
        // exp(x - max) in units of 2^-33.  A bin's mass is gathered in three 32-bit counters of 11 bits of the
        // value each (shared memory adds 32-bit integers natively, 64-bit ones by compare-and-swap: 3.4 times
        // slower here); each stays below 2^32 for up to 2^21 tokens.
        auto fixed_mass = [&](float x) { return __float2ull_rn(expf(x - mx) * 8589934592.0f); };
        if (use_p) {
            unsigned long long z = 0ull;
            for_each_logit(row, V, vec, [&](int, float v) { z += fixed_mass(v * inv_t); });
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
            if ((tid & 31) == 0) atomicAdd(&total_mass, z);
            __syncthreads();
            if (tid == 0) limit_p = (unsigned long long)((double)top_p * (double)total_mass);
        }
        uint32_t prefix_k = 0, prefix_p = 0;                  // the digits found so far, most significant first
        for (int digit = digits - 1; digit >= 0; --digit) {
            const int shift = 8 * digit;
            if (tid < 256) {
                cnt[tid] = 0u;
                piece[0][tid] = piece[1][tid] = piece[2][tid] = 0u;
            }
            __syncthreads();
            for_each_logit(row, V, vec, [&](int, float v) {
                const float x = v * inv_t;
                const uint32_t key = spread(ordered_key(x));
                const uint32_t high = digit == digits - 1 ? 0u : key >> (shift + 8);
                const uint32_t bin = (key >> shift) & 255u;
                if (use_k && high == prefix_k) atomicAdd(&cnt[bin], 1u);
                if (use_p && high == prefix_p) {
                    const unsigned long long q = fixed_mass(x);         // zero for the far tail: nothing to add
                    const unsigned p0 = (unsigned)(q & 0x7FFull), p1 = (unsigned)((q >> 11) & 0x7FFull), p2 = (unsigned)(q >> 22);
                    if (p0) atomicAdd(&piece[0][bin], p0);
                    if (p1) atomicAdd(&piece[1][bin], p1);
                    if (p2) atomicAdd(&piece[2][bin], p2);
                }
            });
            __syncthreads();
            if (tid < 256)
                mass[tid] = (unsigned long long)piece[0][tid] + ((unsigned long long)piece[1][tid] << 11) +
                            ((unsigned long long)piece[2][tid] << 22);
            __syncthreads();
            // inclusive suffix sums over the bins (bin b: everything in bins b..255), in place
            for (int off = 1; off < 256; off <<= 1) {
                unsigned int c = 0u;
                unsigned long long m = 0ull;
                if (tid < 256) {
                    c = cnt[tid] + (tid + off < 256 ? cnt[tid + off] : 0u);
                    m = mass[tid] + (tid + off < 256 ? mass[tid + off] : 0ull);
                }
                __syncthreads();
                if (tid < 256) {
                    cnt[tid] = c;
                    mass[tid] = m;
                }
                __syncthreads();
            }
            if (tid < 256) {
                // top-k: the largest bin with at least `need_k` tokens in it and above it
                const unsigned int c_here = cnt[tid], c_above = tid < 255 ? cnt[tid + 1] : 0u;
                if (use_k && c_here >= need_k && c_above < need_k) pick_k = (unsigned)tid | (c_above << 8);
                // top-p: the smallest bin with no more than the allowed mass above it
                const unsigned long long m_above = tid < 255 ? mass[tid + 1] : 0ull;
                const unsigned long long m_above_lower = mass[tid];          // what lies above bin tid - 1
                if (use_p && above_p + m_above <= limit_p && (tid == 0 || above_p + m_above_lower > limit_p))
                    pick_p = (unsigned)tid;
            }
            __syncthreads();
            if (use_k) prefix_k = (prefix_k << 8) | (pick_k & 255u);
            if (use_p) prefix_p = (prefix_p << 8) | pick_p;
            if (tid == 0) {
                if (use_k) need_k -= pick_k >> 8;             // the tokens above the chosen bin are in
                if (use_p) above_p += pick_p < 255u ? mass[pick_p + 1] : 0ull;
            }
            __syncthreads();
        }
        // prefix_k: the largest (spread) key with at least top_k keys >= it; prefix_p: the smallest one with mass
        // above it <= top_p (the reference's filter, pagedllm/sampler.py:22-29); back to keys of the row
        auto unspread = [&](uint32_t floor2) {
            const uint32_t dist = (full - floor2) >> lsh;
            return dist >= kmax ? 0u : kmax - dist;
        };
        if (use_k) key_floor = unspread(prefix_k);
        if (use_p) key_floor = max(key_floor, unspread(prefix_p));
    }
    const uint64_t seed = seeds[r], counter = counters[r];
    MaxIdx best{-INFINITY, 0x7fffffff};
    for_each_logit(row, V, vec, [&](int i, float v) {
        const float x = v * inv_t;
        if (ordered_key(x) < key_floor) return;
        const float u = uniform01(seed, counter, (uint64_t)i);
        const float score = x - logf(-logf(u));
        if (score > best.v || (score == best.v && i < best.i) || best.i == 0x7fffffff) best = MaxIdx{score, i};
    });
    best = block_argmax(best, red_mi);
    if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

PL_EXPORT int pl_sample(const float* logits, int* out, int rows, int V, long long row_stride, const float* temps,
                        const int* top_ks, const float* top_ps, const unsigned long long* seeds,
                        const unsigned long long* counters, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && V > 0 && V < (1 << 21) && row_stride >= V, "sample: bad sizes rows=%d V=%d", rows, V);
    sample_kernel<<<rows, 1024, 0, stream>>>(logits, out, V, (size_t)row_stride, temps, top_ks, top_ps, seeds, counters);
    PL_LAUNCHED("sample");
    return 0;
}
