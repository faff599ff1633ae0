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
#include <cooperative_groups.h>

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

// f(i, row[i]) for the tokens [lo, hi) of a row (lo a multiple of 4), by all threads of the block; 16-byte loads
// where the row allows.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int lo, int hi, bool vec, F f) {
    if (vec) {
        const int hi4 = lo + ((hi - lo) & ~3);
#pragma unroll 2
        for (int i = lo + threadIdx.x * 4; i < hi4; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            f(i, v.x);
            f(i + 1, v.y);
            f(i + 2, v.z);
            f(i + 3, v.w);
        }
        for (int i = hi4 + threadIdx.x; i < hi; i += blockDim.x) f(i, row[i]);
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) f(i, row[i]);
    }
}

// What the blocks that share a row read of one another (through distributed shared memory).
struct SampleShared {
    unsigned int cnt[256], piece[3][256];      // this block's histogram of the digit at hand
    unsigned int key_lo, key_hi;               // smallest and largest key of its part of the row
    unsigned long long z;                      // mass of its part of the row
    float best_v;                              // its best candidate of the draw
    int best_i;
};

// One row per block (CL == 1), or per thread-block cluster of CL blocks that take a part of the row each (large
// vocabularies: a block alone needs seven sweeps over half a megabyte).  Every block of a cluster adds up the
// others' histograms itself and finds the same thresholds; sums are integers, so the result does not depend on
// the split.
template <int CL>
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V,
                                                      size_t row_stride, const float* __restrict__ temps,
                                                      const int* __restrict__ top_ks, const float* __restrict__ top_ps,
                                                      const unsigned long long* __restrict__ seeds,
                                                      const unsigned long long* __restrict__ counters) {
    namespace cg = cooperative_groups;
    __shared__ MaxIdx red_mi[32];
    __shared__ SampleShared sh;
    const int tid = threadIdx.x;
    int r = blockIdx.x, rank = 0;
    if constexpr (CL > 1) {
        rank = (int)cg::this_cluster().block_rank();
        r = blockIdx.x / CL;
    }
    auto peer = [&](int k) -> const SampleShared* {
        if constexpr (CL > 1) return cg::this_cluster().map_shared_rank(&sh, k);
        else return &sh;
    };
    auto sync_row = [&]() {
        if constexpr (CL > 1) cg::this_cluster().sync();
        else __syncthreads();
    };
    const float* row = logits + (size_t)r * row_stride;
    const bool vec = (row_stride & 3) == 0 && ((uintptr_t)logits & 15) == 0;
    const int per = ((V + CL - 1) / CL + 3) & ~3;
    const int lo = min(V, rank * per), hi = min(V, lo + per);        // this block's part of the row
    // the best of the blocks' best candidates: first index among equals; nobody leaves before it was read
    auto finish = [&](MaxIdx best) {
        best = block_argmax(best, red_mi);
        if (tid == 0) {
            sh.best_v = best.v;
            sh.best_i = best.i;
        }
        sync_row();
        if (rank == 0 && tid == 0) {
            MaxIdx b{sh.best_v, sh.best_i};
            for (int k = 1; k < CL; ++k) b = better(b, MaxIdx{peer(k)->best_v, peer(k)->best_i});
            out[r] = b.i == 0x7fffffff ? 0 : b.i;
        }
        if constexpr (CL > 1) sync_row();
    };
    const float temp = temps[r];
    if (temp < 1e-5f) {                                       // greedy row in a mixed batch
        MaxIdx best{-INFINITY, 0x7fffffff};
        for_each_logit(row, lo, hi, vec, [&](int i, float v) {
            if (v > best.v || (v == best.v && i < best.i) || best.i == 0x7fffffff) best = MaxIdx{v, i};
        });
        finish(best);
        return;
    }
    const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
    const int top_k = top_ks[r];
    const float top_p = top_ps[r];
    uint32_t key_floor = 0;                                   // tokens with ordered_key >= key_floor stay

    const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.0f;
    if (use_k || use_p) {
        __shared__ unsigned int cnt_all[256], warp_cnt[8];
        __shared__ unsigned long long mass[256], warp_mass[8];
        __shared__ unsigned int pick_k, pick_p, need_k;
        __shared__ unsigned long long above_p, limit_p;
        if (tid == 0) {
            sh.z = 0ull;
            need_k = (unsigned)top_k;
            above_p = 0ull;
            sh.key_lo = 0xFFFFFFFFu;
            sh.key_hi = 0u;
        }
        __syncthreads();
        {
            uint32_t klo = 0xFFFFFFFFu, khi = 0u;
            for_each_logit(row, lo, hi, vec, [&](int, float v) {
                const uint32_t key = ordered_key(v * inv_t);
                klo = min(klo, key);
                khi = max(khi, key);
            });
            klo = __reduce_min_sync(0xffffffffu, klo);
            khi = __reduce_max_sync(0xffffffffu, khi);
            if ((tid & 31) == 0) {
                atomicMin(&sh.key_lo, klo);
                atomicMax(&sh.key_hi, khi);
            }
        }
        sync_row();
        uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
        for (int k = 0; k < CL; ++k) {
            kmin = min(kmin, peer(k)->key_lo);
            kmax = max(kmax, peer(k)->key_hi);
        }
        // The search runs over a row's own span of keys: a key becomes its distance from the largest one, shifted
        // so that the span fills whole digits of eight bits, and turned around so that larger still means larger.
        // Its leading digit then spreads over the bins (the leading bits of the keys themselves are almost all alike).
        const uint32_t span = kmax - kmin;
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
            for_each_logit(row, lo, hi, vec, [&](int, float v) { z += fixed_mass(v * inv_t); });
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
            if ((tid & 31) == 0) atomicAdd(&sh.z, z);
            sync_row();
            if (tid == 0) {
                unsigned long long total = 0ull;
                for (int k = 0; k < CL; ++k) total += peer(k)->z;
                limit_p = (unsigned long long)((double)top_p * (double)total);
            }
        }
        uint32_t prefix_k = 0, prefix_p = 0;                  // the digits found so far, most significant first
        for (int digit = digits - 1; digit >= 0; --digit) {
            const int shift = 8 * digit;
            if constexpr (CL > 1) sync_row();                 // the others have read this block's histogram of the digit before
            if (tid < 256) {
                sh.cnt[tid] = 0u;
                sh.piece[0][tid] = sh.piece[1][tid] = sh.piece[2][tid] = 0u;
            }
            __syncthreads();
            for_each_logit(row, lo, hi, vec, [&](int, float v) {
                const float x = v * inv_t;
                const uint32_t key = spread(ordered_key(x));
                const uint32_t high = digit == digits - 1 ? 0u : key >> (shift + 8);
                const uint32_t bin = (key >> shift) & 255u;
                if (use_k && high == prefix_k) atomicAdd(&sh.cnt[bin], 1u);
                if (use_p && high == prefix_p) {
                    const unsigned long long q = fixed_mass(x);         // zero for the far tail: nothing to add
                    const unsigned p0 = (unsigned)(q & 0x7FFull), p1 = (unsigned)((q >> 11) & 0x7FFull), p2 = (unsigned)(q >> 22);
                    if (p0) atomicAdd(&sh.piece[0][bin], p0);
                    if (p1) atomicAdd(&sh.piece[1][bin], p1);
                    if (p2) atomicAdd(&sh.piece[2][bin], p2);
                }
            });
            sync_row();
            if (tid < 256) {
                unsigned int c = 0u;
                unsigned long long p0 = 0ull, p1 = 0ull, p2 = 0ull;
                for (int k = 0; k < CL; ++k) {
                    const SampleShared* q = peer(k);
                    c += q->cnt[tid];
                    p0 += q->piece[0][tid];
                    p1 += q->piece[1][tid];
                    p2 += q->piece[2][tid];
                }
                cnt_all[tid] = c;
                mass[tid] = p0 + (p1 << 11) + (p2 << 22);
            }
            __syncthreads();
            // inclusive suffix sums over the bins (bin b: everything in bins b..255), in place: by shuffles inside
            // the eight warps that hold the bins, then the totals of the warps behind
            {
                unsigned int c = 0u;
                unsigned long long m = 0ull;
                const int lane = tid & 31, w = tid >> 5;
                if (tid < 256) {
                    c = cnt_all[tid];
                    m = mass[tid];
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) {
                        const unsigned int c2 = __shfl_down_sync(0xffffffffu, c, off);
                        const unsigned long long m2 = __shfl_down_sync(0xffffffffu, m, off);
                        if (lane + off < 32) {
                            c += c2;
                            m += m2;
                        }
                    }
                    if (lane == 0) {
                        warp_cnt[w] = c;
                        warp_mass[w] = m;
                    }
                }
                __syncthreads();
                if (tid < 256) {
                    for (int k = w + 1; k < 8; ++k) {
                        c += warp_cnt[k];
                        m += warp_mass[k];
                    }
                    cnt_all[tid] = c;
                    mass[tid] = m;
                }
                __syncthreads();
            }
            if (tid < 256) {
                // top-k: the largest bin with at least `need_k` tokens in it and above it
                const unsigned int c_here = cnt_all[tid], c_above = tid < 255 ? cnt_all[tid + 1] : 0u;
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
    for_each_logit(row, lo, hi, vec, [&](int i, float v) {
        const float x = v * inv_t;
        if (ordered_key(x) < key_floor) return;
        const float u = uniform01(seed, counter, (uint64_t)i);
        const float score = x - logf(-logf(u));
        if (score > best.v || (score == best.v && i < best.i) || best.i == 0x7fffffff) best = MaxIdx{score, i};
    });
    finish(best);
}

template <int CL>
static int launch_sample(const float* logits, int* out, int rows, int V, size_t row_stride, const float* temps,
                         const int* top_ks, const float* top_ps, const unsigned long long* seeds,
                         const unsigned long long* counters, cudaStream_t stream) {
    if (CL == 1) {
        sample_kernel<1><<<rows, 1024, 0, stream>>>(logits, out, V, row_stride, temps, top_ks, top_ps, seeds, counters);
        PL_LAUNCHED("sample");
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * CL);
    cfg.blockDim = dim3(1024);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PL_CUDA(cudaLaunchKernelEx(&cfg, sample_kernel<CL>, logits, out, V, row_stride, temps, top_ks, top_ps, seeds, counters));
    return 0;
}

PL_EXPORT int pl_sample(const float* logits, int* out, int rows, int V, long long row_stride, const float* temps,
                        const int* top_ks, const float* top_ps, const unsigned long long* seeds,
                        const unsigned long long* counters, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && V > 0 && V < (1 << 21) && row_stride >= V, "sample: bad sizes rows=%d V=%d", rows, V);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        PL_CUDA(cudaGetDevice(&dev));
        PL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    // Few rows of a large vocabulary: a cluster of blocks per row, as large as still gives every block an SM of its own
    // (measured at 128,256 tokens with top-p: 8 rows 238 -> 58 us with clusters of 8; 64 rows are best with 2).
    const size_t rs = (size_t)row_stride;
    if (V >= 16384) {
        if (rows * 8 <= sms) return launch_sample<8>(logits, out, rows, V, rs, temps, top_ks, top_ps, seeds, counters, stream);
        if (rows * 4 <= sms) return launch_sample<4>(logits, out, rows, V, rs, temps, top_ks, top_ps, seeds, counters, stream);
        if (rows * 2 <= sms) return launch_sample<2>(logits, out, rows, V, rs, temps, top_ks, top_ps, seeds, counters, stream);
    }
    return launch_sample<1>(logits, out, rows, V, rs, temps, top_ks, top_ps, seeds, counters, stream);
}
