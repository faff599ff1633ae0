// Embedding, RMSNorm (with the residual sum), SiLU*mul, row gather, the rotary
// table, rotary + key/value write into pages, page copy.
//
// What each reproduces (xiyiji/paged-llm): embedding llama.py:197; RMSNorm
// llama.py:80-83; residual sums llama.py:183-184; SiLU*mul llama.py:171; rotary
// table llama.py:111-115; rotation llama.py:117-128; slot write
// kv_cache.py:42-45 with the slot of block_manager.py:237-243; page copy
// kv_cache.py:47-54.  The residual stream is float32 in both precisions; norms,
// angles and the residual sum are computed in float32.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int H, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    const bool valid = id >= 0 && id < V;
    const TW* row = table + (size_t)(valid ? id : 0) * H;
    if ((H & 3) == 0) {                                   // four elements per step, several steps in flight
#pragma unroll 4
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid) {
                if (sizeof(TW) == 4) {
                    v = *reinterpret_cast<const float4*>(row + c);
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(row + c);
                    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                    v = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
                }
            }
            *reinterpret_cast<float4*>(o + c) = v;
        }
        return;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = valid ? to_float(row[c]) : 0.f;
}

PL_EXPORT int pl_embedding(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                           cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(T > 0 && H > 0 && V > 0, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == PL_F32)
        PL_CUDA(launch_pdl(embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, out, H, V));
    else if (table_dtype == PL_BF16)
        PL_CUDA(launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                           (const __nv_bfloat16*)table, ids, out, H, V));
    else
        return pl_fail("embedding: unknown dtype %d", table_dtype);
    return 0;
}

// ------------------------------------------------------------------ RMSNorm
// One block per row.  x is the float32 residual stream; with a branch, x += branch
// is stored back first.  y = x * (1 / sqrt(mean(x^2) + eps)) * w, rounded once.
template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

constexpr int NORM_VEC_ITERS = 4;     // a thread keeps up to 16 elements of its row in registers

template <typename TB, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TB* __restrict__ branch, const TW* __restrict__ w,
                               TO* __restrict__ y, int H, float eps, int mode) {
    extern __shared__ float row_cache[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    if (mode == 2) {
        // H % 4 == 0 and H <= 16 * threads: the row lives in registers, all loads go out together
        float4 v[NORM_VEC_ITERS];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NORM_VEC_ITERS; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < H) {
                v[i] = *reinterpret_cast<const float4*>(x + base + c);
                if (branch != nullptr) {
                    const float4 b = Vec4<TB>::load(branch + base + c);
                    v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
                    *reinterpret_cast<float4*>(x + base + c) = v[i];
                }
                ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
            }
        }
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int i = 0; i < NORM_VEC_ITERS; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < H) {
                const float4 ww = Vec4<TW>::load(w + c);
                Vec4<TO>::store(y + base + c, make_float4(v[i].x * inv * ww.x, v[i].y * inv * ww.y,
                                                          v[i].z * inv * ww.z, v[i].w * inv * ww.w));
            }
        }
        return;
    }
    const int use_smem = mode == 1;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[base + c];
        if (branch != nullptr) {
            v += to_float(branch[base + c]);
            x[base + c] = v;
        }
        if (use_smem) row_cache[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = use_smem ? row_cache[c] : x[base + c];
        y[base + c] = from_float<TO>(v * inv * to_float(w[c]));
    }
}

template <typename TB, typename TW, typename TO>
static int launch_rmsnorm(float* x, const void* branch, const void* w, void* y, int rows, int H, float eps,
                          cudaStream_t stream) {
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    const bool aligned = (H & 3) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 7) == 0 &&
                         ((uintptr_t)w & 7) == 0 && ((uintptr_t)branch & 7) == 0;
    int mode = (size_t)H * 4 <= 40 * 1024 ? 1 : 0;
    if (aligned && H <= threads * 4 * NORM_VEC_ITERS) mode = 2;
    PL_CUDA(launch_pdl(rmsnorm_kernel<TB, TW, TO>, dim3(rows), dim3(threads), mode == 1 ? (size_t)H * 4 : 0, stream, x,
                       (const TB*)branch, (const TW*)w, (TO*)y, H, eps, mode));
    return 0;
}

// branch may be null.  branch_dtype and out_dtype are the compute dtype; w_dtype is the weight's.
PL_EXPORT int pl_rmsnorm(float* x, const void* branch, int branch_dtype, const void* w, int w_dtype, void* y,
                         int out_dtype, int rows, int H, float eps, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && H > 0, "rmsnorm: bad sizes rows=%d H=%d", rows, H);
    const int key = (branch_dtype << 2) | (w_dtype << 1) | out_dtype;
    switch (key) {
        case 0: return launch_rmsnorm<float, float, float>(x, branch, w, y, rows, H, eps, stream);
        case 1: return launch_rmsnorm<float, float, __nv_bfloat16>(x, branch, w, y, rows, H, eps, stream);
        case 2: return launch_rmsnorm<float, __nv_bfloat16, float>(x, branch, w, y, rows, H, eps, stream);
        case 3: return launch_rmsnorm<float, __nv_bfloat16, __nv_bfloat16>(x, branch, w, y, rows, H, eps, stream);
        case 4: return launch_rmsnorm<__nv_bfloat16, float, float>(x, branch, w, y, rows, H, eps, stream);
        case 5: return launch_rmsnorm<__nv_bfloat16, float, __nv_bfloat16>(x, branch, w, y, rows, H, eps, stream);
        case 6: return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16, float>(x, branch, w, y, rows, H, eps, stream);
        case 7: return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(x, branch, w, y, rows, H, eps, stream);
    }
    return pl_fail("rmsnorm: unknown dtypes %d %d %d", branch_dtype, w_dtype, out_dtype);
}

// ------------------------------------------------------------------ SiLU * mul
// 16-byte vectors of T as floats.
template <typename T> struct Vec16 {};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __low2float(h[i]);
            v[2 * i + 1] = __high2float(h[i]);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
    }
};

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int vec) {
    const size_t r = blockIdx.y;
    const T* g = gu + r * 2 * I;
    const T* u = g + I;
    T* o = out + r * I;
    if (vec) {
        constexpr int N = Vec16<T>::N;
#pragma unroll 2
        for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * N; c < I; c += gridDim.x * blockDim.x * N) {
            float gv[8], uv[8], ov[8];
            Vec16<T>::load(g + c, gv);
            Vec16<T>::load(u + c, uv);
#pragma unroll
            for (int i = 0; i < N; ++i) ov[i] = gv[i] / (1.0f + expf(-gv[i])) * uv[i];
            Vec16<T>::store(o + c, ov);
        }
        return;
    }
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < I; c += gridDim.x * blockDim.x) {
        const float gg = to_float(g[c]);
        o[c] = from_float<T>(gg / (1.0f + expf(-gg)) * to_float(u[c]));
    }
}

PL_EXPORT int pl_silu_mul(const void* gate_up, void* out, int dtype, int rows, int I, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && I > 0 && rows <= 65535 * 16, "silu_mul: bad sizes rows=%d I=%d", rows, I);
    const int per = dtype == PL_F32 ? 4 : 8;
    const int vec = I % per == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0;
    const int threads = 256;
    int bx = (I / (vec ? per : 1) + threads - 1) / threads;
    if (bx > 8) bx = 8;
    if (bx < 1) bx = 1;
    for (int r0 = 0; r0 < rows; r0 += 65535) {
        const int nr = rows - r0 < 65535 ? rows - r0 : 65535;
        const size_t esz = dtype == PL_F32 ? 4 : 2;
        const char* src = (const char*)gate_up + (size_t)r0 * 2 * I * esz;
        char* dst = (char*)out + (size_t)r0 * I * esz;
        if (dtype == PL_F32)
            silu_mul_kernel<float><<<dim3(bx, nr), threads, 0, stream>>>((const float*)src, (float*)dst, I, vec);
        else if (dtype == PL_BF16)
            silu_mul_kernel<__nv_bfloat16><<<dim3(bx, nr), threads, 0, stream>>>((const __nv_bfloat16*)src,
                                                                                  (__nv_bfloat16*)dst, I, vec);
        else
            return pl_fail("silu_mul: unknown dtype %d", dtype);
        PL_LAUNCHED("silu_mul");
    }
    return 0;
}

// ------------------------------------------------------------------ row gather
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ idx, T* __restrict__ out, int H,
                                   int rows_in) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = idx[blockIdx.x];
    const bool valid = r >= 0 && r < rows_in;
    T* o = out + (size_t)blockIdx.x * H;
    const T* src = x + (size_t)(valid ? r : 0) * H;
    constexpr int PER = 16 / sizeof(T);
    if (H % PER == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
#pragma unroll 4
        for (int c = threadIdx.x * PER; c < H; c += blockDim.x * PER) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (valid) v = *reinterpret_cast<const uint4*>(src + c);
            *reinterpret_cast<uint4*>(o + c) = v;
        }
        return;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = valid ? src[c] : T(0);
}

PL_EXPORT int pl_gather_rows(const void* x, const int* idx, void* out, int dtype, int n, int H, int rows_in,
                             cudaStream_t stream) {
    if (n == 0) return 0;
    PL_REQUIRE(n > 0 && H > 0, "gather_rows: bad sizes n=%d H=%d", n, H);
    if (dtype == PL_F32)
        PL_CUDA(launch_pdl(gather_rows_kernel<float>, dim3(n), dim3(128), 0, stream, (const float*)x, idx, (float*)out, H,
                           rows_in));
    else if (dtype == PL_BF16)
        PL_CUDA(launch_pdl(gather_rows_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, (const __nv_bfloat16*)x,
                           idx, (__nv_bfloat16*)out, H, rows_in));
    else
        return pl_fail("gather_rows: unknown dtype %d", dtype);
    return 0;
}

// ------------------------------------------------------------------ rotary table
// table[p][j] = (cos(p * inv_freq[j]), sin(p * inv_freq[j])), angle in float32.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float2* __restrict__ table, int P, int half) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)P * half) return;
    const int p = (int)(i / half), j = (int)(i % half);
    const float ang = (float)p * inv_freq[j];
    table[i] = make_float2(cosf(ang), sinf(ang));
}

PL_EXPORT int pl_rope_table(const float* inv_freq, float* table, int P, int half, cudaStream_t stream) {
    PL_REQUIRE(P > 0 && half > 0, "rope_table: bad sizes P=%d half=%d", P, half);
    const size_t total = (size_t)P * half;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, (float2*)table, P, half);
    PL_LAUNCHED("rope_table");
    return 0;
}

// ------------------------------------------------------------------ rotary + K/V write
// One block per token.  q and k heads of the fused projection row are rotated in
// place (float32 arithmetic, one rounding), then k and v go to the token's slot:
// page = block_table[request][pos / page_size], row pos % page_size.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const float2* __restrict__ table,
                                     int table_len, int rotary_dim, int interleaved, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                     int bt_stride, T* __restrict__ kv, int num_pages, int nh, int nkv, int d, int ps,
                                     int write, int vec) {
    const int t = blockIdx.x;
    const int s = token_seq[t];
    if (s < 0) return;
    const int pos = positions[t];
    T* row = qkv + (size_t)t * row_stride;
    const int half = rotary_dim / 2;
    // the page is asked for now and used at the end of the pass: its latency hides behind the rotation
    int page = -1;
    if (write && pos >= 0) page = block_table[(size_t)s * bt_stride + pos / ps];
    const bool to_cache = write && page >= 0 && page < num_pages;
    const int off = pos >= 0 ? pos % ps : 0;
    const bool rotate = half > 0 && pos >= 0 && pos < table_len;
    if (vec && !interleaved && rotate && rotary_dim == d) {
        // One pass: four pairs per step (elements j..j+3 of the first half with their partners);
        // rotated k goes to the row and, from the same registers, to its page slot; v is copied.
        const float2* cs = table + (size_t)pos * half;
        const int quads_per_head = half / 4;
        const int quads = (nh + nkv) * quads_per_head;
        constexpr int PER = 16 / sizeof(T);
        const int v_chunks = nkv * (d / PER);
        for (int i = threadIdx.x; i < quads + v_chunks; i += blockDim.x) {
            if (i < quads) {
                const int h = i / quads_per_head, j = (i - h * quads_per_head) * 4;
                T* head = row + h * d;
                const float4 a = Vec4<T>::load(head + j), b = Vec4<T>::load(head + j + half);
                const float4 c01 = *reinterpret_cast<const float4*>(cs + j);
                const float4 c23 = *reinterpret_cast<const float4*>(cs + j + 2);
                const float4 lo = make_float4(a.x * c01.x - b.x * c01.y, a.y * c01.z - b.y * c01.w,
                                              a.z * c23.x - b.z * c23.y, a.w * c23.z - b.w * c23.w);
                const float4 hi = make_float4(b.x * c01.x + a.x * c01.y, b.y * c01.z + a.y * c01.w,
                                              b.z * c23.x + a.z * c23.y, b.w * c23.z + a.w * c23.w);
                Vec4<T>::store(head + j, lo);
                Vec4<T>::store(head + j + half, hi);
                if (h >= nh && to_cache) {
                    T* dst = kv + ((((size_t)page * 2 + 0) * nkv + (h - nh)) * ps + off) * d;
                    Vec4<T>::store(dst + j, lo);
                    Vec4<T>::store(dst + j + half, hi);
                }
            } else if (to_cache) {
                const int e = i - quads, h = e / (d / PER), c = (e - h * (d / PER)) * PER;
                const T* v = row + (nh + nkv) * d;
                const size_t vdst = ((((size_t)page * 2 + 1) * nkv + h) * ps + off) * d + c;
                *reinterpret_cast<uint4*>(kv + vdst) = *reinterpret_cast<const uint4*>(v + h * d + c);
            }
        }
        return;
    }
    if (rotate) {
        const float2* cs = table + (size_t)pos * half;
        if (vec && !interleaved) {
            // four pairs per step: elements j..j+3 of the first half with their partners
            const int quads = (nh + nkv) * (half / 4);
#pragma unroll 2
            for (int i = threadIdx.x; i < quads; i += blockDim.x) {
                const int h = i / (half / 4), j = (i - h * (half / 4)) * 4;
                T* head = row + h * d;
                const float4 a = Vec4<T>::load(head + j), b = Vec4<T>::load(head + j + half);
                const float4 c01 = *reinterpret_cast<const float4*>(cs + j);
                const float4 c23 = *reinterpret_cast<const float4*>(cs + j + 2);
                Vec4<T>::store(head + j, make_float4(a.x * c01.x - b.x * c01.y, a.y * c01.z - b.y * c01.w,
                                                     a.z * c23.x - b.z * c23.y, a.w * c23.z - b.w * c23.w));
                Vec4<T>::store(head + j + half, make_float4(b.x * c01.x + a.x * c01.y, b.y * c01.z + a.y * c01.w,
                                                            b.z * c23.x + a.z * c23.y, b.w * c23.z + a.w * c23.w));
            }
        } else {
            const int pairs = (nh + nkv) * half;
            for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
                const int h = i / half, j = i - h * half;
                T* head = row + h * d;
                const int ia = interleaved ? 2 * j : j;
                const int ib = interleaved ? 2 * j + 1 : j + half;
                const float a = to_float(head[ia]), b = to_float(head[ib]);
                const float2 c = cs[j];
                head[ia] = from_float<T>(a * c.x - b * c.y);
                head[ib] = from_float<T>(b * c.x + a * c.y);
            }
        }
    }
    if (!to_cache) return;
    __syncthreads();
    const T* k = row + nh * d;
    const T* v = row + (nh + nkv) * d;
    if (vec) {
        constexpr int PER = 16 / sizeof(T);
        const int per_head = d / PER;
        for (int i = threadIdx.x; i < nkv * per_head; i += blockDim.x) {
            const int h = i / per_head, c = (i - h * per_head) * PER;
            const size_t kdst = ((((size_t)page * 2 + 0) * nkv + h) * ps + off) * d + c;
            const size_t vdst = ((((size_t)page * 2 + 1) * nkv + h) * ps + off) * d + c;
            *reinterpret_cast<uint4*>(kv + kdst) = *reinterpret_cast<const uint4*>(k + h * d + c);
            *reinterpret_cast<uint4*>(kv + vdst) = *reinterpret_cast<const uint4*>(v + h * d + c);
        }
        return;
    }
    for (int i = threadIdx.x; i < nkv * d; i += blockDim.x) {
        const int h = i / d, c = i - h * d;
        const size_t kdst = ((((size_t)page * 2 + 0) * nkv + h) * ps + off) * d + c;
        const size_t vdst = ((((size_t)page * 2 + 1) * nkv + h) * ps + off) * d + c;
        kv[kdst] = k[i];
        kv[vdst] = v[i];
    }
}

PL_EXPORT int pl_rope_kv_write(void* qkv, int dtype, int T, int row_stride, const float* table, int table_len,
                               int rotary_dim, int interleaved, const int* positions, const int* token_seq,
                               const int* block_table, int bt_stride, void* kv, int num_pages, int nh, int nkv, int d,
                               int ps, int write, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(T > 0 && nh > 0 && nkv > 0 && d > 0 && ps > 0, "rope_kv_write: bad sizes");
    PL_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0, "rope_kv_write: rotary_dim=%d with d=%d",
               rotary_dim, d);
    PL_REQUIRE(row_stride >= (nh + 2 * nkv) * d, "rope_kv_write: row stride %d too small", row_stride);
    const int threads = 128;
    const int per16 = dtype == PL_F32 ? 4 : 8;
    // 16-byte path: heads, halves and rows start on 16-byte boundaries
    const int vec = d % per16 == 0 && row_stride % per16 == 0 && (rotary_dim / 2) % per16 == 0 &&
                    (((uintptr_t)qkv | (uintptr_t)kv | (uintptr_t)table) & 15) == 0;
    if (dtype == PL_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>((float*)qkv, row_stride, (const float2*)table, table_len,
                                                               rotary_dim, interleaved, positions, token_seq,
                                                               block_table, bt_stride, (float*)kv, num_pages, nh, nkv,
                                                               d, ps, write, vec);
    else if (dtype == PL_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, row_stride, (const float2*)table, table_len, rotary_dim, interleaved, positions,
            token_seq, block_table, bt_stride, (__nv_bfloat16*)kv, num_pages, nh, nkv, d, ps, write, vec);
    else
        return pl_fail("rope_kv_write: unknown dtype %d", dtype);
    PL_LAUNCHED("rope_kv_write");
    return 0;
}

// ------------------------------------------------------------------ page copy (copy-on-write)
// pool: [layers, pages, page_elems]; copies page src -> dst in every layer.
__global__ void copy_page_kernel(uint32_t* __restrict__ pool, size_t layer_words, size_t page_words, int src, int dst) {
    uint32_t* base = pool + (size_t)blockIdx.y * layer_words;
    const uint32_t* s = base + (size_t)src * page_words;
    uint32_t* d = base + (size_t)dst * page_words;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < page_words; i += (size_t)gridDim.x * blockDim.x)
        d[i] = s[i];
}

PL_EXPORT int pl_copy_page(void* pool, int layers, long long pages, long long page_bytes, int src, int dst,
                           cudaStream_t stream) {
    PL_REQUIRE(layers > 0 && page_bytes > 0 && page_bytes % 4 == 0, "copy_page: bad sizes");
    PL_REQUIRE(src >= 0 && src < pages && dst >= 0 && dst < pages, "copy_page: page %d -> %d outside the pool of %lld",
               src, dst, pages);
    if (src == dst) return 0;
    const size_t page_words = (size_t)page_bytes / 4;
    const int blocks = (int)((page_words + 255) / 256 < 64 ? (page_words + 255) / 256 : 64);
    copy_page_kernel<<<dim3(blocks, layers), 256, 0, stream>>>((uint32_t*)pool, (size_t)pages * page_words, page_words,
                                                               src, dst);
    PL_LAUNCHED("copy_page");
    return 0;
}

// ------------------------------------------------------------------ random weights on the device
// out[i] = mean + std * z_i with z ~ N(0, 1) from a counter-based stream: the pair of elements
// (2j, 2j + 1) comes from one 64-bit hash of (seed, tensor key, j) through the Box-Muller transform,
// so a tensor's values depend only on (seed, key, its size), never on the launch shape.  For
// benchmark models too large to draw on the host; the reference has no such mode.
__device__ __forceinline__ uint64_t fill_hash(uint64_t seed, uint64_t key, uint64_t j) {
    uint64_t x = seed + key * 0x9E3779B97F4A7C15ull + j * 0xBF58476D1CE4E5B9ull;
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, uint64_t seed, uint64_t key, float mean, float std) {
    const long long pairs = (n + 1) / 2;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < pairs; j += (long long)gridDim.x * blockDim.x) {
        const uint64_t x = fill_hash(seed, key, (uint64_t)j);
        const float u1 = ((float)(x >> 40) + 0.5f) * (1.0f / 16777216.0f);            // (0, 1)
        const float u2 = ((float)((x >> 16) & 0xFFFFFFull) + 0.5f) * (1.0f / 16777216.0f);
        const float r = sqrtf(-2.0f * logf(u1));
        float s, c;
        sincosf(6.283185307179586f * u2, &s, &c);
        out[2 * j] = from_float<T>(mean + std * r * c);
        if (2 * j + 1 < n) out[2 * j + 1] = from_float<T>(mean + std * r * s);
    }
}

PL_EXPORT int pl_fill_normal(void* out, int dtype, long long n, unsigned long long seed, unsigned long long key,
                             float mean, float std, cudaStream_t stream) {
    PL_REQUIRE(n >= 0 && std >= 0.f, "fill_normal: n=%lld std=%f", n, (double)std);
    if (n == 0) return 0;
    const long long pairs = (n + 1) / 2;
    const int blocks = (int)((pairs + 255) / 256 < 148 * 16 ? (pairs + 255) / 256 : 148 * 16);
    if (dtype == PL_F32)
        fill_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, seed, key, mean, std);
    else if (dtype == PL_BF16)
        fill_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, seed, key, mean, std);
    else
        return pl_fail("fill_normal: unknown dtype %d", dtype);
    PL_LAUNCHED("fill_normal");
    return 0;
}
