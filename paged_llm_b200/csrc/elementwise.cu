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
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_float(row[c]);
}

PL_EXPORT int pl_embedding(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                           cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(T > 0 && H > 0 && V > 0, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == PL_F32)
        embedding_kernel<float><<<T, threads, 0, stream>>>((const float*)table, ids, out, H, V);
    else if (table_dtype == PL_BF16)
        embedding_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, H, V);
    else
        return pl_fail("embedding: unknown dtype %d", table_dtype);
    PL_LAUNCHED("embedding");
    return 0;
}

// ------------------------------------------------------------------ RMSNorm
// One block per row.  x is the float32 residual stream; with a branch, x += branch
// is stored back first.  y = x * (1 / sqrt(mean(x^2) + eps)) * w, rounded once.
template <typename TB, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TB* __restrict__ branch, const TW* __restrict__ w,
                               TO* __restrict__ y, int H, float eps, int use_smem) {
    extern __shared__ float row_cache[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
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
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const int use_smem = (size_t)H * 4 <= 40 * 1024;
    rmsnorm_kernel<TB, TW, TO><<<rows, threads, use_smem ? (size_t)H * 4 : 0, stream>>>(
        x, (const TB*)branch, (const TW*)w, (TO*)y, H, eps, use_smem);
    PL_LAUNCHED("rmsnorm");
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
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / I;
        const int c = (int)(i - r * I);
        const float g = to_float(gu[r * 2 * I + c]);
        const float u = to_float(gu[r * 2 * I + I + c]);
        const float s = g / (1.0f + expf(-g));
        out[i] = from_float<T>(s * u);
    }
}

PL_EXPORT int pl_silu_mul(const void* gate_up, void* out, int dtype, int rows, int I, cudaStream_t stream) {
    if (rows == 0) return 0;
    PL_REQUIRE(rows > 0 && I > 0, "silu_mul: bad sizes rows=%d I=%d", rows, I);
    const size_t total = (size_t)rows * I;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == PL_F32)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total);
    else if (dtype == PL_BF16)
        silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                      (__nv_bfloat16*)out, I, total);
    else
        return pl_fail("silu_mul: unknown dtype %d", dtype);
    PL_LAUNCHED("silu_mul");
    return 0;
}

// ------------------------------------------------------------------ row gather
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ idx, T* __restrict__ out, int H,
                                   int rows_in) {
    const int r = idx[blockIdx.x];
    T* o = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = (r >= 0 && r < rows_in) ? x[(size_t)r * H + c] : T(0);
}

PL_EXPORT int pl_gather_rows(const void* x, const int* idx, void* out, int dtype, int n, int H, int rows_in,
                             cudaStream_t stream) {
    if (n == 0) return 0;
    PL_REQUIRE(n > 0 && H > 0, "gather_rows: bad sizes n=%d H=%d", n, H);
    if (dtype == PL_F32)
        gather_rows_kernel<float><<<n, 128, 0, stream>>>((const float*)x, idx, (float*)out, H, rows_in);
    else if (dtype == PL_BF16)
        gather_rows_kernel<__nv_bfloat16><<<n, 128, 0, stream>>>((const __nv_bfloat16*)x, idx, (__nv_bfloat16*)out, H,
                                                                 rows_in);
    else
        return pl_fail("gather_rows: unknown dtype %d", dtype);
    PL_LAUNCHED("gather_rows");
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
                                     int write) {
    const int t = blockIdx.x;
    const int s = token_seq[t];
    if (s < 0) return;
    const int pos = positions[t];
    T* row = qkv + (size_t)t * row_stride;
    const int half = rotary_dim / 2;
    if (half > 0 && pos >= 0 && pos < table_len) {
        const float2* cs = table + (size_t)pos * half;
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
    if (!write) return;
    __syncthreads();
    const int page = block_table[(size_t)s * bt_stride + pos / ps];
    if (page < 0 || page >= num_pages) return;
    const int off = pos % ps;
    const T* k = row + nh * d;
    const T* v = row + (nh + nkv) * d;
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
    if (dtype == PL_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>((float*)qkv, row_stride, (const float2*)table, table_len,
                                                               rotary_dim, interleaved, positions, token_seq,
                                                               block_table, bt_stride, (float*)kv, num_pages, nh, nkv,
                                                               d, ps, write);
    else if (dtype == PL_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, row_stride, (const float2*)table, table_len, rotary_dim, interleaved, positions,
            token_seq, block_table, bt_stride, (__nv_bfloat16*)kv, num_pages, nh, nkv, d, ps, write);
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
