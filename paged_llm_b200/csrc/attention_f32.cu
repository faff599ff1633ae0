// Paged attention in true float32 on the CUDA cores, for prefill portions and
// for decoding, and the kernel that merges split partials (used by both
// precisions).  Scores, softmax and the weighted sum are float32 with expf.
#include "attention_common.cuh"

constexpr int F32_ROWS = 16;     // query rows per block
constexpr int F32_KEYS = 32;     // keys per iteration: one per lane
constexpr int F32_MAXD = 256;

// grid: (items, kv heads); 128 threads = 4 warps, each owning 4 of the 16 rows.
__global__ void __launch_bounds__(128) attn_f32_kernel(AttnParams p) {
    attn_zero_padding<float>(p);
    const AttnItem it = attn_decode_item(p, blockIdx.x / p.nkv, F32_ROWS, F32_KEYS);
    if (!it.valid) return;
    extern __shared__ float smem[];
    const int d = p.d, kvh = blockIdx.x % p.nkv, G = p.nh / p.nkv;
    float* Qs = smem;                          // [16][d]
    float* Ks = Qs + F32_ROWS * d;             // [32][d + 1]
    float* Vs = Ks + F32_KEYS * (d + 1);       // [32][d]
    float* Ps = Vs + F32_KEYS * d;             // [4][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* q = (const float*)p.q;
    const float* kv = (const float*)p.kv;
    const int* bt = p.block_table + (size_t)it.seq * p.bt_stride;

    for (int e = tid; e < F32_ROWS * d; e += 128) {
        const int r = e / d, c = e - r * d;
        const int R = it.row_base + r;
        float v = 0.f;
        if (R < it.rows_total) v = q[(size_t)(it.q0 + R / G) * p.q_stride + (kvh * G + R % G) * d + c];
        Qs[e] = v;
    }
    int pos[4];
    float m[4], l[4], acc[4][F32_MAXD / 32], slope[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        const int R = it.row_base + warp * 4 + rr;
        pos[rr] = R < it.rows_total ? it.lk - it.nq + R / G : -1;
        slope[rr] = p.slopes != nullptr && R < it.rows_total ? p.slopes[kvh * G + R % G] : 0.f;
        m[rr] = -INFINITY;
        l[rr] = 0.f;
#pragma unroll
        for (int cc = 0; cc < F32_MAXD / 32; ++cc) acc[rr][cc] = 0.f;
    }
    const int ncc = (d + 31) / 32;

    for (int kt = it.key_lo; kt < it.key_hi; kt += F32_KEYS) {
        __syncthreads();
        for (int e = tid; e < F32_KEYS * d; e += 128) {
            const int j = e / d, c = e - j * d;
            const int n = kt + j;
            float kk = 0.f, vv = 0.f;
            if (n < it.key_hi) {
                const int page = bt[n / p.ps];      // (ps_shift is for the bfloat16 kernels)
                if (page >= 0) {
                    const size_t base = ((((size_t)page * 2) * p.nkv + kvh) * p.ps + n % p.ps) * d + c;
                    kk = kv[base];
                    vv = kv[base + (size_t)p.nkv * p.ps * d];
                }
            }
            Ks[j * (d + 1) + c] = kk;
            Vs[j * d + c] = vv;
        }
        __syncthreads();
        const int n = kt + lane;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
            if (pos[rr] < 0) continue;                   // uniform per warp
            const float* qr = Qs + (warp * 4 + rr) * d;
            const float* kr = Ks + lane * (d + 1);
            float s = 0.f;
            for (int c = 0; c < d; ++c) s = fmaf(qr[c], kr[c], s);
            s = attn_score(p, s, slope[rr], n, pos[rr]);
            const bool vis = n < it.key_hi && n <= pos[rr] && (p.window <= 0 || n > pos[rr] - p.window);
            const float m_new = fmaxf(m[rr], warp_max(vis ? s : -INFINITY));
            if (m_new == -INFINITY) continue;
            const float pj = vis ? expf(s - m_new) : 0.f;
            const float alpha = m[rr] == -INFINITY ? 0.f : expf(m[rr] - m_new);
            l[rr] = l[rr] * alpha + warp_sum(pj);
            m[rr] = m_new;
            Ps[warp * 32 + lane] = pj;
            __syncwarp();
#pragma unroll
            for (int cc = 0; cc < F32_MAXD / 32; ++cc) {
                const int c = lane + 32 * cc;
                if (cc < ncc && c < d) {
                    float a = acc[rr][cc] * alpha;
                    for (int j = 0; j < F32_KEYS; ++j) a = fmaf(Ps[warp * 32 + j], Vs[j * d + c], a);
                    acc[rr][cc] = a;
                }
            }
            __syncwarp();
        }
    }

#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        if (pos[rr] < 0) continue;
        const int R = it.row_base + warp * 4 + rr;
        const int tok = R / G, head = kvh * G + R % G;
        if (it.splits <= 1) {
            float* o = (float*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * d;
            const float inv = l[rr] > 0.f ? 1.0f / l[rr] : 0.f;
#pragma unroll
            for (int cc = 0; cc < F32_MAXD / 32; ++cc) {
                const int c = lane + 32 * cc;
                if (cc < ncc && c < d) o[c] = acc[rr][cc] * inv;
            }
        } else {
            float* part = attn_partial(p, it.scratch_base + tok, head, it.split);
            if (lane == 0) {
                part[0] = m[rr];
                part[1] = l[rr];
            }
#pragma unroll
            for (int cc = 0; cc < F32_MAXD / 32; ++cc) {
                const int c = lane + 32 * cc;
                if (cc < ncc && c < d) part[2 + c] = acc[rr][cc];
            }
        }
    }
}

// Merge of split partials.  grid: (small items, heads); the block of an item's
// split 0 merges all splits of every token of its request for one head.
template <typename TO>
__global__ void attn_combine_kernel(AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= p.n_work) return;
    const int4 w = p.work[blockIdx.x];
    if (w.x < 0 || w.z != 0 || w.w <= 1) return;
    const int head = blockIdx.y, splits = w.w, d = p.d;
    const int q0 = p.cu_q[w.x], nq = p.cu_q[w.x + 1] - q0;
    for (int i = 0; i < nq; ++i) {
        float M = -INFINITY;
        for (int j = 0; j < splits; ++j) M = fmaxf(M, attn_partial(p, w.y + i, head, j)[0]);
        float L = 0.f;
        for (int j = 0; j < splits; ++j) {
            const float* part = attn_partial(p, w.y + i, head, j);
            if (part[0] != -INFINITY) L += part[1] * expf(part[0] - M);
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        TO* o = (TO*)p.out + (size_t)(q0 + i) * p.out_stride + head * d;
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            float a = 0.f;
            for (int j = 0; j < splits; ++j) {
                const float* part = attn_partial(p, w.y + i, head, j);
                if (part[0] != -INFINITY) a += part[2 + c] * expf(part[0] - M);
            }
            o[c] = from_float<TO>(a * inv);
        }
    }
}

int pl_attn_check(const AttnParams& p, const char* who) {
    PL_REQUIRE(p.nh > 0 && p.nkv > 0 && p.nh % p.nkv == 0, "%s: %d query heads on %d kv heads", who, p.nh, p.nkv);
    PL_REQUIRE(p.d > 0 && p.d % 16 == 0 && p.d <= 256, "%s: head_dim=%d must be a multiple of 16 up to 256", who, p.d);
    PL_REQUIRE(p.ps > 0, "%s: page_size=%d", who, p.ps);
    PL_REQUIRE(p.window >= 0, "%s: window=%d", who, p.window);
    PL_REQUIRE(p.max_splits >= 1, "%s: max_splits=%d", who, p.max_splits);
    PL_REQUIRE(p.softcap >= 0.f, "%s: softcap=%f must not be negative", who, (double)p.softcap);
    return 0;
}

PL_EXPORT int pl_attention_f32(const AttnParams* params, cudaStream_t stream) {
    AttnParams p = *params;
    if (p.n_work == 0) return 0;
    if (int rc = pl_attn_check(p, "attention_f32")) return rc;
    const size_t smem = ((size_t)F32_ROWS * p.d + F32_KEYS * (p.d + 1) + F32_KEYS * p.d + 4 * 32) * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        PL_CUDA(cudaFuncSetAttribute(attn_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr_set = true;
    }
    attn_f32_kernel<<<dim3(p.n_work * p.nkv), 128, smem, stream>>>(p);
    PL_LAUNCHED("attention_f32");
    return 0;
}

PL_EXPORT int pl_attention_combine(const AttnParams* params, int out_dtype, cudaStream_t stream) {
    AttnParams p = *params;
    if (p.n_work == 0) return 0;
    if (int rc = pl_attn_check(p, "attention_combine")) return rc;
    const int threads = p.d <= 64 ? 64 : (p.d <= 128 ? 128 : 256);
    if (out_dtype == PL_F32)
        PL_CUDA(launch_pdl(attn_combine_kernel<float>, dim3(p.n_work, p.nh), dim3(threads), 0, stream, p));
    else if (out_dtype == PL_BF16)
        PL_CUDA(launch_pdl(attn_combine_kernel<__nv_bfloat16>, dim3(p.n_work, p.nh), dim3(threads), 0, stream, p));
    else
        return pl_fail("attention_combine: unknown dtype %d", out_dtype);
    return 0;
}
