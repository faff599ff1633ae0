// Decode attention with its scratch inside the library; see
// attention_decode_static.h for the why and the contract.
#define PL_DPAD 128
#include "attention_bf16.cuh"
#include "attention_decode_static.h"

// Partials of all splits: [scratch row][head][split][m, l, acc[head_dim]] floats.
static __device__ __align__(256) float g_static_scratch[PL_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};     // device address of the array, per device

// In host code `g_static_scratch` is only a handle; the device address has to be asked for,
// once per device, with that device current.
int static_scratch(float** out) {
    int dev = -1;
    PL_CUDA(cudaGetDevice(&dev));
    PL_REQUIRE(dev >= 0 && dev < kMaxDevices, "attention_decode_static: device index %d is out of range", dev);
    if (g_scratch_address[dev] == nullptr) {
        void* ptr = nullptr;
        PL_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        PL_REQUIRE(ptr != nullptr, "attention_decode_static: the scratch array has no device address");
        g_scratch_address[dev] = static_cast<float*>(ptr);
    }
    *out = g_scratch_address[dev];
    return 0;
}

// Merge of the splits of one request and head; one block per (item of split 0, head).
__global__ void static_combine_kernel(AttnParams p) {
    if ((int)blockIdx.x >= p.n_work) return;
    const int4 w = p.work[blockIdx.x];
    if (w.x < 0 || w.z != 0 || w.w <= 1) return;
    const int head = blockIdx.y, splits = w.w, d = p.d;
    // The attention kernel takes at most 16 query rows per request and kv head and skips scratch rows
    // outside the array: the same two limits here, so that no partial is read that was not written.
    const int q0 = p.cu_q[w.x], nq = min(p.cu_q[w.x + 1] - q0, 16 / (p.nh / p.nkv));
    for (int i = 0; i < nq; ++i) {
        if (!attn_partial_fits(p, w.y + i)) continue;
        float M = -INFINITY;
        for (int j = 0; j < splits; ++j) M = fmaxf(M, attn_partial(p, w.y + i, head, j)[0]);
        float L = 0.f;
        for (int j = 0; j < splits; ++j) {
            const float* part = attn_partial(p, w.y + i, head, j);
            if (part[0] != -INFINITY) L += part[1] * expf(part[0] - M);
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(q0 + i) * p.out_stride + head * d;
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            float a = 0.f;
            for (int j = 0; j < splits; ++j) {
                const float* part = attn_partial(p, w.y + i, head, j);
                if (part[0] != -INFINITY) a += part[2 + c] * expf(part[0] - M);
            }
            o[c] = __float2bfloat16_rn(a * inv);
        }
    }
}

}  // namespace

PL_EXPORT long long pl_attention_decode_static_capacity(void) { return (long long)PL_STATIC_SCRATCH_BYTES; }

PL_EXPORT int pl_attention_decode_static(const void* q, int q_stride, const void* kv_layer, void* out, int out_stride,
                                         const int* block_table, int bt_stride, const int* cu_q, const int* k_lens,
                                         const int* work, int n_work, int max_splits, int scratch_rows,
                                         int num_heads, int num_kv_heads, int head_dim, int page_size, int window,
                                         float scale, cudaStream_t stream) {
    if (n_work == 0) return 0;
    PL_REQUIRE(n_work > 0 && max_splits >= 1 && scratch_rows >= 1, "attention_decode_static: bad counts");
    PL_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0,
               "attention_decode_static: %d query heads on %d kv heads", num_heads, num_kv_heads);
    PL_REQUIRE(head_dim > 0 && head_dim % 16 == 0 && head_dim <= PL_DPAD,
               "attention_decode_static: head_dim=%d must be a multiple of 16 up to %d", head_dim, PL_DPAD);
    PL_REQUIRE(num_heads / num_kv_heads <= 16, "attention_decode_static: at most 16 query heads per kv head");
    PL_REQUIRE(page_size > 0 && window >= 0, "attention_decode_static: bad page size or window");
    PL_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kv_layer & 15) == 0,
               "attention_decode_static: q and the cache must be 16-byte aligned with 16-byte row strides");
    const unsigned long long need =
        (unsigned long long)scratch_rows * num_heads * max_splits * (head_dim + 2) * sizeof(float);
    PL_REQUIRE(need <= PL_STATIC_SCRATCH_BYTES,
               "attention_decode_static: partials need %llu bytes, the built-in scratch holds %u "
               "(rows %d x heads %d x splits %d x (head_dim %d + 2) floats); use fewer splits or the regular entry point",
               need, (unsigned)PL_STATIC_SCRATCH_BYTES, scratch_rows, num_heads, max_splits, head_dim);
    float* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;

    AttnParams p = {};
    p.q = q;
    p.kv = kv_layer;
    p.out = out;
    p.block_table = block_table;
    p.cu_q = cu_q;
    p.k_lens = k_lens;
    p.work = reinterpret_cast<const int4*>(work);
    p.scratch = scratch;
    // what the caller declared, which was checked against the array above; rows beyond it are skipped
    p.scratch_floats = (long long)(need / sizeof(float));
    p.q_stride = q_stride;
    p.out_stride = out_stride;
    p.bt_stride = bt_stride;
    p.n_work = n_work;
    p.max_splits = max_splits;
    p.nh = num_heads;
    p.nkv = num_kv_heads;
    p.d = head_dim;
    p.ps = page_size;
    p.window = window;
    p.is_small = 1;
    p.scale = scale;
    p.ps_shift = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1;
    p.counters = nullptr;                       // the merge runs as its own kernel below
    if (int rc = launch_attn_bf16<PL_DPAD, 1, 4, 32>(p, stream)) return rc;
    if (max_splits > 1) {
        const int threads = head_dim <= 64 ? 64 : 128;
        static_combine_kernel<<<dim3(n_work, num_heads), threads, 0, stream>>>(p);
        PL_LAUNCHED("attention_decode_static merge");
    }
    return 0;
}
