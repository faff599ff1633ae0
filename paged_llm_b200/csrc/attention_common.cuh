// What the attention kernels of both precisions share: how an item of the work
// list becomes query rows and a key range, and the layout of split partials.
//
// Semantics (xiyiji/paged-llm pagedllm/attention/reference.py:23-55 and
// triton_kernel.py:22-93): request s has nq new query tokens and a context of Lk
// keys that includes them; query token i sits at position Lk - nq + i and sees
// keys 0..position (with a window w: the last w of them); query head h reads kv
// head h / (heads / kv_heads); keys and values are read through the block table.
#pragma once

#include "common.cuh"

struct AttnItem {
    int seq, nq, lk, q0;     // request, its new tokens, its context length, its first row in the batch
    int row_base;            // first packed row (token * G + head in group) of this tile
    int rows_total;          // nq * G
    int key_lo, key_hi;      // keys [key_lo, key_hi) are this item's share
    int split, splits;
    int scratch_base;        // first scratch row of the request (split items)
    bool valid;
};

__device__ __forceinline__ AttnItem attn_decode_item(const AttnParams& p, int idx, int block_rows, int key_align) {
    AttnItem it;
    it.valid = false;
    if (idx >= p.n_work) return it;
    const int4 w = p.work[idx];
    if (w.x < 0) return it;
    const int G = p.nh / p.nkv;
    it.seq = w.x;
    it.q0 = p.cu_q[w.x];
    it.nq = p.cu_q[w.x + 1] - it.q0;
    it.lk = p.k_lens[w.x];
    it.rows_total = it.nq * G;
    it.row_base = p.is_small ? 0 : w.y * block_rows;
    it.scratch_base = p.is_small ? w.y : 0;
    it.split = w.z;
    it.splits = w.w;
    if (it.nq <= 0 || it.row_base >= it.rows_total) return it;
    const int last_row = min(it.rows_total, it.row_base + block_rows) - 1;
    const int pos_first = it.lk - it.nq + it.row_base / G;
    const int pos_last = it.lk - it.nq + last_row / G;
    int lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int hi = pos_last + 1;
    if (it.splits > 1) {
        int chunk = (hi - lo + it.splits - 1) / it.splits;
        chunk = (chunk + key_align - 1) / key_align * key_align;
        lo = lo + it.split * chunk;
        hi = min(hi, lo + chunk);
    }
    it.key_lo = lo;
    it.key_hi = max(hi, lo);
    it.valid = true;
    return it;
}

// The same for the cluster form: the request comes from the block index, the split from the
// block's rank in its cluster of `splits` blocks; the keys are cut evenly, in multiples of 32.
__device__ __forceinline__ AttnItem attn_cluster_item(const AttnParams& p, int seq, int rank, int splits) {
    AttnItem it;
    it.valid = false;
    it.seq = seq;
    it.q0 = p.cu_q[seq];
    it.nq = p.cu_q[seq + 1] - it.q0;
    it.lk = p.k_lens[seq];
    const int G = p.nh / p.nkv;
    it.rows_total = it.nq * G;
    it.row_base = 0;
    it.scratch_base = 0;
    it.split = rank;
    it.splits = splits;
    if (it.nq <= 0) return it;
    const int pos_first = it.lk - it.nq;
    const int lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int hi = it.lk;
    int chunk = (hi - lo + splits - 1) / splits;
    chunk = (chunk + 31) / 32 * 32;
    it.key_lo = min(hi, lo + rank * chunk);
    it.key_hi = min(hi, it.key_lo + chunk);
    it.valid = true;
    return it;
}

// Zeroes the rows of `out` that pad the step (see AttnParams::pad_to); block 0 only, after the wait for the
// kernel in front (the buffer may be memory that kernel still reads under another name).
template <typename T>
__device__ __forceinline__ void attn_zero_padding(const AttnParams& p) {
    if (blockIdx.x != 0 || blockIdx.y != 0 || p.pad_to <= 0) return;
    const int row0 = p.cu_q[p.pad_seqs];
    if (row0 < 0 || row0 >= p.pad_to) return;
    T* o = (T*)p.out + (size_t)row0 * p.out_stride;
    const size_t n = (size_t)(p.pad_to - row0) * p.out_stride;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) o[i] = T(0);
}

// Partial result of (scratch row, head, split): [m, l, acc[0..d)] with m the
// running maximum of the scaled scores (natural-log units) and acc, l not yet
// divided.
__device__ __forceinline__ float* attn_partial(const AttnParams& p, int scratch_row, int head, int split) {
    return p.scratch + (((size_t)scratch_row * p.nh + head) * p.max_splits + split) * (size_t)(p.d + 2);
}

// Whether all partials of a scratch row lie inside the scratch the caller declared
// (p.scratch_floats).  A work item that names a row beyond it is skipped, never written.
__device__ __forceinline__ bool attn_partial_fits(const AttnParams& p, int scratch_row) {
    return scratch_row >= 0 &&
           (unsigned long long)(scratch_row + 1) * p.nh * p.max_splits * (unsigned long long)(p.d + 2) <=
               (unsigned long long)p.scratch_floats;
}
