// Per-row merge of the sampling head: the records EpiTopK wrote per (vocab tile, row) -> the k largest
// scaled logits of the row with their vocabulary indices (larger first; lower index first on ties) and the
// row's logsumexp. One CTA per row.
//
// Every candidate is packed into one 64-bit key whose unsigned order is the wanted order: the float's bits
// made order-preserving in the high word, 0xffffffff - column in the low word. Key 0 is "nothing".
// The CTA keeps the best kTopkMaxK keys seen so far at the front of a shared-memory array and folds further
// candidates in by sorting them together with that front (bitonic, descending).
//
// Exactness: a tile delivered only its kTileTop best. If the weakest of those still outranks the current
// k-th key, the tile may hide entries that belong to the result; the CTA then recomputes that tile's logits
// itself (dot products on the CUDA cores, fp32 accumulation), replaces the tile's entries and folds all of
// them in. The k-th key only rises while entries are folded in, so one pass over the tiles settles it.
#pragma once

#include "epilogues.cuh"
#include "row_kernels.cuh"

namespace lce {

constexpr int kTopkThreads = 256;
constexpr int kTopkMaxK = 64;
constexpr int kTopkSortN = 4096;  // keys sorted at a time: 32 KB of shared memory
constexpr int kTopkFlagBatch = 2048;  // tiles tested for repair at a time

__device__ __forceinline__ unsigned long long topk_key(float v, int col) {
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return (static_cast<unsigned long long>(u) << 32) | (0xffffffffu - static_cast<unsigned>(col));
}
__device__ __forceinline__ float topk_key_value(unsigned long long key) {
    unsigned u = static_cast<unsigned>(key >> 32);
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(u);
}
__device__ __forceinline__ int topk_key_col(unsigned long long key) {
    return static_cast<int>(0xffffffffu - static_cast<unsigned>(key & 0xffffffffull));
}

// Bitonic sort of n keys (n a power of two) in shared memory, largest first, by the whole CTA.
__device__ __forceinline__ void topk_sort_desc(unsigned long long* keys, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a < b) == desc) {
                    keys[lo] = b;
                    keys[hi] = a;
                }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int topk_pow2_at_least(int n) {
    int p = 64;
    while (p < n) p <<= 1;
    return p;
}

// partial: [n_tiles][kTopRecord][row_stride] (EpiTopK), bn = tile width the GEMM core used.
// top_val / top_idx: [N][K] (scaled logits, global vocabulary indices; -inf / -1 where the shard has fewer
// than K columns). lse_out: [N] logsumexp of the scaled logits of this shard.
template <class T>
__global__ void __launch_bounds__(kTopkThreads)
merge_topk_kernel(const float* partial, int n_tiles, int bn, long long row_stride, int N,
                  const T* __restrict__ x, const T* __restrict__ w, int H, int V, float scale, long long vocab_start,
                  int K, float* __restrict__ top_val, long long* __restrict__ top_idx, float* __restrict__ lse_out) {
    __shared__ unsigned long long keys[kTopkSortN];
    __shared__ float red_m[kTopkThreads / 32], red_s[kTopkThreads / 32];
    const int row = blockIdx.x;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // `partial` is the preceding GEMM's output
    const float* rec = partial + row;

    // ---- logsumexp of the row: thread t folds tiles t, t + 256, ..., then lanes and warps in a fixed order
    {
        float m = -INFINITY, s = 0.f;
        for (int b = t; b < n_tiles; b += kTopkThreads) {
            const float* base = rec + static_cast<long long>(b) * kTopRecord * row_stride;
            merge_ms(m, s, base[0], base[row_stride]);
        }
        for (int off = 1; off < 32; off <<= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, off), os = __shfl_xor_sync(0xffffffffu, s, off);
            merge_ms(m, s, om, os);
        }
        if (lane == 0) {
            red_m[warp] = m;
            red_s[warp] = s;
        }
        __syncthreads();
        if (t == 0) {
            for (int k = 1; k < kTopkThreads / 32; ++k) merge_ms(m, s, red_m[k], red_s[k]);
            lse_out[row] = m + logf(s);
        }
    }

    // ---- the k best of the tiles' candidates
    // A bound first: the k-th largest of the tiles' maxima (record slot 0) is a lower bound of the k-th
    // largest logit, because k tiles hold a logit at least that large. Only candidates that reach it can be
    // among the k best - a few dozen to a few hundred of the n_tiles x kTileTop - so the main sort is small.
    __shared__ int n_kept;
    bool selected = false;
    const int total = n_tiles * kTileTop;
    if (n_tiles <= kTopkSortN) {
        const int nt = topk_pow2_at_least(n_tiles);
        for (int i = t; i < nt; i += kTopkThreads)
            keys[i] = i < n_tiles ? topk_key(rec[static_cast<long long>(i) * kTopRecord * row_stride], 0) : 0ull;
        topk_sort_desc(keys, nt);
        const unsigned bound = n_tiles >= K ? static_cast<unsigned>(keys[K - 1] >> 32) : 0u;
        __syncthreads();
        if (t == 0) n_kept = 0;
        __syncthreads();
        for (int i = t; i < total; i += kTopkThreads) {
            const int tile = i / kTileTop, slot = i % kTileTop;
            const float* r0 = rec + static_cast<long long>(tile) * kTopRecord * row_stride;
            const float val = r0[(2 + slot) * row_stride];
            if (static_cast<unsigned>(topk_key(val, 0) >> 32) >= bound) {
                const int col = __float_as_int(r0[(2 + kTileTop + slot) * row_stride]);
                if (col >= 0) {
                    const int pos = atomicAdd(&n_kept, 1);  // the order of arrival does not matter: sorted below
                    if (pos < kTopkSortN) keys[pos] = topk_key(val, col);
                }
            }
        }
        __syncthreads();
        const int kept = n_kept;
        if (kept <= kTopkSortN) {  // (else: too many equal values reach the bound - take the general path)
            const int n = topk_pow2_at_least(kept);
            for (int i = kept + t; i < n; i += kTopkThreads) keys[i] = 0ull;
            topk_sort_desc(keys, n);
            selected = true;
        }
    }
    if (!selected) {  // general path: every candidate, kTopkSortN at a time together with the best so far
        __syncthreads();
        for (int i = t; i < kTopkMaxK; i += kTopkThreads) keys[i] = 0ull;
        const int per_pass = kTopkSortN - kTopkMaxK;
        for (int base = 0; base < total; base += per_pass) {
            const int cnt = min(per_pass, total - base);
            const int n = topk_pow2_at_least(kTopkMaxK + cnt);
            __syncthreads();
            for (int i = t; i < n - kTopkMaxK; i += kTopkThreads) {
                unsigned long long key = 0ull;
                if (i < cnt) {
                    const int tile = (base + i) / kTileTop, slot = (base + i) % kTileTop;
                    const float* r0 = rec + static_cast<long long>(tile) * kTopRecord * row_stride;
                    const int col = __float_as_int(r0[(2 + kTileTop + slot) * row_stride]);
                    if (col >= 0) key = topk_key(r0[(2 + slot) * row_stride], col);
                }
                keys[kTopkMaxK + i] = key;
            }
            topk_sort_desc(keys, n);
        }
    }

    // ---- repair: tiles whose weakest kept entry still outranks the k-th key are recomputed in full.
    // All tiles are tested at once against the k-th key as it stands (it only rises later, so this can flag a
    // tile too many, never one too few); the flagged ones, usually none, are then taken one by one.
    __shared__ int flagged[kTopkFlagBatch];
    __shared__ int n_flagged;
    for (int tile0 = 0; tile0 < n_tiles; tile0 += kTopkFlagBatch) {
        if (t == 0) n_flagged = 0;
        __syncthreads();
        const unsigned long long kth = keys[K - 1];
        for (int tile = tile0 + t; tile < min(n_tiles, tile0 + kTopkFlagBatch); tile += kTopkThreads) {
            const float* r0 = rec + static_cast<long long>(tile) * kTopRecord * row_stride;
            const int last_col = __float_as_int(r0[(2 + 2 * kTileTop - 1) * row_stride]);
            // a tile with fewer than kTileTop columns delivered all of them
            if (last_col >= 0 && topk_key(r0[(2 + kTileTop - 1) * row_stride], last_col) > kth)
                flagged[atomicAdd(&n_flagged, 1)] = tile;
        }
        __syncthreads();
        const int count = n_flagged;
        for (int f = 0; f < count; ++f) {
            const int tile = flagged[f];  // any order: the result is the k best of the same set of entries
            const int col0 = tile * bn;
            __syncthreads();
            for (int i = t; i < kTopkMaxK; i += kTopkThreads) {
                const unsigned long long key = keys[i];
                const int c = topk_key_col(key);
                if (key != 0ull && c >= col0 && c < col0 + bn) keys[i] = 0ull;  // superseded by the recomputed values
            }
            const int n = topk_pow2_at_least(kTopkMaxK + bn);
            for (int i = t; i < n - kTopkMaxK; i += kTopkThreads)
                if (i >= bn || col0 + i >= V) keys[kTopkMaxK + i] = 0ull;
            const T* xr = x + static_cast<long long>(row) * H;
            for (int c = warp; c < bn && col0 + c < V; c += kTopkThreads / 32) {
                const T* wr = w + static_cast<long long>(col0 + c) * H;
                float acc = 0.f;
                for (int k = lane; k < H; k += 32) acc = fmaf(Cvt<T>::to_f(xr[k]), Cvt<T>::to_f(wr[k]), acc);
                for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (lane == 0) keys[kTopkMaxK + c] = topk_key(acc * scale, col0 + c);
            }
            topk_sort_desc(keys, n);
        }
        __syncthreads();
    }

    for (int i = t; i < K; i += kTopkThreads) {
        const unsigned long long key = keys[i];
        top_val[static_cast<long long>(row) * K + i] = key ? topk_key_value(key) : -INFINITY;
        top_idx[static_cast<long long>(row) * K + i] = key ? vocab_start + topk_key_col(key) : -1ll;
    }
}

}  // namespace lce
