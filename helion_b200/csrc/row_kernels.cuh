// Small per-row kernels around the GEMMs: merging partial softmax statistics, the final
// logsumexp / loss, the deterministic loss reduction and the per-row gradient scale.
#pragma once

#include "epilogues.cuh"

namespace lce {

// Merges two (max, sum-exp) pairs; the sum is expressed relative to the new max.
__device__ __forceinline__ void merge_ms(float& m, float& s, float bm, float bs) {
    const float nm = fmaxf(m, bm);
    if (nm != -INFINITY) s = s * ptx::ex2((m - nm) * kLog2e) + bs * ptx::ex2((bm - nm) * kLog2e);
    m = nm;
}

// partial: [n_tiles][3][row_stride]  ->  stats: [3][N]
// One CTA = 32 rows x 32 tile lanes: lane j folds tiles j, j+32, ... in ascending order, then the 32
// lane results are folded in lane order by the first warp. Loads are 128-byte coalesced along the
// rows; the merge order depends only on n_tiles, so the result is the same on every run.
constexpr int kMergeRows = 32;
constexpr int kMergeLanes = 32;

__global__ void __launch_bounds__(kMergeRows * kMergeLanes)
merge_partials_kernel(const float* __restrict__ partial, int n_tiles, long long row_stride, int N,
                      float* __restrict__ stats) {
    __shared__ float sm[kMergeLanes][kMergeRows + 1], ss[kMergeLanes][kMergeRows + 1],
        st[kMergeLanes][kMergeRows + 1];
    const int r = threadIdx.x % kMergeRows;
    const int j = threadIdx.x / kMergeRows;
    const int row = blockIdx.x * kMergeRows + r;
    float m = -INFINITY, s = 0.f, t = -INFINITY;
    if (row < N) {
        for (int b = j; b < n_tiles; b += kMergeLanes) {
            const float* base = partial + static_cast<long long>(b) * 3 * row_stride + row;
            merge_ms(m, s, base[0], base[row_stride]);
            t = fmaxf(t, base[2 * row_stride]);
        }
    }
    sm[j][r] = m;
    ss[j][r] = s;
    st[j][r] = t;
    __syncthreads();
    if (j == 0 && row < N) {
        for (int k = 1; k < kMergeLanes; ++k) {
            merge_ms(m, s, sm[k][r], ss[k][r]);
            t = fmaxf(t, st[k][r]);
        }
        stats[row] = m;
        stats[static_cast<long long>(N) + row] = s;
        stats[2ll * N + row] = t;
    }
}

// stats: [R][3][N] -> lse[N], per-row loss (0 for ignored rows).
// A target outside the vocabulary that is not ignore_index leaves target_logit = -inf and the
// row loss +inf, as in the reference (tritium/ops/cross_entropy.py:240-244, 286-287).
__global__ void finalize_rows_kernel(const float* __restrict__ stats, int R, const void* tgt,
                                     int tgt_i64, int N, long long ignore_index,
                                     float* __restrict__ lse, float* __restrict__ loss_rows) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= N) return;
    float m = -INFINITY, s = 0.f, t = -INFINITY;
    for (int r = 0; r < R; ++r) {
        const float* base = stats + static_cast<long long>(r) * 3 * N + row;
        const float bm = base[0];
        const float bs = base[N];
        const float bt = base[2ll * N];
        merge_ms(m, s, bm, bs);
        t = fmaxf(t, bt);
    }
    const float l = m + logf(s);
    lse[row] = l;
    const bool valid = load_target(tgt, tgt_i64, row) != ignore_index;
    loss_rows[row] = valid ? (l - t) : 0.f;
}

// Fixed-shape reduction (one CTA of 1024 threads: strided serial sums, then a shared-memory tree):
// the summation order depends on N only, so the result is bit-identical from run to run.
__device__ __forceinline__ float block_sum_1024(float v, float* sh) {
    sh[threadIdx.x] = v;
    __syncthreads();
    for (int off = 512; off > 0; off >>= 1) {
        if (threadIdx.x < off) sh[threadIdx.x] += sh[threadIdx.x + off];
        __syncthreads();
    }
    const float r = sh[0];
    __syncthreads();
    return r;
}

// loss_rows[N] (+ targets) -> loss scalar (mean or sum) and the valid-row count.
__global__ void __launch_bounds__(1024)
reduce_loss_kernel(const float* __restrict__ loss_rows, const void* tgt, int tgt_i64, int N,
                   long long ignore_index, int mean, float* __restrict__ loss_out,
                   float* __restrict__ valid_count) {
    __shared__ float sh[1024];
    float acc = 0.f, cnt = 0.f;
    for (int i = threadIdx.x; i < N; i += 1024) {
        acc += loss_rows[i];
        cnt += (load_target(tgt, tgt_i64, i) != ignore_index) ? 1.f : 0.f;
    }
    const float total = block_sum_1024(acc, sh);
    const float count = block_sum_1024(cnt, sh);
    if (threadIdx.x == 0) {
        if (loss_out) *loss_out = mean ? total / count : total;  // count == 0 -> NaN, as torch
        if (valid_count) *valid_count = count;
    }
}

__global__ void __launch_bounds__(1024)
count_valid_kernel(const void* tgt, int tgt_i64, int N, long long ignore_index,
                   float* __restrict__ valid_count) {
    __shared__ float sh[1024];
    float cnt = 0.f;
    for (int i = threadIdx.x; i < N; i += 1024)
        cnt += (load_target(tgt, tgt_i64, i) != ignore_index) ? 1.f : 0.f;
    const float count = block_sum_1024(cnt, sh);
    if (threadIdx.x == 0) *valid_count = count;
}

// rowscale[i] = upstream gradient factor of row i (0 for ignored rows); grad_out stays on device.
__global__ void rowscale_kernel(const void* tgt, int tgt_i64, int N, long long ignore_index,
                                const float* __restrict__ grad_out, int per_row, int mean,
                                const float* __restrict__ valid_count,
                                float* __restrict__ rowscale) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= N) return;
    const bool valid = load_target(tgt, tgt_i64, row) != ignore_index;
    float g = per_row ? grad_out[row] : grad_out[0];
    if (mean) g = g / *valid_count;
    rowscale[row] = valid ? g : 0.f;
}

}  // namespace lce
