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

// FINALIZE = false: writes the merged statistics (stats [3][N]) for a later cross-shard merge.
// FINALIZE = true: this shard is the whole vocabulary, so logsumexp and the per-row loss are
// written directly (lse[N], loss_rows[N]; 0 for ignored rows) and the statistics never reach memory.
template <bool FINALIZE>
__global__ void __launch_bounds__(kMergeRows * kMergeLanes)
merge_partials_kernel(const float* partial, int n_tiles, long long row_stride, int N,
                      float* __restrict__ stats, const void* tgt, int tgt_i64, long long ignore_index,
                      float* __restrict__ lse, float* __restrict__ loss_rows) {
    __shared__ float sm[kMergeLanes][kMergeRows + 1], ss[kMergeLanes][kMergeRows + 1],
        st[kMergeLanes][kMergeRows + 1];
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // `partial` is the preceding GEMM's output (this kernel may have started under its tail)
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
        if constexpr (FINALIZE) {
            const float l = m + logf(s);
            lse[row] = l;
            loss_rows[row] = (load_target(tgt, tgt_i64, row) != ignore_index) ? (l - t) : 0.f;
        } else {
            stats[row] = m;
            stats[static_cast<long long>(N) + row] = s;
            stats[2ll * N + row] = t;
        }
    }
}

// Small batches (N <= 1024) of an unsharded vocabulary: merge, finalize and the loss reduction in ONE launch
// of one CTA. The 1024 threads form R = roundup(N, 32) row lanes x J = 1024 / R tile lanes (at most 32): tile
// lane j folds tiles j, j + J, ... of its row in ascending order, tile lane 0 then folds the J results in lane
// order, and the rows are added by the fixed tree of block_sum_1024 - the same bits on every run (not the
// bits of the three-kernel path, which folds a row's tiles in a different, equally fixed order).
__device__ __forceinline__ float block_sum_1024(float v, float* sh);

__global__ void __launch_bounds__(1024)
merge_finalize_small_kernel(const float* partial, int n_tiles, long long row_stride, int N,
                            const void* tgt, int tgt_i64, long long ignore_index, int reduction,
                            float* __restrict__ lse, float* __restrict__ loss, float* __restrict__ valid_count) {
    __shared__ float sh[1024], sm[1024], ss[1024], st[1024];
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // `partial` is the preceding GEMM's output
    const int R = (N + 31) / 32 * 32;
    const int J = min(32, 1024 / R);
    const int r = threadIdx.x % R, j = threadIdx.x / R;
    float m = -INFINITY, s = 0.f, t = -INFINITY;
    if (j < J && r < N) {
        for (int b = j; b < n_tiles; b += J) {
            const float* base = partial + static_cast<long long>(b) * 3 * row_stride + r;
            merge_ms(m, s, base[0], base[row_stride]);
            t = fmaxf(t, base[2 * row_stride]);
        }
    }
    sm[threadIdx.x] = m;
    ss[threadIdx.x] = s;
    st[threadIdx.x] = t;
    __syncthreads();
    float nll = 0.f, cnt = 0.f;
    if (j == 0 && r < N) {
        for (int k = 1; k < J; ++k) {
            merge_ms(m, s, sm[k * R + r], ss[k * R + r]);
            t = fmaxf(t, st[k * R + r]);
        }
        const float l = m + logf(s);
        lse[r] = l;
        const bool valid = load_target(tgt, tgt_i64, r) != ignore_index;
        nll = valid ? (l - t) : 0.f;
        cnt = valid ? 1.f : 0.f;
        if (reduction == 0) loss[r] = nll;  // LCE_REDUCTION_NONE
    }
    if (reduction == 0 && valid_count == nullptr) return;
    const float total = block_sum_1024(nll, sh);
    const float count = block_sum_1024(cnt, sh);
    if (threadIdx.x == 0) {
        if (reduction == 1) *loss = total / count;  // mean; count == 0 -> NaN, as torch
        else if (reduction == 2) *loss = total;
        if (valid_count) *valid_count = count;
    }
}

// The same tail inside the forward GEMM launch: run by all kGemmThreads threads of the CTA that finished last,
// after every CTA's partial statistics are visible. Thread t takes rows t, t + kGemmThreads, ... and folds a
// row's tiles in ascending order; the rows are then added lane by lane, warp by warp - fixed orders, so the
// bits are the same on every run (they are not the bits of the separate-launch tails, whose orders differ).
// The partials were written by other SMs during this launch: they are read past L1 (__ldcg).
__device__ inline void EpiStats::finish(const Params& p) {
    __shared__ float red_a[kGemmThreads / 32], red_b[kGemmThreads / 32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float nll = 0.f, cnt = 0.f;
    for (int r = t; r < p.rows; r += kGemmThreads) {
        float m = -INFINITY, s = 0.f, tl = -INFINITY;
        for (int b = 0; b < p.fin_n_tiles; ++b) {
            const float* base = p.partial + static_cast<long long>(b) * 3 * p.row_stride + r;
            merge_ms(m, s, __ldcg(base), __ldcg(base + p.row_stride));
            tl = fmaxf(tl, __ldcg(base + 2 * p.row_stride));
        }
        const float l = m + logf(s);
        p.fin_lse[r] = l;
        const bool valid = load_target(p.tgt, p.tgt_i64, r) != p.fin_ignore_index;
        const float row_nll = valid ? (l - tl) : 0.f;
        if (p.fin_reduction == 0) p.fin_loss[r] = row_nll;  // LCE_REDUCTION_NONE
        nll += row_nll;
        cnt += valid ? 1.f : 0.f;
    }
    if (p.fin_reduction == 0 && p.fin_valid_count == nullptr) return;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        nll += __shfl_xor_sync(0xffffffffu, nll, off);
        cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
    }
    if (lane == 0) {
        red_a[warp] = nll;
        red_b[warp] = cnt;
    }
    __syncthreads();
    if (t == 0) {
        float total = 0.f, count = 0.f;
        for (int k = 0; k < kGemmThreads / 32; ++k) {
            total += red_a[k];
            count += red_b[k];
        }
        if (p.fin_reduction == 1) *p.fin_loss = total / count;  // mean; count == 0 -> NaN, as torch
        else if (p.fin_reduction == 2) *p.fin_loss = total;
        if (p.fin_valid_count) *p.fin_valid_count = count;
    }
}

// Greedy head: partial [n_tiles][3][row_stride] of EpiTop1 -> token[N] (global vocabulary index of the
// largest logit; the lowest index on ties), logprob[N] = log softmax at that token, optionally lse[N].
// Same CTA shape and fold order as merge_partials_kernel.
__device__ __forceinline__ void merge_top1(float& m, float& s, int& a, float bm, float bs, int ba) {
    if (bm > m || (bm == m && ba < a)) a = ba;
    merge_ms(m, s, bm, bs);
}

__global__ void __launch_bounds__(kMergeRows * kMergeLanes)
merge_top1_kernel(const float* partial, int n_tiles, long long row_stride, int N, long long vocab_start,
                  long long* __restrict__ token, float* __restrict__ logprob, float* __restrict__ lse) {
    __shared__ float sm[kMergeLanes][kMergeRows + 1], ss[kMergeLanes][kMergeRows + 1];
    __shared__ int sa[kMergeLanes][kMergeRows + 1];
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // `partial` is the preceding GEMM's output
    const int r = threadIdx.x % kMergeRows, j = threadIdx.x / kMergeRows;
    const int row = blockIdx.x * kMergeRows + r;
    float m = -INFINITY, s = 0.f;
    int a = 0x7fffffff;
    if (row < N) {
        for (int b = j; b < n_tiles; b += kMergeLanes) {
            const float* base = partial + static_cast<long long>(b) * 3 * row_stride + row;
            merge_top1(m, s, a, base[0], base[row_stride], __float_as_int(base[2 * row_stride]));
        }
    }
    sm[j][r] = m;
    ss[j][r] = s;
    sa[j][r] = a;
    __syncthreads();
    if (j == 0 && row < N) {
        for (int k = 1; k < kMergeLanes; ++k) merge_top1(m, s, a, sm[k][r], ss[k][r], sa[k][r]);
        const float log_s = logf(s);
        token[row] = vocab_start + a;
        logprob[row] = -log_s;
        if (lse != nullptr) lse[row] = m + log_s;
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
// valid_count == nullptr (small N): every CTA counts the valid rows itself instead of waiting for a
// separate counting launch; the count is an integer below 2^24, so any summation order is exact.
__global__ void __launch_bounds__(256)
rowscale_kernel(const void* tgt, int tgt_i64, int N, long long ignore_index,
                const float* __restrict__ grad_out, int per_row, int mean,
                const float* __restrict__ valid_count, float* __restrict__ rowscale) {
    __shared__ int warp_counts[8];
    __shared__ float count_sh;
    ptx::grid_dep_launch();  // the GEMM that follows may set itself up now; it waits for this grid before it reads
    float count = 1.f;
    if (mean) {
        if (valid_count != nullptr) {
            count = *valid_count;
        } else {
            int c = 0;
            for (int i = threadIdx.x; i < N; i += 256) c += load_target(tgt, tgt_i64, i) != ignore_index;
            c = __reduce_add_sync(0xffffffffu, c);
            if ((threadIdx.x & 31) == 0) warp_counts[threadIdx.x >> 5] = c;
            __syncthreads();
            if (threadIdx.x == 0) {
                int total = 0;
                for (int k = 0; k < 8; ++k) total += warp_counts[k];
                count_sh = static_cast<float>(total);
            }
            __syncthreads();
            count = count_sh;
        }
    }
    const int row = blockIdx.x * 256 + threadIdx.x;
    if (row >= N) return;
    const bool valid = load_target(tgt, tgt_i64, row) != ignore_index;
    float g = per_row ? grad_out[row] : grad_out[0];
    if (mean) g = g / count;
    rowscale[row] = valid ? g : 0.f;
}

// Adds the `slices` slabs a split-K launch left in tile-blocked scratch (see EpiStore) in slice order
// and writes the [rows, cols] result row-major. One thread per (tile, column quad, row): reads are
// 16-byte coalesced along the rows of a tile.
template <class T>
__global__ void splitk_reduce_kernel(const float* scratch, int slices, long long slab_floats,
                                     int m_tiles, int n_tiles, int bn, int rows, int cols,
                                     T* __restrict__ out, long long ldo) {
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();  // `scratch` holds the slices of the preceding GEMM
    const long long quads = static_cast<long long>(m_tiles) * n_tiles * (bn / 4) * kBM;
    for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < quads;
         q += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row_in_tile = static_cast<int>(q % kBM);
        const long long rest = q / kBM;
        const int c4 = static_cast<int>(rest % (bn / 4));
        const long long tile = rest / (bn / 4);
        const int n_tile = static_cast<int>(tile % n_tiles);
        const int m_tile = static_cast<int>(tile / n_tiles);
        const int row = m_tile * kBM + row_in_tile;
        const int col = n_tile * bn + c4 * 4;
        if (row >= rows || col >= cols) continue;
        const float4* sp = reinterpret_cast<const float4*>(scratch) + q;
        float4 acc = sp[0];
        for (int s = 1; s < slices; ++s) {
            const float4 v = sp[static_cast<long long>(s) * (slab_floats / 4)];
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        T* dst = out + static_cast<long long>(row) * ldo + col;
        const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col + j < cols) dst[j] = Cvt<T>::from_f(vals[j]);
    }
}

// Second half of the dX reduce-scatter + all-gather across vocabulary shards. `staging` is THIS GPU's
// buffer [world][rows_per_rank][H] fp32, filled by every rank's dX epilogue (slot = sending rank) with the
// partial sums of the rows this GPU owns. Each thread adds the `world` partials of four columns in rank
// order (the same order on every run), rounds once to T and stores the result into the final dX buffer of
// EVERY rank (peer stores), rows [row0, row0 + n_rows).
struct PeerOutputs {
    void* out[kMaxPeers];
};

template <class T>
__global__ void dx_reduce_gather_kernel(const float* __restrict__ staging, int world, long long rows_per_rank,
                                        long long H, long long row0, long long n_rows, PeerOutputs outs) {
    const long long quads_per_row = H / 4;
    const long long total = n_rows * quads_per_row;
    const long long slot_floats = rows_per_rank * H;
    for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < total;
         q += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = q / quads_per_row;
        const long long c = (q % quads_per_row) * 4;
        const float* src = staging + r * H + c;
        float4 acc = *reinterpret_cast<const float4*>(src);
        for (int k = 1; k < world; ++k) {
            const float4 v = *reinterpret_cast<const float4*>(src + k * slot_floats);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        alignas(8) T packed[4] = {Cvt<T>::from_f(acc.x), Cvt<T>::from_f(acc.y), Cvt<T>::from_f(acc.z),
                                  Cvt<T>::from_f(acc.w)};
        for (int k = 0; k < world; ++k) {
            T* dst = static_cast<T*>(outs.out[k]) + (row0 + r) * H + c;
            if constexpr (sizeof(T) == 2) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(packed);
            else *reinterpret_cast<float4*>(dst) = acc;
        }
    }
}

// The reduce half alone: sums the `world` staging slots of this rank's row slice in rank order, rounds once
// and writes the slice to LOCAL memory (out is [rows_per_rank, H]); an all-gather by the caller follows.
template <class T>
__global__ void dx_reduce_slice_kernel(const float* __restrict__ staging, int world, long long rows_per_rank,
                                       long long H, long long n_rows, T* __restrict__ out) {
    const long long quads_per_row = H / 4;
    const long long total = n_rows * quads_per_row;
    const long long slot_floats = rows_per_rank * H;
    for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < total;
         q += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float* src = staging + q * 4;
        float4 acc = *reinterpret_cast<const float4*>(src);
        for (int k = 1; k < world; ++k) {
            const float4 v = *reinterpret_cast<const float4*>(src + k * slot_floats);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        T* dst = out + q * 4;
        if constexpr (sizeof(T) == 2) {
            alignas(8) T packed[4] = {Cvt<T>::from_f(acc.x), Cvt<T>::from_f(acc.y), Cvt<T>::from_f(acc.z),
                                      Cvt<T>::from_f(acc.w)};
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(packed);
        } else {
            *reinterpret_cast<float4*>(dst) = acc;
        }
    }
}

}  // namespace lce
