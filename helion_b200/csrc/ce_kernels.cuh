// Cross-entropy on materialised logits (the reference's tritium.cross_entropy / cross_entropy_backward,
// tritium/ops/cross_entropy.py:36-100): bandwidth-bound row kernels that share the statistics format,
// the merge and the loss reduction with the fused linear-cross-entropy path.
//
// A row is cut into chunks of 256 threads x 4 vectors of 16 bytes (8192 16-bit or 4096 fp32 columns),
// vectorised when the row pitch allows. Forward: a CTA walks up to 8 consecutive chunks of one row
// with the next chunk's loads in flight while it reduces the current one, and ends with
// (max, sum exp(z - max), target logit or -inf) - the same three numbers the GEMM epilogue emits per
// vocabulary tile - so rows longer than one CTA's span go through merge_partials_kernel<true>; shorter
// rows are finalised in place. Backward is a pure streaming pass, one CTA per (row, chunk).
// Unlike the reference there is no limit on the vocabulary size (it holds a whole row in one
// program and refuses next_pow2(V) > 131072).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "row_kernels.cuh"

namespace lce {

constexpr int kCeThreads = 256;
constexpr int kCeVectors = 4;       // 16-byte vectors per thread and chunk
constexpr int kCeChunksPerCta = 8;  // forward: consecutive chunks one CTA walks (next one prefetched)

template <class T>
struct CeTile {
    static constexpr int kVec = 16 / sizeof(T);
    static constexpr int kPerThread = kCeVectors * kVec;     // 32 (16-bit) or 16 (fp32)
    static constexpr int kChunk = kCeThreads * kPerThread;   // columns per chunk: 8192 or 4096
};

// Element j of vector g of this thread is column col0 + (g * 256 + thread) * VEC + j, so that a warp
// reads consecutive 16-byte vectors. Raw 16-byte loads (no conversion yet) so that the loads of the
// next chunk can be in flight while the current one is reduced.
template <class T, bool VECTOR>
__device__ __forceinline__ void ce_load_raw(const T* __restrict__ row, long long col0, long long V,
                                            uint4 (&raw)[kCeVectors]) {
    constexpr int VEC = CeTile<T>::kVec;
#pragma unroll
    for (int g = 0; g < kCeVectors; ++g) {
        const long long c = col0 + (static_cast<long long>(g) * kCeThreads + threadIdx.x) * VEC;
        if (VECTOR && c + VEC <= V) {
            raw[g] = *reinterpret_cast<const uint4*>(row + c);
        } else {
            alignas(16) T tmp[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) tmp[j] = (c + j < V) ? row[c + j] : Cvt<T>::from_f(0.f);
            raw[g] = *reinterpret_cast<const uint4*>(tmp);
        }
    }
}

// Converts vector g of this thread to floats; columns at or beyond V become `fill`.
template <class T>
__device__ __forceinline__ void ce_unpack_one(const uint4& raw, long long col0, int g, long long V, float fill,
                                              float (&v)[CeTile<T>::kVec]) {
    constexpr int VEC = CeTile<T>::kVec;
    const long long c = col0 + (static_cast<long long>(g) * kCeThreads + threadIdx.x) * VEC;
    alignas(16) T tmp[VEC];
    *reinterpret_cast<uint4*>(tmp) = raw;
    if (c + VEC <= V) {  // whole vector in range (one test per vector, not per element)
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = Cvt<T>::to_f(tmp[j]);
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = (c + j < V) ? Cvt<T>::to_f(tmp[j]) : fill;
    }
}

// Folds PER logits into a running (max, sum-exp). Four independent chains for the max and for the sum
// (the serial versions stall on FMNMX / FADD latency with this few warps per SM); the order of the
// additions is fixed, so the result is the same on every run.
template <int PER>
__device__ __forceinline__ void ce_fold(const float (&v)[PER], float& m, float& s) {
    static_assert(PER % 4 == 0, "four chains");
    float m0 = v[0], m1 = v[1], m2 = v[2], m3 = v[3];
#pragma unroll
    for (int j = 4; j < PER; j += 4) {
        m0 = fmaxf(m0, v[j]);
        m1 = fmaxf(m1, v[j + 1]);
        m2 = fmaxf(m2, v[j + 2]);
        m3 = fmaxf(m3, v[j + 3]);
    }
    const float nm = fmaxf(m, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
    const float nm2 = (nm == -INFINITY) ? 0.f : nm * kLog2e;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j += 4) {
        a0 += ptx::ex2(fmaf(v[j], kLog2e, -nm2));
        a1 += ptx::ex2(fmaf(v[j + 1], kLog2e, -nm2));
        a2 += ptx::ex2(fmaf(v[j + 2], kLog2e, -nm2));
        a3 += ptx::ex2(fmaf(v[j + 3], kLog2e, -nm2));
    }
    s = s * ptx::ex2(fmaf(m, kLog2e, -nm2)) + ((a0 + a1) + (a2 + a3));
    m = nm;
}

// Fast fold of one whole in-range chunk straight from the raw 16-byte vectors of a 16-bit type: the chunk
// maximum is taken on packed pairs (exact: the maximum of two 16-bit floats is one of them), each word is
// split into its two values with one instruction each, and four independent chains sum the exponentials.
// About 5 instructions per logit where the general path needs 16 (a capture of the forward on 4096 x 50304
// bf16 showed it issue-bound at 0.82 instructions per scheduler cycle, not memory-bound). The order of the
// additions is fixed, so the result is the same on every run.
template <class T>
__device__ __forceinline__ void ce_fold_raw16(const uint4 (&raw)[kCeVectors], float& m, float& s) {
    static_assert(sizeof(T) == 2, "16-bit types");
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    unsigned w[4 * kCeVectors];
#pragma unroll
    for (int g = 0; g < kCeVectors; ++g) {
        w[4 * g + 0] = raw[g].x;
        w[4 * g + 1] = raw[g].y;
        w[4 * g + 2] = raw[g].z;
        w[4 * g + 3] = raw[g].w;
    }
    float cm;
    if constexpr (kBf16) {
        __nv_bfloat162 mx = *reinterpret_cast<const __nv_bfloat162*>(&w[0]);
#pragma unroll
        for (int i = 1; i < 4 * kCeVectors; ++i) mx = __hmax2(mx, *reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        cm = fmaxf(__low2float(mx), __high2float(mx));
    } else {
        __half2 mx = *reinterpret_cast<const __half2*>(&w[0]);
#pragma unroll
        for (int i = 1; i < 4 * kCeVectors; ++i) mx = __hmax2(mx, *reinterpret_cast<const __half2*>(&w[i]));
        cm = fmaxf(__low2float(mx), __high2float(mx));
    }
    const float nm = fmaxf(m, cm);
    const float nm2 = (nm == -INFINITY) ? 0.f : nm * kLog2e;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4 * kCeVectors; i += 2) {
        float l0, h0, l1, h1;
        if constexpr (kBf16) {  // a bf16 is the upper half of the float with the same value
            l0 = __uint_as_float(w[i] << 16);
            h0 = __uint_as_float(w[i] & 0xffff0000u);
            l1 = __uint_as_float(w[i + 1] << 16);
            h1 = __uint_as_float(w[i + 1] & 0xffff0000u);
        } else {
            const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&w[i + 1]));
            l0 = p0.x;
            h0 = p0.y;
            l1 = p1.x;
            h1 = p1.y;
        }
        a0 += ptx::ex2(fmaf(l0, kLog2e, -nm2));
        a1 += ptx::ex2(fmaf(h0, kLog2e, -nm2));
        a2 += ptx::ex2(fmaf(l1, kLog2e, -nm2));
        a3 += ptx::ex2(fmaf(h1, kLog2e, -nm2));
    }
    s = s * ptx::ex2(fmaf(m, kLog2e, -nm2)) + ((a0 + a1) + (a2 + a3));
    m = nm;
}

// The logit in register slot `slot` (0 .. kPerThread-1) of this thread, from the raw vectors.
template <class T>
__device__ __forceinline__ float ce_pick_raw(const uint4 (&raw)[kCeVectors], int slot) {
    constexpr int VEC = CeTile<T>::kVec;
    float out = -INFINITY;
#pragma unroll
    for (int g = 0; g < kCeVectors; ++g) {
        alignas(16) T tmp[VEC];
        *reinterpret_cast<uint4*>(tmp) = raw[g];
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (g * VEC + j == slot) out = Cvt<T>::to_f(tmp[j]);
    }
    return out;
}

// Index (0 .. kPerThread-1) of the register of THIS thread that holds column `target`, or -1.
template <class T>
__device__ __forceinline__ int ce_target_slot(long long col0, long long target) {
    constexpr int VEC = CeTile<T>::kVec;
    const long long rel = target - col0;
    if (rel < 0 || rel >= CeTile<T>::kChunk) return -1;
    const int group = static_cast<int>(rel / (kCeThreads * VEC));
    const int within = static_cast<int>(rel % (kCeThreads * VEC));
    return (within / VEC == static_cast<int>(threadIdx.x)) ? group * VEC + within % VEC : -1;
}

// grid.x = N * n_groups; CTA (row, group) walks chunks [group * kCeChunksPerCta, ...) of its row with a
// thread-local online (max, sum-exp), prefetching the next chunk, and reduces once at the end.
// FINAL (n_groups == 1): writes lse / loss_rows; else partial statistics
// partial[(group*3 + c) * row_stride + row].
template <class T, bool VECTOR, bool FINAL>
__global__ void __launch_bounds__(kCeThreads, 4)  // 64 registers: 1024 threads x 64 B of loads in flight per SM
ce_row_stats_kernel(const T* __restrict__ logits, const void* tgt, int tgt_i64, int N, long long V, int n_chunks,
                    int n_groups, float* __restrict__ partial, long long row_stride, long long ignore_index,
                    float* __restrict__ lse, float* __restrict__ loss_rows) {
    __shared__ float wm[kCeThreads / 32], ws_[kCeThreads / 32], wt[kCeThreads / 32];
    constexpr int VEC = CeTile<T>::kVec;
    constexpr int PER = CeTile<T>::kPerThread;
    const int row = blockIdx.x / n_groups;
    const int group = blockIdx.x % n_groups;
    const int c_begin = group * kCeChunksPerCta;
    const int c_end = min(n_chunks, c_begin + kCeChunksPerCta);
    const T* rowp = logits + static_cast<long long>(row) * V;
    const long long target = load_target(tgt, tgt_i64, row);

    float m = -INFINITY, s = 0.f, t = -INFINITY;
    uint4 next[kCeVectors];
    ce_load_raw<T, VECTOR>(rowp, static_cast<long long>(c_begin) * CeTile<T>::kChunk, V, next);
    for (int c = c_begin; c < c_end; ++c) {
        const long long col0 = static_cast<long long>(c) * CeTile<T>::kChunk;
        uint4 cur[kCeVectors];
#pragma unroll
        for (int g = 0; g < kCeVectors; ++g) cur[g] = next[g];
        if (c + 1 < c_end) ce_load_raw<T, VECTOR>(rowp, col0 + CeTile<T>::kChunk, V, next);
        if constexpr (sizeof(T) == 2) {
            if (col0 + CeTile<T>::kChunk <= V) {  // whole chunk in range (the same for every thread of the CTA)
                ce_fold_raw16<T>(cur, m, s);
                const int slot = ce_target_slot<T>(col0, target);
                if (slot >= 0) t = ce_pick_raw<T>(cur, slot);  // at most one thread of the CTA, in one chunk
                continue;
            }
        }
        float v[PER];
#pragma unroll
        for (int g = 0; g < kCeVectors; ++g) {
            float part[VEC];
            ce_unpack_one<T>(cur[g], col0, g, V, -INFINITY, part);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[g * VEC + j] = part[j];
        }
        ce_fold<PER>(v, m, s);
        const int slot = ce_target_slot<T>(col0, target);
        if (slot >= 0) {  // at most one thread of the CTA, in one chunk
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (j == slot) t = v[j];
        }
    }
    // fixed butterfly inside the warp, then the 8 warps in order: deterministic
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, off);
        const float os = __shfl_xor_sync(0xffffffffu, s, off);
        const float ot = __shfl_xor_sync(0xffffffffu, t, off);
        merge_ms(m, s, om, os);
        t = fmaxf(t, ot);
    }
    if ((threadIdx.x & 31) == 0) {
        wm[threadIdx.x >> 5] = m;
        ws_[threadIdx.x >> 5] = s;
        wt[threadIdx.x >> 5] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < kCeThreads / 32; ++k) {
            merge_ms(m, s, wm[k], ws_[k]);
            t = fmaxf(t, wt[k]);
        }
        if constexpr (FINAL) {
            const float l = m + logf(s);
            lse[row] = l;
            loss_rows[row] = (target != ignore_index) ? (l - t) : 0.f;
        } else {
            float* base = partial + static_cast<long long>(group) * 3 * row_stride + row;
            base[0] = m;
            base[row_stride] = s;
            base[2 * row_stride] = t;
        }
    }
}

// dlogits = (exp(z - lse[row]) - [col == target[row]]) * rowscale[row], in the logits dtype
// (reference: tritium/ops/cross_entropy.py:71-100; rowscale carries grad_out / divisor).
template <class T, bool VECTOR>
__global__ void __launch_bounds__(kCeThreads, 5)
ce_backward_kernel(const T* __restrict__ logits, const void* tgt, int tgt_i64, long long V, int n_chunks,
                   const float* __restrict__ lse, const float* __restrict__ rowscale, T* __restrict__ dlogits) {
    constexpr int VEC = CeTile<T>::kVec;
    constexpr int PER = CeTile<T>::kPerThread;
    const int row = blockIdx.x / n_chunks;
    const int chunk = blockIdx.x % n_chunks;
    const long long col0 = static_cast<long long>(chunk) * CeTile<T>::kChunk;
    const T* rowp = logits + static_cast<long long>(row) * V;
    T* outp = dlogits + static_cast<long long>(row) * V;
    const long long target = load_target(tgt, tgt_i64, row);
    const float l2 = lse[row] * kLog2e;
    const float sc = rowscale[row];

    float v[PER];
#pragma unroll
    for (int g = 0; g < kCeVectors; ++g) {  // load and convert vector by vector: fewest live registers
        const long long c = col0 + (static_cast<long long>(g) * kCeThreads + threadIdx.x) * VEC;
        if (VECTOR && c + VEC <= V) {
            alignas(16) T tmp[VEC];
            *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(rowp + c);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[g * VEC + j] = Cvt<T>::to_f(tmp[j]);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[g * VEC + j] = (c + j < V) ? Cvt<T>::to_f(rowp[c + j]) : 0.f;
        }
    }
    const int slot = ce_target_slot<T>(col0, target);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        float grad = (sc == 0.f) ? 0.f : ptx::ex2(fmaf(v[j], kLog2e, -l2)) * sc;
        if (j == slot) grad -= sc;
        v[j] = grad;
    }
#pragma unroll
    for (int g = 0; g < kCeVectors; ++g) {
        const long long c = col0 + (static_cast<long long>(g) * kCeThreads + threadIdx.x) * VEC;
        if (VECTOR && c + VEC <= V) {
            alignas(16) T tmp[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) tmp[j] = Cvt<T>::from_f(v[g * VEC + j]);
            *reinterpret_cast<uint4*>(outp + c) = *reinterpret_cast<const uint4*>(tmp);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (c + j < V) outp[c + j] = Cvt<T>::from_f(v[g * VEC + j]);
        }
    }
}

}  // namespace lce
