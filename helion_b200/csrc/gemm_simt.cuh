// CUDA-core GEMM core with the same epilogue contract as the tcgen05 core.
//
//   D[m, n] = sum_k A[m, k] * B[n, k]     fp32 FMA, k ascending, no tensor cores
//
// It serves the inputs the tensor-core path cannot take: fp32 tensors (the reference demands
// 1e-5 agreement with fp32 torch there, so TF32 is not an option), hidden sizes that are not a
// multiple of 8 (TMA needs 16-byte row pitches) and unaligned bases. Operands are addressed through
// explicit (row, k) strides, so any majorness works.
//
// One CTA of 256 threads computes a 128 x 128 tile. Thread (ty, tx) of a 16 x 16 grid keeps an 8 x 8
// block of it in registers, as rows {ty*4.., 64 + ty*4..} x columns {tx*4.., 64 + tx*4..}: four
// conflict-free 16-byte shared-memory loads feed 64 FMAs. The operand tiles are double-buffered in
// shared memory and the next ones are fetched into registers while the current ones are multiplied
// (one barrier per 8 k). When the contraction is done the tile goes through shared memory in two
// 64-column halves so that the epilogue sees it the way every epilogue expects: one thread = one
// row, 32 columns at a time (threads 0..127).
#pragma once

#include "epilogues.cuh"

namespace lce {

constexpr int kSimtBN = 128;
constexpr int kSimtBK = 8;
constexpr int kSimtThreads = 256;
constexpr int kSimtPitch = 128 + 4;   // operand tiles [k][mn] in floats: rows stay 16-byte aligned, the pad
                                      // spreads a k-contiguous deposit over the banks
constexpr int kSimtCPitch = 64 + 4;   // one 64-column half of the C tile
constexpr int kSimtLoads = 128 * kSimtBK / kSimtThreads;  // 8 elements of each operand per thread and k step
static_assert(kBM == 128, "the thread layout below is written for 128 x 128 tiles");

template <class T>
struct SimtOperand {
    const T* ptr;
    long long stride_mn;  // elements between consecutive m (resp. n)
    long long stride_k;   // elements between consecutive k
    int extent_mn;        // valid m (resp. n)
};

// One thread's share of a (128 x 16) operand tile: element i sits at (mn_t + i * mn_step,
// k_t + i * k_step) of the tile, chosen so that consecutive threads walk the contiguous direction
// of the operand in global memory.
struct SimtLane {
    int mn_t, k_t, mn_step, k_step;
};

__device__ __forceinline__ SimtLane simt_lane(bool k_contiguous, int t) {
    SimtLane l;
    if (k_contiguous) { l.k_t = t % kSimtBK; l.mn_t = t / kSimtBK; l.mn_step = kSimtThreads / kSimtBK; l.k_step = 0; }
    else { l.mn_t = t % 128; l.k_t = t / 128; l.mn_step = 0; l.k_step = kSimtThreads / 128; }
    return l;
}

template <class T>
__device__ __forceinline__ void simt_fetch(const SimtOperand<T>& op, const SimtLane& l, int mn0, int k0, int k_end,
                                           float (&r)[kSimtLoads]) {
    const T* p = op.ptr + static_cast<long long>(mn0 + l.mn_t) * op.stride_mn +
                 static_cast<long long>(k0 + l.k_t) * op.stride_k;
    const long long step = l.mn_step * op.stride_mn + l.k_step * op.stride_k;
#pragma unroll
    for (int i = 0; i < kSimtLoads; ++i) {
        r[i] = 0.f;
        if (mn0 + l.mn_t + i * l.mn_step < op.extent_mn && k0 + l.k_t + i * l.k_step < k_end)
            r[i] = Cvt<T>::to_f(p[i * step]);
    }
}

__device__ __forceinline__ void simt_deposit(float* tile, const SimtLane& l, const float (&r)[kSimtLoads]) {
#pragma unroll
    for (int i = 0; i < kSimtLoads; ++i)
        tile[(l.k_t + i * l.k_step) * kSimtPitch + l.mn_t + i * l.mn_step] = r[i];
}

template <class T, class Epi>
__global__ void __launch_bounds__(kSimtThreads, 2)
gemm_simt_kernel(SimtOperand<T> A, SimtOperand<T> B, int K, int m_tiles, int n_tiles, int k_splits,
                 const typename Epi::Params ep) {
    // main loop: two buffers of As[k][m] + Bs[k][n]; afterwards the same memory stages half a C tile
    constexpr int kTileFloats = kSimtBK * kSimtPitch;
    __shared__ __align__(16) float smem[128 * kSimtCPitch];
    static_assert(4 * kTileFloats <= 128 * kSimtCPitch, "two buffers of both operand tiles fit in the C staging area");

    const int t = threadIdx.x;
    const int ty = t >> 4, tx = t & 15;
    const SimtLane la = simt_lane(A.stride_k == 1, t), lb = simt_lane(B.stride_k == 1, t);
    // k_splits > 1: work item = (tile, slice of the contraction); the epilogue stores slices side by side
    // (kStoreSlice) and splitk_reduce_kernel adds them in slice order.
    const int total_tiles = m_tiles * n_tiles;
    const int k_per_slice = ((K + k_splits - 1) / k_splits + kSimtBK - 1) / kSimtBK * kSimtBK;
    for (int work = blockIdx.x; work < total_tiles * k_splits; work += gridDim.x) {
        const int tile = work % total_tiles;
        const int k_slice = work / total_tiles;
        const int k_begin = k_slice * k_per_slice;
        const int k_end = min(K, k_begin + k_per_slice);
        const int n_tile = tile % n_tiles;
        const int m_tile = tile / n_tiles;
        const int m0 = m_tile * kBM;
        const int n0 = n_tile * kSimtBN;

        float acc[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

        float ra[kSimtLoads], rb[kSimtLoads];
        simt_fetch<T>(A, la, m0, k_begin, k_end, ra);
        simt_fetch<T>(B, lb, n0, k_begin, k_end, rb);
        simt_deposit(smem, la, ra);
        simt_deposit(smem + kTileFloats, lb, rb);
        __syncthreads();
        int cur = 0;
        for (int k0 = k_begin; k0 < k_end; k0 += kSimtBK) {
            const bool more = k0 + kSimtBK < k_end;
            if (more) {  // in flight while this step multiplies
                simt_fetch<T>(A, la, m0, k0 + kSimtBK, k_end, ra);
                simt_fetch<T>(B, lb, n0, k0 + kSimtBK, k_end, rb);
            }
            const float* As = smem + cur * 2 * kTileFloats;
            const float* Bs = As + kTileFloats;
#pragma unroll
            for (int k = 0; k < kSimtBK; ++k) {
                const float4 a0 = *reinterpret_cast<const float4*>(As + k * kSimtPitch + ty * 4);
                const float4 a1 = *reinterpret_cast<const float4*>(As + k * kSimtPitch + 64 + ty * 4);
                const float4 b0 = *reinterpret_cast<const float4*>(Bs + k * kSimtPitch + tx * 4);
                const float4 b1 = *reinterpret_cast<const float4*>(Bs + k * kSimtPitch + 64 + tx * 4);
                const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            if (more) {
                float* nxt = smem + (cur ^ 1) * 2 * kTileFloats;
                simt_deposit(nxt, la, ra);
                simt_deposit(nxt + kTileFloats, lb, rb);
            }
            __syncthreads();
            cur ^= 1;
        }

        // C tile through shared memory, one 64-column half at a time: blocked registers -> one row per thread
        TileCtx tc{m_tile, n_tile, n_tiles, t & 127, kSimtBN, k_slice, nullptr};
        typename Epi::State st;
        if (t < kBM) Epi::begin(st, ep, tc);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int row = (i < 4 ? 0 : 64) + ty * 4 + (i & 3);
                *reinterpret_cast<float4*>(&smem[row * kSimtCPitch + tx * 4]) =
                    make_float4(acc[i][half * 4 + 0], acc[i][half * 4 + 1], acc[i][half * 4 + 2], acc[i][half * 4 + 3]);
            }
            __syncthreads();
            if (t < kBM) {
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    float v[32];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 x = *reinterpret_cast<const float4*>(&smem[t * kSimtCPitch + c * 32 + q * 4]);
                        v[4 * q + 0] = x.x;
                        v[4 * q + 1] = x.y;
                        v[4 * q + 2] = x.z;
                        v[4 * q + 3] = x.w;
                    }
                    Epi::chunk(st, ep, tc, half * 64 + c * 32, v);
                }
            }
            __syncthreads();  // the staging area is free again (next half, or operand tiles of the next item)
        }
        if (t < kBM) Epi::end(st, ep, tc);
    }
}

}  // namespace lce
