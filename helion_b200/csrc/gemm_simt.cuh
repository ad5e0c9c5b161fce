// CUDA-core GEMM core with the same epilogue contract as the tcgen05 core.
//
//   D[m, n] = sum_k A[m, k] * B[n, k]     fp32 FMA, k ascending, no tensor cores
//
// It serves the inputs the tensor-core path cannot take: fp32 tensors (the reference demands
// 1e-5 agreement with fp32 torch there, so TF32 is not an option), hidden sizes that are not a
// multiple of 8 (TMA needs 16-byte row pitches) and problems too small to fill a 128 x 256 tile.
// Operands are addressed through explicit (row, k) strides, so any majorness works.
//
// One CTA of 128 threads computes a 128 x 32 tile; thread t owns row t and all 32 columns, which
// is exactly the "one thread = one row, 32 columns at a time" shape the epilogues expect.
#pragma once

#include "epilogues.cuh"

namespace lce {

constexpr int kSimtBN = 32;
constexpr int kSimtBK = 16;
constexpr int kSimtThreads = 128;

template <class T>
struct SimtOperand {
    const T* ptr;
    long long stride_mn;  // elements between consecutive m (resp. n)
    long long stride_k;   // elements between consecutive k
    int extent_mn;        // valid m (resp. n)
};

template <class T, class Epi>
__global__ void __launch_bounds__(kSimtThreads)
gemm_simt_kernel(SimtOperand<T> A, SimtOperand<T> B, int K, int m_tiles, int n_tiles, int k_splits,
                 const typename Epi::Params ep) {
    __shared__ float As[kSimtBK][kBM + 1];
    __shared__ __align__(16) float Bs[kSimtBK][kSimtBN];

    const int t = threadIdx.x;
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

        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0.f;

        for (int k0 = k_begin; k0 < k_end; k0 += kSimtBK) {
            // A tile: 128 x 16. Walk the contiguous direction with consecutive threads.
#pragma unroll
            for (int i = 0; i < (kBM * kSimtBK) / kSimtThreads; ++i) {
                const int idx = t + i * kSimtThreads;
                int m, k;
                if (A.stride_k == 1) { k = idx % kSimtBK; m = idx / kSimtBK; }
                else { m = idx % kBM; k = idx / kBM; }
                float val = 0.f;
                if (m0 + m < A.extent_mn && k0 + k < k_end)
                    val = Cvt<T>::to_f(A.ptr[(long long)(m0 + m) * A.stride_mn + (long long)(k0 + k) * A.stride_k]);
                As[k][m] = val;
            }
#pragma unroll
            for (int i = 0; i < (kSimtBN * kSimtBK) / kSimtThreads; ++i) {
                const int idx = t + i * kSimtThreads;
                int n, k;
                if (B.stride_k == 1) { k = idx % kSimtBK; n = idx / kSimtBK; }
                else { n = idx % kSimtBN; k = idx / kSimtBN; }
                float val = 0.f;
                if (n0 + n < B.extent_mn && k0 + k < k_end)
                    val = Cvt<T>::to_f(B.ptr[(long long)(n0 + n) * B.stride_mn + (long long)(k0 + k) * B.stride_k]);
                Bs[k][n] = val;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < kSimtBK; ++k) {
                const float a = As[k][t];
#pragma unroll
                for (int j4 = 0; j4 < kSimtBN / 4; ++j4) {
                    const float4 b = *reinterpret_cast<const float4*>(&Bs[k][j4 * 4]);
                    acc[4 * j4 + 0] = fmaf(a, b.x, acc[4 * j4 + 0]);
                    acc[4 * j4 + 1] = fmaf(a, b.y, acc[4 * j4 + 1]);
                    acc[4 * j4 + 2] = fmaf(a, b.z, acc[4 * j4 + 2]);
                    acc[4 * j4 + 3] = fmaf(a, b.w, acc[4 * j4 + 3]);
                }
            }
            __syncthreads();
        }

        TileCtx tc{m_tile, n_tile, n_tiles, t, kSimtBN, k_slice, nullptr};
        typename Epi::State st;
        Epi::begin(st, ep, tc);
        Epi::chunk(st, ep, tc, 0, acc);
        Epi::end(st, ep, tc);
    }
}

}  // namespace lce
