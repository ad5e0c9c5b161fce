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
constexpr int kSimtBK = 16;
constexpr int kSimtThreads = 256;
constexpr int kSimtPitch = 128 + 4;   // operand tiles [k][mn] in floats: rows stay 16-byte aligned, the pad
                                      // spreads a k-contiguous deposit over the banks
constexpr int kSimtCPitch = 64 + 4;   // one 64-column half of the C tile
constexpr int kSimtLoads = 128 * kSimtBK / kSimtThreads;  // 8 elements of each operand per thread and k step
constexpr int kSimtVecs = kSimtLoads / 4;                  // = two 16-byte vectors for the vector loaders
static_assert(kBM == 128, "the thread layout below is written for 128 x 128 tiles");

template <class T>
struct SimtOperand {
    const T* ptr;
    long long stride_mn;  // elements between consecutive m (resp. n)
    long long stride_k;   // elements between consecutive k
    int extent_mn;        // valid m (resp. n)
};

// How a thread fetches its share (4 elements) of a 128 x 8 operand tile:
//   kSimtGeneric  four scalar loads with run-time strides and per-element bounds tests: any dtype,
//                 any alignment, any majorness (consecutive threads walk the contiguous direction);
//   kSimtVecK     fp32, k contiguous: one 16-byte load of 4 consecutive k of one row (thread t: row t/2,
//                 k 4*(t%2)), deposited as four conflict-free scalar stores (the tile is [k][mn]);
//   kSimtVecMN    fp32, m/n contiguous: one 16-byte load of 4 consecutive m/n at one k (thread t: k t/32,
//                 m/n 4*(t%32)), deposited as one 16-byte store.
// The vector modes need a 16-byte aligned base, strides and the vectorised extent in multiples of 4;
// the host picks them (launch_simt). Row validity is settled once per tile, and the pointer just advances.
enum SimtMode { kSimtGeneric = 0, kSimtVecK = 1, kSimtVecMN = 2 };

template <class T, int MODE>
struct SimtLoader;

template <class T>
struct SimtLoader<T, kSimtGeneric> {
    static constexpr bool kAsync = false;
    const T* p;
    long long step, k_adv;
    int mn_t, k_t, mn_step, k_step, mn_left;
    __device__ __forceinline__ void init(const SimtOperand<T>& op, int mn0, int k_begin, int t) {
        if (op.stride_k == 1) { k_t = t % kSimtBK; mn_t = t / kSimtBK; mn_step = kSimtThreads / kSimtBK; k_step = 0; }
        else { mn_t = t % 128; k_t = t / 128; mn_step = 0; k_step = kSimtThreads / 128; }
        p = op.ptr + static_cast<long long>(mn0 + mn_t) * op.stride_mn + static_cast<long long>(k_begin + k_t) * op.stride_k;
        step = mn_step * op.stride_mn + k_step * op.stride_k;
        k_adv = kSimtBK * op.stride_k;
        mn_left = op.extent_mn - mn0 - mn_t;  // element i is in range iff i * mn_step < mn_left
    }
    __device__ __forceinline__ void fetch(int k0, int k_end, float (&r)[kSimtLoads], float*) {
#pragma unroll
        for (int i = 0; i < kSimtLoads; ++i) {
            r[i] = 0.f;
            if (i * mn_step < mn_left && k0 + k_t + i * k_step < k_end) r[i] = Cvt<T>::to_f(p[i * step]);
        }
        p += k_adv;
    }
    __device__ __forceinline__ void deposit(float* tile, const float (&r)[kSimtLoads]) const {
#pragma unroll
        for (int i = 0; i < kSimtLoads; ++i) tile[(k_t + i * k_step) * kSimtPitch + mn_t + i * mn_step] = r[i];
    }
};

template <>
struct SimtLoader<float, kSimtVecK> {
    // thread t, vector i: row (t / (BK/4)) + i * (256 / (BK/4)), k offset 4 * (t % (BK/4))
    static constexpr bool kAsync = false;
    static constexpr int kPerRow = kSimtBK / 4;
    static constexpr int kRowStep = kSimtThreads / kPerRow;
    const float* p;
    long long row_adv;
    int row, k4;
    bool valid[kSimtVecs];
    __device__ __forceinline__ void init(const SimtOperand<float>& op, int mn0, int k_begin, int t) {
        row = t / kPerRow;
        k4 = (t % kPerRow) * 4;
#pragma unroll
        for (int i = 0; i < kSimtVecs; ++i) valid[i] = mn0 + row + i * kRowStep < op.extent_mn;
        p = op.ptr + static_cast<long long>(mn0 + row) * op.stride_mn + k_begin + k4;
        row_adv = static_cast<long long>(kRowStep) * op.stride_mn;
    }
    __device__ __forceinline__ void fetch(int k0, int k_end, float (&r)[kSimtLoads], float*) {
#pragma unroll
        for (int i = 0; i < kSimtVecs; ++i) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid[i] && k0 + k4 < k_end) v = *reinterpret_cast<const float4*>(p + i * row_adv);  // K % 4 == 0: all four or none
            r[4 * i + 0] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        p += kSimtBK;
    }
    __device__ __forceinline__ void deposit(float* tile, const float (&r)[kSimtLoads]) const {
#pragma unroll
        for (int i = 0; i < kSimtVecs; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) tile[(k4 + j) * kSimtPitch + row + i * kRowStep] = r[4 * i + j];
    }
};

template <>
struct SimtLoader<float, kSimtVecMN> {
    // thread t, vector i: k (t / 32) + i * 8, m/n offset 4 * (t % 32). The tile in shared memory is [k][mn], so a
    // 16-byte vector of consecutive m/n lands as it is: the copy goes global -> shared with cp.async and needs
    // no registers between fetch and deposit (out-of-range vectors are zero-filled by a source size of 0).
    static constexpr bool kAsync = true;
    const float* p;
    long long k_adv, k_half;
    int k, mn4;
    bool valid;
    __device__ __forceinline__ void init(const SimtOperand<float>& op, int mn0, int k_begin, int t) {
        k = t >> 5;
        mn4 = (t & 31) * 4;
        valid = mn0 + mn4 < op.extent_mn;  // extent % 4 == 0: all four or none
        p = op.ptr + (mn0 + mn4) + static_cast<long long>(k_begin + k) * op.stride_k;
        k_adv = kSimtBK * op.stride_k;
        k_half = (kSimtThreads / 32) * op.stride_k;
        if (!valid) p = op.ptr;  // never dereferenced (source size 0), but keep the address inside the tensor
    }
    __device__ __forceinline__ void fetch(int k0, int k_end, float (&)[kSimtLoads], float* tile) {
#pragma unroll
        for (int i = 0; i < kSimtVecs; ++i) {
            const bool in = valid && k0 + k + i * (kSimtThreads / 32) < k_end;
            const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(tile + (k + i * (kSimtThreads / 32)) * kSimtPitch + mn4));
            const float* src = in ? p + i * k_half : p;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
        }
        if (valid) p += k_adv;
    }
    __device__ __forceinline__ void deposit(float*, const float (&)[kSimtLoads]) const {}
};

template <class T, class Epi, int AMODE = kSimtGeneric, int BMODE = kSimtGeneric>
__global__ void __launch_bounds__(kSimtThreads, 2)
gemm_simt_kernel(SimtOperand<T> A, SimtOperand<T> B, int K, int m_tiles, int n_tiles, int k_splits,
                 const typename Epi::Params ep) {
    // main loop: two buffers of As[k][m] + Bs[k][n]; afterwards the same memory stages half a C tile
    constexpr int kTileFloats = kSimtBK * kSimtPitch;
    __shared__ __align__(16) float smem[128 * kSimtCPitch];
    static_assert(4 * kTileFloats <= 128 * kSimtCPitch, "two buffers of both operand tiles fit in the C staging area");

    const int t = threadIdx.x;
    const int ty = t >> 4, tx = t & 15;
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

        SimtLoader<T, AMODE> la;
        SimtLoader<T, BMODE> lb;
        la.init(A, m0, k_begin, t);
        lb.init(B, n0, k_begin, t);
        constexpr bool kAnyAsync = SimtLoader<T, AMODE>::kAsync || SimtLoader<T, BMODE>::kAsync;
        float ra[kSimtLoads], rb[kSimtLoads];
        la.fetch(k_begin, k_end, ra, smem);
        lb.fetch(k_begin, k_end, rb, smem + kTileFloats);
        la.deposit(smem, ra);
        lb.deposit(smem + kTileFloats, rb);
        if constexpr (kAnyAsync) asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        int cur = 0;
        for (int k0 = k_begin; k0 < k_end; k0 += kSimtBK) {
            const bool more = k0 + kSimtBK < k_end;
            float* nxt = smem + (cur ^ 1) * 2 * kTileFloats;
            if (more) {  // in flight while this step multiplies (straight into the other buffer where the copy is async)
                la.fetch(k0 + kSimtBK, k_end, ra, nxt);
                lb.fetch(k0 + kSimtBK, k_end, rb, nxt + kTileFloats);
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
                la.deposit(nxt, ra);
                lb.deposit(nxt + kTileFloats, rb);
                if constexpr (kAnyAsync) asm volatile("cp.async.wait_all;" ::: "memory");
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
