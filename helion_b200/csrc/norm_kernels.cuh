// RMSNorm and residual-add RMSNorm (the reference's tritium.rmsnorm / residual_rmsnorm /
// rmsnorm_backward, tritium/ops/rmsnorm.py:29-280): the producer of the hidden states that the
// fused linear-cross-entropy head consumes. Pure HBM streaming.
//
//   forward    z = x (+ residual);  rstd = 1 / sqrt(mean(z^2) + eps);  out = z * rstd * weight
//   backward   wd = dy * weight;  c = sum(wd * x)
//              dx = rstd * wd - (rstd^3 / H) * x * c   (+ dresidual)
//              dweight = sum over rows of dy * x * rstd
//
// Every input element is read from HBM exactly once and every output written once. Unlike the
// reference, whose backward reads dy and x a second time to form dweight (tritium/ops/rmsnorm.py:383-439),
// the backward here is a single pass: each thread owns the same columns for every row its CTA walks,
// accumulates their dweight contributions in registers and writes one partial row per CTA at the end;
// rms_dw_reduce_kernel adds the partial rows in a fixed order (no atomics: the same bits on every run).
//
// Three forms, chosen by the host (lce_rmsnorm_forward / lce_rmsnorm_backward):
//   ring      16-byte-aligned rows: rows stream into a shared-memory ring with cp.async.bulk (below);
//   register  unaligned rows or odd widths (and small forwards): the CTA keeps ROWS rows packed in
//             registers, element-wise loads where 16-byte ones are not legal;
//   wide      rows beyond 256 threads x 8 vectors: two passes, the second one re-reads the row from L2.
#pragma once

#include "row_kernels.cuh"

namespace lce {

constexpr int kRmsMaxThreads = 256;
constexpr int kRmsMaxPartials = 592;  // backward CTAs = partial dweight rows (4 per SM on 148 SMs)

template <class T>
struct RmsTile {
    static constexpr int kVec = 16 / sizeof(T);
    static constexpr int kMaxVpt = 8;  // 256 threads x 8 vectors: 16384 16-bit or 8192 fp32 columns
};

// Columns c .. c + VEC of one row as a raw 16-byte vector; columns at or beyond H read as zero.
template <class T, bool VECTOR>
__device__ __forceinline__ uint4 rms_load(const T* __restrict__ row, int c, int H) {
    constexpr int VEC = RmsTile<T>::kVec;
    if (VECTOR) {
        return c < H ? *reinterpret_cast<const uint4*>(row + c) : make_uint4(0u, 0u, 0u, 0u);
    } else {
        alignas(16) T tmp[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) tmp[j] = (c + j < H) ? row[c + j] : Cvt<T>::from_f(0.f);
        return *reinterpret_cast<const uint4*>(tmp);
    }
}

// 16-byte vector <-> floats. The 16-bit forms convert two elements per instruction where the hardware
// can (bf16 -> fp32 is a shift or a mask of the packed word; fp32 -> 16-bit pairs is one cvt).
template <class T>
__device__ __forceinline__ void rms_unpack(const uint4& raw, float (&v)[RmsTile<T>::kVec]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    if constexpr (std::is_same<T, float>::value) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(w[j]);
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    }
}

template <class T>
__device__ __forceinline__ uint4 rms_pack(const float (&v)[RmsTile<T>::kVec]) {
    uint32_t w[4];
    if constexpr (std::is_same<T, float>::value) {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(v[j]);
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// 1 / sqrt(ss / H + eps) from a precomputed 1 / H: the hardware reciprocal square root plus one Newton
// step (relative error ~1e-7) - an exactly rounded divide and square root would cost every thread more
// instructions than the rest of its row.
__device__ __forceinline__ float rms_rstd(float ss, float inv_h, float eps) {
    const float a = fmaf(ss, inv_h, eps);
    const float y = rsqrtf(a);
    return y * fmaf(-0.5f * a * y, y, 1.5f);
}

template <class T, bool VECTOR>
__device__ __forceinline__ void rms_store(T* __restrict__ row, int c, int H, const uint4& raw) {
    constexpr int VEC = RmsTile<T>::kVec;
    if (VECTOR) {
        if (c < H) *reinterpret_cast<uint4*>(row + c) = raw;
    } else {
        alignas(16) T tmp[VEC];
        *reinterpret_cast<uint4*>(tmp) = raw;
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (c + j < H) row[c + j] = tmp[j];
    }
}

template <int N> struct RmsLog2 { static constexpr int value = 1 + RmsLog2<N / 2>::value; };
template <> struct RmsLog2<1> { static constexpr int value = 0; };

// Sums NV values (NV a power of two <= 32) over a CTA of at most 32 warps; every thread gets the totals.
//  1. inside a warp, a transposed butterfly: at each of the first log2(NV) steps a lane keeps half of its
//     values and trades the other half with its partner, so NV values cost NV - 1 + (5 - log2 NV) shuffles
//     instead of 5 NV; lane l ends up with the warp total of value l >> (5 - log2 NV);
//  2. the warp totals go through shared memory: lane l picks up the partials p = l, l + 32, ...
//     (p = warp * NV + value), a strided butterfly leaves the total of value l % NV in lane l, and NV
//     broadcasts hand every lane all of them.
// The order of the additions is fixed, so the result does not depend on timing. `red` holds 32 x NV floats
// and must not be reused before the next __syncthreads() (callers alternate two buffers).
template <int NV>
__device__ __forceinline__ void rms_block_sum(float (&v)[NV], float* red) {
    static_assert(NV >= 1 && NV <= 32 && (NV & (NV - 1)) == 0, "power of two");
    constexpr int L = RmsLog2<NV>::value;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int s = 0; s < L; ++s) {
        const int o = 16 >> s, half = NV >> (s + 1);
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    float r = v[0];
#pragma unroll
    for (int s = L; s < 5; ++s) r += __shfl_xor_sync(0xffffffffu, r, 16 >> s);
    if ((lane & ((32 >> L) - 1)) == 0) red[warp * NV + (lane >> (5 - L))] = r;
    __syncthreads();
    float part = 0.f;
    for (int p = lane; p < n_warps * NV; p += 32) part += red[p];
#pragma unroll
    for (int o = NV; o < 32; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = __shfl_sync(0xffffffffu, part, i);
}

// ---------------------------------------------------------------------------------------------
// forward (register-resident rows)
// A CTA walks groups of ROWS consecutive rows: the loads of all ROWS rows are issued before anything
// is reduced (ROWS x VPT 16-byte vectors in flight per thread and input - what keeps HBM busy when a
// row is only a few KB), and the ROWS row sums share one barrier. The rows stay PACKED in registers
// across the barrier and are unpacked again for the output pass.
// ---------------------------------------------------------------------------------------------
template <int VPT>
struct RmsRows {
    static constexpr int kRows = VPT >= 4 ? 1 : 4 / VPT;  // ROWS x VPT >= 4 vectors per thread and input
};

template <class T, int VPT, bool VECTOR, bool RESIDUAL>
__global__ void __launch_bounds__(kRmsMaxThreads)
rms_forward_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                   T* __restrict__ out, T* __restrict__ residual_out, float* __restrict__ rstd_out,
                   int n_rows, int H, float eps) {
    const float inv_h = 1.0f / static_cast<float>(H);
    constexpr int VEC = RmsTile<T>::kVec;
    constexpr int ROWS = RmsRows<VPT>::kRows;
    __shared__ float red[2][ROWS * 32];
    const int t = threadIdx.x;

    uint4 wraw[VPT];  // this thread's weight columns, loaded once
#pragma unroll
    for (int i = 0; i < VPT; ++i) wraw[i] = rms_load<T, VECTOR>(weight, (i * blockDim.x + t) * VEC, H);

    int it = 0;
    for (int row0 = blockIdx.x * ROWS; row0 < n_rows; row0 += gridDim.x * ROWS, ++it) {
        uint4 rx[ROWS][VPT], rr[RESIDUAL ? ROWS : 1][VPT];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const long long off = static_cast<long long>(row0 + r) * H;
            const int h = row0 + r < n_rows ? H : 0;  // rows past the end read as zeros
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int c = (i * blockDim.x + t) * VEC;
                rx[r][i] = rms_load<T, VECTOR>(x + off, c, h);
                if (RESIDUAL) rr[r][i] = rms_load<T, VECTOR>(residual + off, c, h);
            }
        }
        float ss[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const long long off = static_cast<long long>(row0 + r) * H;
            const int h = row0 + r < n_rows ? H : 0;
            ss[r] = 0.f;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                float z[VEC];
                rms_unpack<T>(rx[r][i], z);
                if (RESIDUAL) {
                    float q[VEC];
                    rms_unpack<T>(rr[r][i], q);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) z[j] += q[j];
                    rms_store<T, VECTOR>(residual_out + off, (i * blockDim.x + t) * VEC, h, rms_pack<T>(z));
                }
#pragma unroll
                for (int j = 0; j < VEC; ++j) ss[r] = fmaf(z[j], z[j], ss[r]);
            }
        }
        rms_block_sum<ROWS>(ss, red[it & 1]);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const long long off = static_cast<long long>(row0 + r) * H;
            const int h = row0 + r < n_rows ? H : 0;
            const float rstd = rms_rstd(ss[r], inv_h, eps);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                float z[VEC], w[VEC];
                rms_unpack<T>(rx[r][i], z);
                if (RESIDUAL) {
                    float q[VEC];
                    rms_unpack<T>(rr[r][i], q);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) z[j] += q[j];
                }
                rms_unpack<T>(wraw[i], w);
#pragma unroll
                for (int j = 0; j < VEC; ++j) z[j] = z[j] * rstd * w[j];
                rms_store<T, VECTOR>(out + off, (i * blockDim.x + t) * VEC, h, rms_pack<T>(z));
            }
            if (t == 0 && rstd_out != nullptr && h != 0) rstd_out[row0 + r] = rstd;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Plain forward, one row per CTA: what measured fastest for the plain (non-residual) forward of rows of
// 8 KB and more. HBM bandwidth needs bytes in flight, and here they come from MANY small CTAs per SM rather
// than from a few large ones: a CTA of 128 (or 256) threads holds its row in VPT 16-byte vectors per thread,
// keeps nothing else across the row sum - the weights are fetched after it, out of L1/L2 - and so stays at
// 40-85 registers (1536 / 1152 / 768 resident threads per SM for 2 / 4 / 8 vectors per thread: 50-100 KB of
// loads in flight per SM); the grid is one CTA per row and the hardware deals them out as CTAs retire.
// ---------------------------------------------------------------------------------------------
template <class T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS, (VPT <= 2 ? 1536 : (VPT == 4 ? 1152 : 768)) / THREADS)
rms_forward_row_kernel(const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ out,
                       float* __restrict__ rstd_out, int n_rows, int H, float eps) {
    constexpr int VEC = RmsTile<T>::kVec;
    __shared__ float red[THREADS / 32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const float inv_h = 1.0f / static_cast<float>(H);
    for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
        const T* xr = x + static_cast<long long>(row) * H;
        T* orow = out + static_cast<long long>(row) * H;
        uint4 rx[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) rx[i] = rms_load<T, true>(xr, (i * THREADS + t) * VEC, H);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float z[VEC];
            rms_unpack<T>(rx[i], z);
#pragma unroll
            for (int j = 0; j < VEC; ++j) ss = fmaf(z[j], z[j], ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        __syncthreads();  // `red` of the previous row has been read by everyone
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int k = 0; k < THREADS / 32; ++k) total += red[k];  // same order in every thread
        const float rstd = rms_rstd(total, inv_h, eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = (i * THREADS + t) * VEC;
            float z[VEC], w[VEC];
            rms_unpack<T>(rx[i], z);
            rms_unpack<T>(rms_load<T, true>(weight, c, H), w);
#pragma unroll
            for (int j = 0; j < VEC; ++j) z[j] = z[j] * rstd * w[j];
            rms_store<T, true>(orow, c, H, rms_pack<T>(z));
        }
        if (t == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    }
}

// ---------------------------------------------------------------------------------------------
// Ring kernels: the form every 16-byte-aligned problem takes.
//
// A row is only a few KB, so what keeps HBM busy is how many bytes a CTA has in flight - and registers
// are a poor landing zone for them. Here one elected thread streams groups of ROWS consecutive rows
// (contiguous in memory: one bulk copy per input tensor) into a ring of shared-memory stages with
// cp.async.bulk, completion counted on an mbarrier per stage; the CTA's threads compute out of shared
// memory (each thread owns the same columns of every row, two passes over the stage: row sums, then
// outputs) and write results straight to global memory. The stage is refilled as soon as the CTA is
// done with it, so up to STAGES - 1 stages per CTA are always in flight regardless of register use.
// Waits on the mbarriers are bounded; on a timeout the CTA records kDevErrNormTimeout in the device
// status word, drains what it issued (bounded again) and returns.
// ---------------------------------------------------------------------------------------------
// Rows per stage: enough that the per-stage costs (barriers, the cross-warp sum) are spread over
// 8 vectors per thread when one tensor streams in, 4 when two or three do (the stage must stay small
// enough for a multi-stage ring).
template <int VPT, int NS>
struct RmsRingRows {
    static constexpr int kTarget = NS == 1 ? 8 : 4;
    static constexpr int kRows = VPT >= kTarget ? 1 : kTarget / VPT;
};

constexpr int kRmsMaxStages = 4;
constexpr int kRmsRingBytesPerSm = 200 * 1024;
constexpr int kDevErrNormTimeout = 111;

// Streaming hints of the ring forward (experiment knob, set from HELION_B200_RMS_HINT at first use):
// bit 0 = the bulk loads carry an L2 evict_first policy, bit 1 = the outputs are stored with st.global.cs.
__device__ int g_rms_hint = 0;

struct RmsRing {
    uint64_t full[kRmsMaxStages];
    int abort_flag;
    int drain_flag;
};

// Thread 0: start the loads of this CTA's k-th row group into stage k % stages (nothing if the group
// does not exist). `src` holds NS input tensors; stage layout = [tensor][row in group][H].
template <class T, int ROWS, int NS>
__device__ __forceinline__ void rms_ring_issue(RmsRing& ring, unsigned char* data, const T* const* src, int k,
                                               int stages, int n_rows, int H) {
    const long long group = blockIdx.x + static_cast<long long>(k) * gridDim.x;
    const long long row0 = group * ROWS;
    if (row0 >= n_rows) return;
    const int s = k % stages;
    const int nr = n_rows - row0 < ROWS ? static_cast<int>(n_rows - row0) : ROWS;
    const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
    const uint32_t bar = ptx::smem_u32(&ring.full[s]);
    // g_debug_announce_extra is 0 except in the wait-expiry test (a read of a cached word per row group)
    ptx::mbar_arrive_expect_tx(bar, nr * row_bytes * NS + ptx::g_debug_announce_extra);
    unsigned char* dst = data + static_cast<size_t>(s) * (ROWS * NS * row_bytes);
    if (g_rms_hint & 1) {
        const uint64_t policy = ptx::make_l2_policy(ptx::kL2EvictFirst);
#pragma unroll
        for (int n = 0; n < NS; ++n)
            ptx::bulk_load_1d_hint(ptx::smem_u32(dst + n * ROWS * row_bytes), src[n] + row0 * H, nr * row_bytes, bar, policy);
        return;
    }
#pragma unroll
    for (int n = 0; n < NS; ++n)
        ptx::bulk_load_1d(ptx::smem_u32(dst + n * ROWS * row_bytes), src[n] + row0 * H, nr * row_bytes, bar);
}

// After a timeout: thread 0 waits (bounded) for the loads that were issued but never consumed, so that
// no copy is still writing into this CTA's shared memory when it exits.
__device__ __forceinline__ void rms_ring_drain(RmsRing& ring, int k_next, int stages, long long n_groups, int* status) {
    if (status != nullptr) atomicCAS(status, 0, kDevErrNormTimeout);
    ring.drain_flag = 0;
    for (int k = k_next; k < k_next + stages; ++k) {
        if (blockIdx.x + static_cast<long long>(k) * gridDim.x >= n_groups) break;
        ptx::mbar_wait(ptx::smem_u32(&ring.full[k % stages]), (k / stages) & 1, &ring.drain_flag);
    }
}

// Forward on the ring (plain rmsnorm; the residual form is faster on the register kernels).
template <class T, int VPT>
__global__ void __launch_bounds__(kRmsMaxThreads, 2)
rms_ring_forward_kernel(const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ out,
                        float* __restrict__ rstd_out,
                        int n_rows, int H, float eps, int stages, int* __restrict__ status) {
    const float inv_h = 1.0f / static_cast<float>(H);
    constexpr int VEC = RmsTile<T>::kVec;
    constexpr int NS = 1;
    constexpr int ROWS = RmsRingRows<VPT, NS>::kRows;
    constexpr bool kWeightUnpacked = VPT * VEC <= 16;  // else kept packed and unpacked per use
    extern __shared__ __align__(128) unsigned char ring_data[];
    __shared__ RmsRing ring;
    __shared__ float red[2][ROWS * 32];
    const int t = threadIdx.x;
    const long long n_groups = (static_cast<long long>(n_rows) + ROWS - 1) / ROWS;
    const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
    const T* const srcs[1] = {x};
    const bool stream_stores = (g_rms_hint & 2) != 0;

    if (t == 0) {
        for (int s = 0; s < stages; ++s) ptx::mbar_init(ptx::smem_u32(&ring.full[s]), 1);
        ring.abort_flag = 0;
        ptx::fence_mbar_init();
        for (int k = 0; k < stages; ++k) rms_ring_issue<T, ROWS, NS>(ring, ring_data, srcs, k, stages, n_rows, H);
    }
    uint4 wraw[kWeightUnpacked ? 1 : VPT];  // this thread's weight columns
    float wf[kWeightUnpacked ? VPT : 1][VEC];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const uint4 raw = rms_load<T, true>(weight, (i * blockDim.x + t) * VEC, H);
        if (kWeightUnpacked) rms_unpack<T>(raw, wf[i]);
        else wraw[i] = raw;
    }
    __syncthreads();

    int k = 0;
    bool failed = false;
    for (;; ++k) {
        const long long group = blockIdx.x + static_cast<long long>(k) * gridDim.x;
        if (group >= n_groups) break;
        const long long row0 = group * ROWS;
        const int s = k % stages;
        ptx::mbar_wait(ptx::smem_u32(&ring.full[s]), (k / stages) & 1, &ring.abort_flag);
        const unsigned char* st = ring_data + static_cast<size_t>(s) * (ROWS * NS * row_bytes);
        float ss[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            ss[r] = 0.f;
            if (row0 + r < n_rows) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int c = (i * blockDim.x + t) * VEC;
                    if (c < H) {
                        float z[VEC];
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + r * row_bytes + c * sizeof(T)), z);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) ss[r] = fmaf(z[j], z[j], ss[r]);
                    }
                }
            }
        }
        rms_block_sum<ROWS>(ss, red[k & 1]);
        if (ring.abort_flag) {  // written before the barrier inside rms_block_sum: every thread sees it
            failed = true;
            break;
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (row0 + r < n_rows) {
                const float rstd = rms_rstd(ss[r], inv_h, eps);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int c = (i * blockDim.x + t) * VEC;
                    if (c < H) {
                        float z[VEC], w[VEC];
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + r * row_bytes + c * sizeof(T)), z);
                        if (!kWeightUnpacked) rms_unpack<T>(wraw[i], w);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) z[j] = z[j] * rstd * (kWeightUnpacked ? wf[i][j] : w[j]);
                        if (stream_stores) __stcs(reinterpret_cast<uint4*>(out + (row0 + r) * H + c), rms_pack<T>(z));
                        else *reinterpret_cast<uint4*>(out + (row0 + r) * H + c) = rms_pack<T>(z);
                    }
                }
                if (t == 0 && rstd_out != nullptr) rstd_out[row0 + r] = rstd;
            }
        }
        __syncthreads();  // the CTA is done with stage s
        if (t == 0) {
            ptx::fence_proxy_async_smem();
            rms_ring_issue<T, ROWS, NS>(ring, ring_data, srcs, k + stages, stages, n_rows, H);
        }
    }
    if (failed && t == 0) rms_ring_drain(ring, k, stages, n_groups, status);
}

// Backward on the ring. NS = 2 (dy, x) or 3 (+ dresidual). The dweight contributions of the columns a
// thread owns stay in its registers over all the rows its CTA walks; partial[blockIdx.x][H] at the end.
template <class T, int VPT, bool DRES>
__global__ void __launch_bounds__(kRmsMaxThreads, 2)
rms_ring_backward_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ weight,
                         const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
                         float* __restrict__ partial, int n_rows, int H, float eps, int stages,
                         int* __restrict__ status) {
    const float inv_h = 1.0f / static_cast<float>(H);
    constexpr int VEC = RmsTile<T>::kVec;
    constexpr int NS = DRES ? 3 : 2;
    constexpr int ROWS = RmsRingRows<VPT, NS>::kRows;
    constexpr bool kWeightInRegs = VPT * VEC <= 16;
    extern __shared__ __align__(128) unsigned char ring_data[];
    __shared__ RmsRing ring;
    __shared__ float red[2][2 * ROWS * 32];
    const int t = threadIdx.x;
    const long long n_groups = (static_cast<long long>(n_rows) + ROWS - 1) / ROWS;
    const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
    const T* const srcs[3] = {dy, x, dres};

    if (t == 0) {
        for (int s = 0; s < stages; ++s) ptx::mbar_init(ptx::smem_u32(&ring.full[s]), 1);
        ring.abort_flag = 0;
        ptx::fence_mbar_init();
        for (int k = 0; k < stages; ++k) rms_ring_issue<T, ROWS, NS>(ring, ring_data, srcs, k, stages, n_rows, H);
    }
    uint4 wraw[kWeightInRegs ? VPT : 1];
    if (kWeightInRegs) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) wraw[i] = rms_load<T, true>(weight, (i * blockDim.x + t) * VEC, H);
    }
    float dwacc[VPT][VEC];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) dwacc[i][j] = 0.f;
    __syncthreads();

    int k = 0;
    bool failed = false;
    for (;; ++k) {
        const long long group = blockIdx.x + static_cast<long long>(k) * gridDim.x;
        if (group >= n_groups) break;
        const long long row0 = group * ROWS;
        const int s = k % stages;
        ptx::mbar_wait(ptx::smem_u32(&ring.full[s]), (k / stages) & 1, &ring.abort_flag);
        const unsigned char* st = ring_data + static_cast<size_t>(s) * (ROWS * NS * row_bytes);
        // pass A: per row c = sum(dy * w * x) and sum(x^2)
        float sums[2 * ROWS];
#pragma unroll
        for (int r = 0; r < 2 * ROWS; ++r) sums[r] = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = (i * blockDim.x + t) * VEC;
            if (c < H) {
                float w[VEC];
                if (kWeightInRegs) rms_unpack<T>(wraw[i], w);
                else rms_unpack<T>(*reinterpret_cast<const uint4*>(weight + c), w);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    if (row0 + r < n_rows) {
                        float d[VEC], xv[VEC];
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + r * row_bytes + c * sizeof(T)), d);
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + (ROWS + r) * row_bytes + c * sizeof(T)), xv);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) {
                            sums[2 * r] = fmaf(d[j] * w[j], xv[j], sums[2 * r]);
                            sums[2 * r + 1] = fmaf(xv[j], xv[j], sums[2 * r + 1]);
                        }
                    }
                }
            }
        }
        rms_block_sum<2 * ROWS>(sums, red[k & 1]);
        if (ring.abort_flag) {
            failed = true;
            break;
        }
        // pass B: dx and the dweight contributions
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (row0 + r < n_rows) {
                const float rstd = rstd_in != nullptr ? rstd_in[row0 + r]
                                                      : rms_rstd(sums[2 * r + 1], inv_h, eps);
                // dx = rstd * w * dy - (rstd^3 / H * c) * x, two scalars per row hoisted out of the columns
                const float coefc = rstd * rstd * rstd * inv_h * sums[2 * r];
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int c = (i * blockDim.x + t) * VEC;
                    if (c < H) {
                        float w[VEC], d[VEC], xv[VEC], o[VEC];
                        if (kWeightInRegs) rms_unpack<T>(wraw[i], w);
                        else rms_unpack<T>(*reinterpret_cast<const uint4*>(weight + c), w);
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + r * row_bytes + c * sizeof(T)), d);
                        rms_unpack<T>(*reinterpret_cast<const uint4*>(st + (ROWS + r) * row_bytes + c * sizeof(T)), xv);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) {
                            dwacc[i][j] = fmaf(d[j] * xv[j], rstd, dwacc[i][j]);
                            o[j] = fmaf(rstd * w[j], d[j], -coefc * xv[j]);
                        }
                        if (DRES) {
                            float q[VEC];
                            rms_unpack<T>(*reinterpret_cast<const uint4*>(st + (2 * ROWS + r) * row_bytes + c * sizeof(T)), q);
#pragma unroll
                            for (int j = 0; j < VEC; ++j) o[j] = Cvt<T>::to_f(Cvt<T>::from_f(o[j])) + q[j];
                        }
                        *reinterpret_cast<uint4*>(dx + (row0 + r) * H + c) = rms_pack<T>(o);
                    }
                }
            }
        }
        __syncthreads();  // the CTA is done with stage s
        if (t == 0) {
            ptx::fence_proxy_async_smem();
            rms_ring_issue<T, ROWS, NS>(ring, ring_data, srcs, k + stages, stages, n_rows, H);
        }
    }
    if (failed && t == 0) rms_ring_drain(ring, k, stages, n_groups, status);
    if (partial != nullptr) {
        float* prow = partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = (i * blockDim.x + t) * VEC;
            if (c < H) {
                float4* dst = reinterpret_cast<float4*>(prow + c);
#pragma unroll
                for (int j = 0; j < VEC; j += 4)
                    dst[j / 4] = make_float4(dwacc[i][j], dwacc[i][j + 1], dwacc[i][j + 2], dwacc[i][j + 3]);
            }
        }
    }
}

// forward, any width: two passes over the row (the second one hits L2)
template <class T, bool RESIDUAL>
__global__ void __launch_bounds__(kRmsMaxThreads)
rms_forward_wide_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                        T* __restrict__ out, T* __restrict__ residual_out, float* __restrict__ rstd_out,
                        int n_rows, int H, float eps) {
    const float inv_h = 1.0f / static_cast<float>(H);
    __shared__ float red[2][32];
    int it = 0;
    for (int row = blockIdx.x; row < n_rows; row += gridDim.x, ++it) {
        const long long off = static_cast<long long>(row) * H;
        float ss[1] = {0.f};
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float z = Cvt<T>::to_f(x[off + c]);
            if (RESIDUAL) {
                z += Cvt<T>::to_f(residual[off + c]);
                residual_out[off + c] = Cvt<T>::from_f(z);
            }
            ss[0] = fmaf(z, z, ss[0]);
        }
        rms_block_sum<1>(ss, red[it & 1]);
        const float rstd = rms_rstd(ss[0], inv_h, eps);
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float z = Cvt<T>::to_f(x[off + c]);
            if (RESIDUAL) z += Cvt<T>::to_f(residual[off + c]);
            out[off + c] = Cvt<T>::from_f(z * rstd * Cvt<T>::to_f(weight[c]));
        }
        if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    }
}

// ---------------------------------------------------------------------------------------------
// backward (register-resident row, dweight partials in registers)
//   rstd_in == nullptr  recompute rstd from x and eps (the reference's rmsnorm_backward)
//   dres != nullptr     dx = round(dx) + dres, the two roundings of the reference's
//                       `dz.add_(dresidual_out)` on a tensor of the input dtype
//   partial != nullptr  this CTA's dweight contributions go to partial[blockIdx.x][H]
// ---------------------------------------------------------------------------------------------
template <class T, int VPT, bool VECTOR>
__global__ void __launch_bounds__(kRmsMaxThreads)
rms_backward_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ weight,
                    const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
                    float* __restrict__ partial, int n_rows, int H, float eps) {
    const float inv_h = 1.0f / static_cast<float>(H);
    constexpr int VEC = RmsTile<T>::kVec;
    constexpr int ROWS = RmsRows<VPT>::kRows;
    constexpr bool kWeightInRegs = VPT * VEC <= 16;  // wider rows re-read the weights (L1 hits) every step
    __shared__ float red[2][2 * ROWS * 32];
    const int t = threadIdx.x;

    uint4 wraw[kWeightInRegs ? VPT : 1];
    if (kWeightInRegs) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) wraw[i] = rms_load<T, VECTOR>(weight, (i * blockDim.x + t) * VEC, H);
    }
    float dwacc[VPT][VEC];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) dwacc[i][j] = 0.f;

    int it = 0;
    for (int row0 = blockIdx.x * ROWS; row0 < n_rows; row0 += gridDim.x * ROWS, ++it) {
        uint4 rdy[ROWS][VPT], rx[ROWS][VPT];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const long long off = static_cast<long long>(row0 + r) * H;
            const int h = row0 + r < n_rows ? H : 0;  // rows past the end read as zeros
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int c = (i * blockDim.x + t) * VEC;
                rdy[r][i] = rms_load<T, VECTOR>(dy + off, c, h);
                rx[r][i] = rms_load<T, VECTOR>(x + off, c, h);
            }
        }
        // pass A over the registers: per row c = sum(dy * w * x) and sum(x^2)
        float sums[2 * ROWS];
#pragma unroll
        for (int r = 0; r < 2 * ROWS; ++r) sums[r] = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float w[VEC];
            if (kWeightInRegs) rms_unpack<T>(wraw[i], w);
            else rms_unpack<T>(rms_load<T, VECTOR>(weight, (i * blockDim.x + t) * VEC, H), w);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float d[VEC], xv[VEC];
                rms_unpack<T>(rdy[r][i], d);
                rms_unpack<T>(rx[r][i], xv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    sums[2 * r] = fmaf(d[j] * w[j], xv[j], sums[2 * r]);
                    sums[2 * r + 1] = fmaf(xv[j], xv[j], sums[2 * r + 1]);
                }
            }
        }
        rms_block_sum<2 * ROWS>(sums, red[it & 1]);
        // pass B: the rows stayed packed in registers; unpack one vector at a time
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const long long off = static_cast<long long>(row0 + r) * H;
            const int h = row0 + r < n_rows ? H : 0;
            float rstd = 0.f;  // a row past the end adds nothing to dweight
            if (h != 0)
                rstd = rstd_in != nullptr ? rstd_in[row0 + r]
                                          : rms_rstd(sums[2 * r + 1], inv_h, eps);
            const float coef = rstd * rstd * rstd * inv_h;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int c = (i * blockDim.x + t) * VEC;
                float w[VEC], d[VEC], xv[VEC], o[VEC];
                if (kWeightInRegs) rms_unpack<T>(wraw[i], w);
                else rms_unpack<T>(rms_load<T, VECTOR>(weight, c, H), w);
                rms_unpack<T>(rdy[r][i], d);
                rms_unpack<T>(rx[r][i], xv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    dwacc[i][j] = fmaf(d[j] * xv[j], rstd, dwacc[i][j]);
                    o[j] = rstd * (d[j] * w[j]) - coef * xv[j] * sums[2 * r];
                }
                if (dres != nullptr) {
                    float q[VEC];
                    rms_unpack<T>(rms_load<T, VECTOR>(dres + off, c, h), q);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) o[j] = Cvt<T>::to_f(Cvt<T>::from_f(o[j])) + q[j];
                }
                rms_store<T, VECTOR>(dx + off, c, h, rms_pack<T>(o));
            }
        }
    }
    if (partial != nullptr) {
        float* prow = partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = (i * blockDim.x + t) * VEC;
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (c + j < H) prow[c + j] = dwacc[i][j];
        }
    }
}

// backward, any width: pass 1 forms c (and rstd), pass 2 writes dx; rstd goes to rstd_ws for the
// column kernel below.
template <class T>
__global__ void __launch_bounds__(kRmsMaxThreads)
rms_backward_wide_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ weight,
                         const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
                         float* __restrict__ rstd_ws, int n_rows, int H, float eps) {
    const float inv_h = 1.0f / static_cast<float>(H);
    __shared__ float red[2][64];
    int it = 0;
    for (int row = blockIdx.x; row < n_rows; row += gridDim.x, ++it) {
        const long long off = static_cast<long long>(row) * H;
        float sums[2] = {0.f, 0.f};
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float xv = Cvt<T>::to_f(x[off + c]);
            const float wd = Cvt<T>::to_f(dy[off + c]) * Cvt<T>::to_f(weight[c]);
            sums[0] = fmaf(wd, xv, sums[0]);
            sums[1] = fmaf(xv, xv, sums[1]);
        }
        rms_block_sum<2>(sums, red[it & 1]);
        const float rstd = rstd_in != nullptr ? rstd_in[row] : rms_rstd(sums[1], inv_h, eps);
        const float coef = rstd * rstd * rstd * inv_h;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float xv = Cvt<T>::to_f(x[off + c]);
            const float wd = Cvt<T>::to_f(dy[off + c]) * Cvt<T>::to_f(weight[c]);
            float o = rstd * wd - coef * xv * sums[0];
            if (dres != nullptr) o = Cvt<T>::to_f(Cvt<T>::from_f(o)) + Cvt<T>::to_f(dres[off + c]);
            dx[off + c] = Cvt<T>::from_f(o);
        }
        if (threadIdx.x == 0 && rstd_ws != nullptr) rstd_ws[row] = rstd;
    }
}

// dweight partials for the wide form: one thread per column, one partial row per block of rows.
template <class T>
__global__ void __launch_bounds__(256)
rms_dw_wide_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ rstd,
                   float* __restrict__ partial, int n_rows, int H, int rows_per_block) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= H) return;
    const int r0 = blockIdx.y * rows_per_block;
    const int r1 = min(n_rows, r0 + rows_per_block);
    float acc = 0.f;
    for (int r = r0; r < r1; ++r) {
        const long long off = static_cast<long long>(r) * H + col;
        acc = fmaf(Cvt<T>::to_f(dy[off]) * Cvt<T>::to_f(x[off]), rstd[r], acc);
    }
    partial[static_cast<long long>(blockIdx.y) * H + col] = acc;
}

// dweight[col] = sum over partial rows, in a fixed order: 8 strided sub-sums per column, then those
// 8 in order. Block (32, 8): 32 consecutive columns per CTA.
template <class T>
__global__ void __launch_bounds__(256)
rms_dw_reduce_kernel(const float* __restrict__ partial, int n_partials, int H, T* __restrict__ dweight) {
    __shared__ float sm[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    float a0 = 0.f, a1 = 0.f;
    if (col < H) {
        int p = threadIdx.y;
        for (; p + 8 < n_partials; p += 16) {
            a0 += partial[static_cast<long long>(p) * H + col];
            a1 += partial[static_cast<long long>(p + 8) * H + col];
        }
        if (p < n_partials) a0 += partial[static_cast<long long>(p) * H + col];
    }
    sm[threadIdx.y][threadIdx.x] = a0 + a1;
    __syncthreads();
    if (threadIdx.y == 0 && col < H) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += sm[k][threadIdx.x];
        dweight[col] = Cvt<T>::from_f(s);
    }
}

}  // namespace lce
