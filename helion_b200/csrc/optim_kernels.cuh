// Consumers of dW: the AdamW step (the reference's tritium.adamw_step, tritium/ops/adamw.py:21-54) and the
// sum of squares behind gradient clipping (helion.clip_grad_norm, helion/training.py:36-49). Both are
// bandwidth-bound streaming kernels over tensors the loss path has just written.
#pragma once

#include "row_kernels.cuh"

namespace lce {

constexpr int kOptThreads = 256;

// One thread = one 16-byte vector of the parameter (8 16-bit or 4 fp32 elements) per grid-stride step.
// Arithmetic exactly as the reference kernel, in fp32:
//   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p -= lr wd p;  p -= (lr / bc1) m / (sqrt(v / bc2) + eps)
// grad_scale (optional device scalar) multiplies g first: the clipping coefficient applied without a
// separate pass over the gradients.
template <class T>
__global__ void __launch_bounds__(kOptThreads)
adamw_step_kernel(T* __restrict__ param, const T* __restrict__ grad, float* __restrict__ exp_avg,
                  float* __restrict__ exp_avg_sq, long long n, float lr, float beta1, float beta2, float eps,
                  float weight_decay, float bias_correction1, float bias_correction2,
                  const float* __restrict__ grad_scale) {
    constexpr int VEC = 16 / sizeof(T);
    const float gs = grad_scale ? *grad_scale : 1.f;
    const float step_size = lr / bias_correction1;
    const long long n_vec = n / VEC;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec; i += stride) {
        alignas(16) T p[VEC], g[VEC];
        alignas(16) float m[VEC], v[VEC];
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(param + i * VEC);
        *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(grad + i * VEC);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            *reinterpret_cast<float4*>(m + 4 * q) = *reinterpret_cast<const float4*>(exp_avg + i * VEC + 4 * q);
            *reinterpret_cast<float4*>(v + 4 * q) = *reinterpret_cast<const float4*>(exp_avg_sq + i * VEC + 4 * q);
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float gj = Cvt<T>::to_f(g[j]) * gs;
            float pj = Cvt<T>::to_f(p[j]);
            m[j] = beta1 * m[j] + (1.f - beta1) * gj;
            v[j] = beta2 * v[j] + (1.f - beta2) * gj * gj;
            pj = pj - lr * weight_decay * pj;
            pj = pj - step_size * m[j] / (sqrtf(v[j] / bias_correction2) + eps);
            p[j] = Cvt<T>::from_f(pj);
        }
        *reinterpret_cast<uint4*>(param + i * VEC) = *reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            *reinterpret_cast<float4*>(exp_avg + i * VEC + 4 * q) = *reinterpret_cast<const float4*>(m + 4 * q);
            *reinterpret_cast<float4*>(exp_avg_sq + i * VEC + 4 * q) = *reinterpret_cast<const float4*>(v + 4 * q);
        }
    }
    // ragged tail (n not a multiple of the vector width): the last few elements, one thread each
    const long long tail0 = n_vec * VEC;
    const long long t = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (t < n) {
        const float gj = Cvt<T>::to_f(grad[t]) * gs;
        float pj = Cvt<T>::to_f(param[t]);
        const float mj = beta1 * exp_avg[t] + (1.f - beta1) * gj;
        const float vj = beta2 * exp_avg_sq[t] + (1.f - beta2) * gj * gj;
        pj = pj - lr * weight_decay * pj;
        pj = pj - step_size * mj / (sqrtf(vj / bias_correction2) + eps);
        exp_avg[t] = mj;
        exp_avg_sq[t] = vj;
        param[t] = Cvt<T>::from_f(pj);
    }
}

// Sum of squares, deterministically: a fixed grid of kSumsqBlocks CTAs, each a fixed strided serial
// sum per thread plus a fixed tree, writes one partial; the last step adds the partials in order.
constexpr int kSumsqBlocks = 1184;  // 148 x 8

template <class T>
__global__ void __launch_bounds__(kOptThreads)
sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partials) {
    __shared__ float sh[kOptThreads];
    constexpr int VEC = 16 / sizeof(T);
    const long long n_vec = n / VEC;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    float a0 = 0.f, a1 = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec; i += stride) {
        alignas(16) T v[VEC];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(x + i * VEC);
#pragma unroll
        for (int j = 0; j < VEC; j += 2) {
            const float u = Cvt<T>::to_f(v[j]), w = Cvt<T>::to_f(v[j + 1]);
            a0 = fmaf(u, u, a0);
            a1 = fmaf(w, w, a1);
        }
    }
    const long long t = n_vec * VEC + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (t < n) {
        const float u = Cvt<T>::to_f(x[t]);
        a0 = fmaf(u, u, a0);
    }
    sh[threadIdx.x] = a0 + a1;
    __syncthreads();
    for (int off = kOptThreads / 2; off > 0; off >>= 1) {
        if (threadIdx.x < off) sh[threadIdx.x] += sh[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) partials[blockIdx.x] = sh[0];
}

// out (+)= sum of the partials, added in index order by one CTA.
__global__ void __launch_bounds__(1024)
sumsq_final_kernel(const float* __restrict__ partials, int count, float* __restrict__ out, int accumulate) {
    __shared__ float sh[1024];
    float acc = 0.f;
    for (int i = threadIdx.x; i < count; i += 1024) acc += partials[i];
    const float total = block_sum_1024(acc, sh);
    if (threadIdx.x == 0) *out = accumulate ? *out + total : total;
}

}  // namespace lce
