// CUDA-core GEMM used where the tensor-core path does not apply: fp32 inputs
// (the fp32 tolerance of 1e-4 rules out TF32), rows whose byte stride is not a
// multiple of 16 (TMA cannot address them) and very small problems.
//   y[m,n] = sum_k x[m,k] * w[n,k] (+ bias[n]),  fp32 accumulate, one rounding.
// 64x64 output tile per CTA, 16-wide K slabs staged in shared memory as fp32,
// 4x4 outputs per thread; every edge is predicated so any M, N, K works.
#pragma once

#include "common.cuh"

namespace cck {

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                 T* __restrict__ y, int64_t m, int64_t k, int64_t n) {
    __shared__ float xs[kSimtK][kSimtTile + 4];
    __shared__ float ws[kSimtK][kSimtTile + 4];
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kSimtTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kSimtTile;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12

    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < k; k0 += kSimtK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int64_t kk = k0 + lk + e;
            const int64_t xr = m0 + lr, wr = n0 + lr;
            xs[lk + e][lr] = (xr < m && kk < k) ? Store<T>::load1(x + xr * k + kk) : 0.0f;
            ws[lk + e][lr] = (wr < n && kk < k) ? Store<T>::load1(w + wr * k + kk) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSimtK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = xs[kk][ty * 4 + i];
                b[i] = ws[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = m0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = n0 + tx * 4 + j;
            if (c < n) {
                const float b = bias ? Store<T>::load1(bias + c) : 0.0f;
                Store<T>::store1(y + r * n + c, acc[i][j] + b);
            }
        }
    }
}

template <typename T>
cudaError_t gemm_simt(const void* x, const void* w, const void* bias, void* y, int64_t m, int64_t k,
                      int64_t n, cudaStream_t s) {
    const int64_t gx = ceil_div64(n, kSimtTile), gy = ceil_div64(m, kSimtTile);
    if (gy > 65535) return cudaErrorInvalidValue;
    gemm_simt_kernel<T><<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, s>>>(
        static_cast<const T*>(x), static_cast<const T*>(w), static_cast<const T*>(bias),
        static_cast<T*>(y), m, k, n);
    return cudaGetLastError();
}

// The same tiling for the FP8 GEMM where the tensor-core path does not apply (K not a multiple
// of 16, unaligned operands, very small problems): operands are one-byte float8 codes
// (e4m3 when !E5M2), decoded to fp32 in shared memory; epilogue
//   y = acc * a_scale[m] * w_scale[n] + bias[n]   (the tensor-core epilogue's formula).
template <bool E5M2>
__device__ __forceinline__ float fp8_code_to_float(uint8_t c) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half2float(__half(h));
}

template <typename T>
__global__ void __launch_bounds__(256)
gemm_fp8_simt_kernel(const uint8_t* __restrict__ x, const float* __restrict__ x_scale, const uint8_t* __restrict__ w,
                     const float* __restrict__ w_scale, const T* __restrict__ bias, T* __restrict__ y, int64_t m,
                     int64_t k, int64_t n) {
    __shared__ float xs[kSimtK][kSimtTile + 4];
    __shared__ float ws[kSimtK][kSimtTile + 4];
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kSimtTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kSimtTile;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;

    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < k; k0 += kSimtK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int64_t kk = k0 + lk + e;
            const int64_t xr = m0 + lr, wr = n0 + lr;
            xs[lk + e][lr] = (xr < m && kk < k) ? fp8_code_to_float<false>(x[xr * k + kk]) : 0.0f;
            ws[lk + e][lr] = (wr < n && kk < k) ? fp8_code_to_float<false>(w[wr * k + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSimtK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = xs[kk][ty * 4 + i];
                b[i] = ws[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = m0 + ty * 4 + i;
        if (r >= m) continue;
        const float sa = x_scale[r];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = n0 + tx * 4 + j;
            if (c < n) {
                const float b = bias ? Store<T>::load1(bias + c) : 0.0f;
                Store<T>::store1(y + r * n + c, fmaf(acc[i][j] * sa, w_scale[c], b));
            }
        }
    }
}

template <typename T>
cudaError_t gemm_fp8_simt(const uint8_t* x, const float* x_scale, const uint8_t* w, const float* w_scale,
                          const void* bias, void* y, int64_t m, int64_t k, int64_t n, cudaStream_t s) {
    const int64_t gx = ceil_div64(n, kSimtTile), gy = ceil_div64(m, kSimtTile);
    if (gy > 65535) return cudaErrorInvalidValue;
    gemm_fp8_simt_kernel<T><<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, s>>>(
        x, x_scale, w, w_scale, static_cast<const T*>(bias), static_cast<T*>(y), m, k, n);
    return cudaGetLastError();
}

}  // namespace cck
