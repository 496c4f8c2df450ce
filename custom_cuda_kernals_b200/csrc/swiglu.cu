// SwiGLU gated activation: y = silu(gate) * up, flat over n elements.
//
// Replaces the reference's csrc/kernels/swiglu.cu:49-206 (three kernels plus a
// second launch for the scalar tail).  One kernel here: every thread keeps
// kUnroll 16-byte vectors of `gate` and of `up` in flight (2*kUnroll loads
// issued before the first use), the ragged tail (n not a multiple of the vector
// width) is folded into the last CTA, and read-once / write-once traffic uses
// streaming cache policies.  Rounding follows the PyTorch baseline
// (baselines/swiglu.py:109-112): silu in fp32, rounded to the storage type,
// then multiplied by `up` and rounded again.
//
// HBM-bound: 3 tensors * n * sizeof(T) bytes per launch.
#include "common.cuh"

namespace cck {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y,
              int64_t n_vec, int64_t n) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;
    const Vec16* g16 = reinterpret_cast<const Vec16*>(gate);
    const Vec16* u16 = reinterpret_cast<const Vec16*>(up);
    Vec16* y16 = reinterpret_cast<Vec16*>(y);

    Vec16 gv[kUnroll], uv[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
        const int64_t i = base + static_cast<int64_t>(j) * kThreads;
        if (i < n_vec) {
            gv[j] = ld_stream(g16 + i);
            uv[j] = ld_stream(u16 + i);
        }
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
        const int64_t i = base + static_cast<int64_t>(j) * kThreads;
        if (i < n_vec) {
            float g[kPer], u[kPer], o[kPer];
            unpack<T>(gv[j], g);
            unpack<T>(uv[j], u);
#pragma unroll
            for (int e = 0; e < kPer; ++e) o[e] = glu1<T>(g[e], u[e]);
            st_stream(y16 + i, pack<T>(o));
        }
    }
    // ragged tail: fewer than one vector of elements, done by the last CTA
    if (blockIdx.x == gridDim.x - 1) {
        const int64_t t = n_vec * kPer + threadIdx.x;
        if (t < n) Store<T>::store1(y + t, glu1<T>(Store<T>::load1(gate + t), Store<T>::load1(up + t)));
    }
}

// Fallback for buffers that are not 16-byte aligned (sliced views).
template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
        Store<T>::store1(y + i, glu1<T>(Store<T>::load1(gate + i), Store<T>::load1(up + i)));
}

template <typename T>
cudaError_t run(const void* gate, const void* up, void* y, int64_t n, cudaStream_t stream) {
    const T* g = static_cast<const T*>(gate);
    const T* u = static_cast<const T*>(up);
    T* o = static_cast<T*>(y);
    if (aligned16(gate) && aligned16(up) && aligned16(y)) {
        const int64_t n_vec = n / Store<T>::kPerVec;
        const int64_t ctas = ceil_div64(n_vec, kThreads * kUnroll);
        swiglu_kernel<T><<<static_cast<unsigned>(ctas > 0 ? ctas : 1), kThreads, 0, stream>>>(g, u, o, n_vec, n);
    } else {
        const int64_t ctas = ceil_div64(n, kThreads);
        const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
        swiglu_scalar_kernel<T><<<static_cast<unsigned>(ctas < cap ? ctas : cap), kThreads, 0, stream>>>(g, u, o, n);
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace cck

extern "C" int32_t launch_swiglu_fwd(const void* gate, const void* up, void* y, int64_t n,
                                     int32_t dtype, void* stream) {
    if (n <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run<float>(gate, up, y, n, s);
        case cck::kF16:  return cck::run<__half>(gate, up, y, n, s);
        case cck::kBF16: return cck::run<__nv_bfloat16>(gate, up, y, n, s);
        default:         return cudaErrorInvalidValue;
    }
}

CCK_DEBUG_BOUNDS_EXPORT(swiglu)
