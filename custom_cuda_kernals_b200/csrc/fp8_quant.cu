// Dynamic FP8 quantisation: scale = max(amax / FP8_MAX, 1e-12), code = fp8(x / scale).
// Three scale granularities:
//   token  - one scale per row            (scale [M,1]);      one launch, row read once
//   block  - one scale per 128x128 tile   (scale [ceil(M/128), ceil(N/128)]); one launch, tile read once
//   tensor - one scale for the matrix     (scale [1]);        amax launch + cast launch
//
// Replaces the reference's csrc/kernels/fp8_quant.cu:66-314 (block and tensor;
// token granularity has no counterpart there).  Differences that matter:
//   * Both divisions are IEEE round-to-nearest (`amax / FP8_MAX` and `x / scale`),
//     as in the PyTorch baseline (baselines/fp8_quant.py:162-178), so codes and
//     scales are bit-identical to it.  The reference kernel multiplies by an
//     approximate reciprocal and is off by one code on ~5e-4 of the elements.
//     `x / scale` is evaluated as a correctly rounded quotient from the correctly
//     rounded reciprocal of the (row / tile / tensor-wide) scale and two
//     FMA residual corrections (struct ExactDiv) - 6 instructions per element
//     instead of a full division.  This file must not be compiled with
//     --use_fast_math.
//   * The row / tile is held in registers between the amax pass and the cast,
//     so HBM is read once; loads are 16-byte, stores are 16 codes (16 bytes).
//
// HBM-bound: M*N*(sizeof(T) + 1) bytes per launch (+ scales).
#include "common.cuh"

namespace cck {
namespace {

constexpr float kScaleFloor = 1e-12f;
constexpr int kTile = 128;

template <bool E5M2> struct Fmt;
template <> struct Fmt<false> {
    static constexpr float kMax = 448.0f;
    __device__ static __forceinline__ uint32_t cvt2(float lo, float hi) {
        return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
    }
};
template <> struct Fmt<true> {
    static constexpr float kMax = 57344.0f;
    __device__ static __forceinline__ uint32_t cvt2(float lo, float hi) {
        return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E5M2);
    }
};

template <bool E5M2>
__device__ __forceinline__ float scale_of(float amax) {
    return fmaxf(__fdiv_rn(amax, Fmt<E5M2>::kMax), kScaleFloor);
}
// a / s, correctly rounded, for a fixed positive finite divisor s.
// With y = RN(1/s): q0 = RN(a*y) is within 1.5 ulp of a/s; one residual step
// makes it faithful (within 1 ulp); for a faithful q the residual a - s*q is
// exact in an FMA and RN(q + r*y) is the correctly rounded quotient (Markstein's
// theorem).  No intermediate can underflow while the quotient still matters:
// s >= 1e-12 and |a/s| <= FP8_MAX, and a quotient below 2^-11 becomes a zero code
// whatever its last bits are.  The sign is taken from `a` so that -0.0 stays -0.0.
struct ExactDiv {
    float s, y;
    __device__ __forceinline__ explicit ExactDiv(float scale) : s(scale), y(__frcp_rn(scale)) {}
    __device__ __forceinline__ float operator()(float a) const {
        const float q0 = __fmul_rn(a, y);
        const float r0 = __fmaf_rn(-s, q0, a);
        const float q1 = __fmaf_rn(r0, y, q0);
        const float r1 = __fmaf_rn(-s, q1, a);
        return copysignf(__fmaf_rn(r1, y, q1), a);
    }
};

template <bool E5M2>
__device__ __forceinline__ uint8_t quant1(float x, float scale) {
    return static_cast<uint8_t>(Fmt<E5M2>::cvt2(ExactDiv(scale)(x), 0.0f) & 0xffu);
}

// A "unit" is 16 consecutive elements: 16*sizeof(T) bytes in, 16 bytes out.
template <typename T> struct Unit {
    static constexpr int kVecs = 16 / Store<T>::kPerVec;  // Vec16 per unit: 2 (16-bit) or 4 (fp32)
    Vec16 v[kVecs];
    __device__ __forceinline__ void load(const T* p) {
#pragma unroll
        for (int i = 0; i < kVecs; ++i) v[i] = ld_stream(p + i * Store<T>::kPerVec);
    }
    __device__ __forceinline__ float amax() const {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < kVecs; ++i)
#pragma unroll
            for (int e = 0; e < Store<T>::kPerVec; ++e) m = fmaxf(m, fabsf(Store<T>::get(v[i], e)));
        return m;
    }
    template <bool E5M2>
    __device__ __forceinline__ Vec16 quantise(float scale) const {
        Vec16 out;
        float f[16];
        const ExactDiv div(scale);
#pragma unroll
        for (int i = 0; i < kVecs; ++i)
#pragma unroll
            for (int e = 0; e < Store<T>::kPerVec; ++e)
                f[i * Store<T>::kPerVec + e] = div(Store<T>::get(v[i], e));
#pragma unroll
        for (int w = 0; w < 4; ++w)
            out.w[w] = Fmt<E5M2>::cvt2(f[4 * w], f[4 * w + 1]) | (Fmt<E5M2>::cvt2(f[4 * w + 2], f[4 * w + 3]) << 16);
        return out;
    }
};

__device__ __forceinline__ float cta_max_dyn(float v, float* slots) {
    v = warp_max(v);
    const int warps = blockDim.x >> 5;
    if (warps == 1) return v;
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    for (int i = 0; i < warps; ++i) r = fmaxf(r, slots[i]);
    __syncthreads();
    return r;
}

// ------------------------------------------------------------------ token granularity
template <typename T, bool E5M2, int UPT>
__global__ void __launch_bounds__(1024)
fp8_token_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                 int64_t n, int units) {
    __shared__ float slots[32];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * n;
    uint8_t* cr = codes + row * n;
    Unit<T> u[UPT];
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < UPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < units) u[j].load(xr + static_cast<int64_t>(i) * 16);
    }
#pragma unroll
    for (int j = 0; j < UPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < units) m = fmaxf(m, u[j].amax());
    }
    const float sc = scale_of<E5M2>(cta_max_dyn(m, slots));
    if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
    for (int j = 0; j < UPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < units) st_stream(cr + static_cast<int64_t>(i) * 16, u[j].template quantise<E5M2>(sc));
    }
}

// any n / alignment: scalar, the row is read twice (second time from L1/L2)
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
fp8_token_generic_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                         int64_t n) {
    __shared__ float slots[32];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * n;
    float m = 0.0f;
    for (int64_t c = threadIdx.x; c < n; c += blockDim.x) m = fmaxf(m, fabsf(Store<T>::load1(xr + c)));
    const float sc = scale_of<E5M2>(cta_max_dyn(m, slots));
    if (threadIdx.x == 0) scale[row] = sc;
    for (int64_t c = threadIdx.x; c < n; c += blockDim.x)
        codes[row * n + c] = quant1<E5M2>(Store<T>::load1(xr + c), sc);
}

// ------------------------------------------------------------------ block granularity
// One CTA of 256 threads per 128x128 tile: 8 units per tile row, 4 units per thread.
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
fp8_block_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                 int64_t m, int64_t n) {
    __shared__ float slots[32];
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kTile, c0 = static_cast<int64_t>(blockIdx.x) * kTile;
    Unit<T> u[4];
    bool live[4];
    int64_t off[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int id = threadIdx.x + j * 256;   // 0..1023
        const int64_t r = r0 + (id >> 3), c = c0 + (id & 7) * 16;
        live[j] = r < m && c < n;               // n % 16 == 0 on this path
        off[j] = r * n + c;
        if (live[j]) u[j].load(x + off[j]);
    }
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (live[j]) mx = fmaxf(mx, u[j].amax());
    const float sc = scale_of<E5M2>(cta_max_dyn(mx, slots));
    if (threadIdx.x == 0) scale[static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x] = sc;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (live[j]) st_stream(codes + off[j], u[j].template quantise<E5M2>(sc));
}

template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
fp8_block_generic_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                         int64_t m, int64_t n) {
    __shared__ float slots[32];
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kTile, c0 = static_cast<int64_t>(blockIdx.x) * kTile;
    float mx = 0.0f;
    for (int id = threadIdx.x; id < kTile * kTile; id += 256) {
        const int64_t r = r0 + (id >> 7), c = c0 + (id & 127);
        if (r < m && c < n) mx = fmaxf(mx, fabsf(Store<T>::load1(x + r * n + c)));
    }
    const float sc = scale_of<E5M2>(cta_max_dyn(mx, slots));
    if (threadIdx.x == 0) scale[static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x] = sc;
    for (int id = threadIdx.x; id < kTile * kTile; id += 256) {
        const int64_t r = r0 + (id >> 7), c = c0 + (id & 127);
        if (r < m && c < n) codes[r * n + c] = quant1<E5M2>(Store<T>::load1(x + r * n + c), sc);
    }
}

// ------------------------------------------------------------------ tensor granularity
// Pass 1: amax into *amax_bits (caller-zeroed).  Non-negative floats order like ints.
template <typename T>
__global__ void __launch_bounds__(256)
fp8_amax_kernel(const T* __restrict__ x, int32_t* __restrict__ amax_bits, int64_t total, bool vec_ok) {
    __shared__ float slots[32];
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    float m = 0.0f;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t n_vec = total / kPer;
        for (int64_t i = tid; i < n_vec; i += stride) {
            const Vec16 v = ld_cached(x + i * kPer);   // default policy: the cast pass re-reads it from L2
#pragma unroll
            for (int e = 0; e < kPer; ++e) m = fmaxf(m, fabsf(Store<T>::get(v, e)));
        }
        done = n_vec * kPer;
    }
    for (int64_t i = done + tid; i < total; i += stride) m = fmaxf(m, fabsf(Store<T>::load1(x + i)));
    m = cta_max_dyn(m, slots);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_int(m));
}

// Pass 2: cast with the tensor-wide scale.
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
fp8_cast_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                const int32_t* __restrict__ amax_bits, int64_t total, bool vec_ok) {
    const float sc = scale_of<E5M2>(__int_as_float(*amax_bits));
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    if (tid == 0) scale[0] = sc;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t units = total / 16;
        for (int64_t i = tid; i < units; i += stride) {
            Unit<T> u;
            u.load(x + i * 16);
            st_stream(codes + i * 16, u.template quantise<E5M2>(sc));
        }
        done = units * 16;
    }
    for (int64_t i = done + tid; i < total; i += stride) codes[i] = quant1<E5M2>(Store<T>::load1(x + i), sc);
}

// ------------------------------------------------------------------ host dispatch
template <typename T, bool E5M2>
cudaError_t run_token(const void* x, uint8_t* codes, float* scale, int64_t m, int64_t n, cudaStream_t s) {
    if (m > 0x7fffffffLL) return cudaErrorInvalidValue;
    const T* xp = static_cast<const T*>(x);
    const unsigned grid = static_cast<unsigned>(m);
    const int64_t units = n / 16;
    if (n % 16 == 0 && aligned16(x) && aligned16(codes) && units <= 8 * 1024) {
        const int upt = units <= 2048 ? 2 : (units <= 4096 ? 4 : 8);
        int threads = static_cast<int>(ceil_div64(ceil_div64(units, upt), 32) * 32);
        if (threads < 32) threads = 32;
        const int un = static_cast<int>(units);
        if (upt == 2) fp8_token_kernel<T, E5M2, 2><<<grid, threads, 0, s>>>(xp, codes, scale, n, un);
        else if (upt == 4) fp8_token_kernel<T, E5M2, 4><<<grid, threads, 0, s>>>(xp, codes, scale, n, un);
        else fp8_token_kernel<T, E5M2, 8><<<grid, threads, 0, s>>>(xp, codes, scale, n, un);
    } else {
        fp8_token_generic_kernel<T, E5M2><<<grid, 256, 0, s>>>(xp, codes, scale, n);
    }
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_block(const void* x, uint8_t* codes, float* scale, int64_t m, int64_t n, cudaStream_t s) {
    const int64_t gx = ceil_div64(n, kTile), gy = ceil_div64(m, kTile);
    if (gy > 65535 || gx > 0x7fffffffLL) return cudaErrorInvalidValue;
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    const T* xp = static_cast<const T*>(x);
    if (n % 16 == 0 && aligned16(x) && aligned16(codes))
        fp8_block_kernel<T, E5M2><<<grid, 256, 0, s>>>(xp, codes, scale, m, n);
    else
        fp8_block_generic_kernel<T, E5M2><<<grid, 256, 0, s>>>(xp, codes, scale, m, n);
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_tensor(const void* x, uint8_t* codes, float* scale, int32_t* amax_bits, int64_t m, int64_t n,
                       cudaStream_t s) {
    const T* xp = static_cast<const T*>(x);
    const int64_t total = m * n;
    const bool vec_ok = aligned16(x) && aligned16(codes);
    int64_t ctas = ceil_div64(total, 256 * 16);
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    fp8_amax_kernel<T><<<static_cast<unsigned>(ctas), 256, 0, s>>>(xp, amax_bits, total, vec_ok);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    fp8_cast_kernel<T, E5M2><<<static_cast<unsigned>(ctas), 256, 0, s>>>(xp, codes, scale, amax_bits, total, vec_ok);
    return cudaGetLastError();
}

enum Gran { kToken, kBlock, kTensor };

template <typename T>
cudaError_t by_format(Gran g, const void* x, uint8_t* codes, float* scale, int32_t* amax_bits, int64_t m,
                      int64_t n, int32_t fp8_format, cudaStream_t s) {
    const bool e5 = fp8_format == kF8E5M2;
    if (!e5 && fp8_format != kF8E4M3) return cudaErrorInvalidValue;
    switch (g) {
        case kToken:
            return e5 ? run_token<T, true>(x, codes, scale, m, n, s) : run_token<T, false>(x, codes, scale, m, n, s);
        case kBlock:
            return e5 ? run_block<T, true>(x, codes, scale, m, n, s) : run_block<T, false>(x, codes, scale, m, n, s);
        default:
            return e5 ? run_tensor<T, true>(x, codes, scale, amax_bits, m, n, s)
                      : run_tensor<T, false>(x, codes, scale, amax_bits, m, n, s);
    }
}

cudaError_t dispatch(Gran g, const void* x, uint8_t* codes, float* scale, int32_t* amax_bits, int64_t m,
                     int64_t n, int32_t dtype, int32_t fp8_format, void* stream) {
    if (m <= 0 || n <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case kF32:  return by_format<float>(g, x, codes, scale, amax_bits, m, n, fp8_format, s);
        case kF16:  return by_format<__half>(g, x, codes, scale, amax_bits, m, n, fp8_format, s);
        case kBF16: return by_format<__nv_bfloat16>(g, x, codes, scale, amax_bits, m, n, fp8_format, s);
        default:    return cudaErrorInvalidValue;
    }
}

}  // namespace
}  // namespace cck

extern "C" int32_t launch_fp8_quant_token_fwd(const void* x, uint8_t* x_fp8, float* scale, int64_t m, int64_t n,
                                              int32_t dtype, int32_t fp8_format, void* stream) {
    return cck::dispatch(cck::kToken, x, x_fp8, scale, nullptr, m, n, dtype, fp8_format, stream);
}

extern "C" int32_t launch_fp8_quant_block_fwd(const void* x, uint8_t* x_fp8, float* scale, int64_t m, int64_t n,
                                              int32_t dtype, int32_t fp8_format, void* stream) {
    return cck::dispatch(cck::kBlock, x, x_fp8, scale, nullptr, m, n, dtype, fp8_format, stream);
}

extern "C" int32_t launch_fp8_quant_tensor_fwd(const void* x, uint8_t* x_fp8, float* scale, int32_t* amax_scratch,
                                               int64_t m, int64_t n, int32_t dtype, int32_t fp8_format,
                                               void* stream) {
    if (amax_scratch == nullptr && m > 0 && n > 0) return cudaErrorInvalidValue;
    return cck::dispatch(cck::kTensor, x, x_fp8, scale, amax_scratch, m, n, dtype, fp8_format, stream);
}
