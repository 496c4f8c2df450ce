// Shared device helpers for the bandwidth-bound kernels: storage-type traits,
// 16-byte streaming loads/stores, warp and CTA reductions.
//
// Covers the role of the reference's csrc/includes/common.cuh:28-153 (dtype
// tags, to_float/from_float, warp/block reductions) with a different design:
// every global access is a 128-bit vector, reductions use xor-shuffles so all
// lanes end with the result, and loads that are read once bypass L1.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cck {

// dtype tags of the C ABI (values fixed by the reference: src/kernels/dtype.rs:6-12).
enum : int32_t { kF32 = 0, kF16 = 1, kBF16 = 2, kF8E4M3 = 3, kF8E5M2 = 4 };

constexpr int kNumSMs = 148;  // B200

// ---------------------------------------------------------------- debug bounds build
// With -DCC_DEBUG_BOUNDS (python -m custom_cuda_kernals_b200._build --debug-bounds) every global
// access that goes through the helpers below (16-byte vector loads / stores and the scalar
// Store<T>::load1 / store1) is first checked against a table of address ranges the host
// registered for the launch; an access outside every range is SKIPPED and counted, so a wrong
// index shows up as a count instead of a fault.  Stands in for compute-sanitizer's memcheck on
// machines where that tool is not available.  Each translation unit has its own table; the
// CCK_DEBUG_BOUNDS_EXPORT(tag) macro at the end of a .cu file exports its two host calls:
//   cck_dbg_set_ranges_<tag>(const void* const* base, const int64_t* bytes, int n)   (n <= 8; clears the count)
//   cck_dbg_take_violations_<tag>(uint32_t* out)                                     (synchronises)
#ifdef CC_DEBUG_BOUNDS
namespace dbg {
constexpr int kMaxRanges = 8;
struct Table {
    unsigned long long lo[kMaxRanges], hi[kMaxRanges];
    int n;
    unsigned int violations;
};
static __device__ Table g_table;
__device__ __forceinline__ bool ok(const void* p, unsigned bytes) {
    const unsigned long long a = reinterpret_cast<unsigned long long>(p);
    for (int i = 0; i < g_table.n; ++i)
        if (a >= g_table.lo[i] && a + bytes <= g_table.hi[i]) return true;
    atomicAdd(&g_table.violations, 1u);
    return false;
}
static inline int32_t set_ranges(const void* const* base, const int64_t* bytes, int n) {
    if (n < 0 || n > kMaxRanges) return cudaErrorInvalidValue;
    Table t = {};
    t.n = n;
    for (int i = 0; i < n; ++i) {
        t.lo[i] = reinterpret_cast<unsigned long long>(base[i]);
        t.hi[i] = t.lo[i] + static_cast<unsigned long long>(bytes[i]);
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    return cudaMemcpyToSymbol(g_table, &t, sizeof(t));
}
static inline int32_t take_violations(uint32_t* out) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    Table t;
    e = cudaMemcpyFromSymbol(&t, g_table, sizeof(t));
    if (e != cudaSuccess) return e;
    *out = t.violations;
    t.violations = 0;
    return cudaMemcpyToSymbol(g_table, &t, sizeof(t));
}
}  // namespace dbg
#define CCK_DBG_OK(p, bytes) (::cck::dbg::ok((p), (bytes)))
#define CCK_DEBUG_BOUNDS_EXPORT(tag)                                                                              \
    extern "C" int32_t cck_dbg_set_ranges_##tag(const void* const* base, const int64_t* bytes, int32_t n) {      \
        return ::cck::dbg::set_ranges(base, bytes, n);                                                           \
    }                                                                                                             \
    extern "C" int32_t cck_dbg_take_violations_##tag(uint32_t* out) { return ::cck::dbg::take_violations(out); }
#else
#define CCK_DBG_OK(p, bytes) (true)
#define CCK_DEBUG_BOUNDS_EXPORT(tag)
#endif

// ---------------------------------------------------------------- 16-byte vectors
struct alignas(16) Vec16 {
    uint32_t w[4];
};

// Read-once data: non-coherent path, do not keep in L1.
__device__ __forceinline__ Vec16 ld_stream(const void* p) {
    Vec16 v;
    if (!CCK_DBG_OK(p, 16)) return Vec16{};
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}
// Re-used data (weights, tables): default caching.
__device__ __forceinline__ Vec16 ld_cached(const void* p) {
    if (!CCK_DBG_OK(p, 16)) return Vec16{};
    return *reinterpret_cast<const Vec16*>(p);
}
// Write-once data: streaming store (evict-first).
__device__ __forceinline__ void st_stream(void* p, const Vec16& v) {
    if (!CCK_DBG_OK(p, 16)) return;
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3])
                 : "memory");
}
__device__ __forceinline__ void st_stream8(void* p, uint32_t a, uint32_t b) {
    if (!CCK_DBG_OK(p, 8)) return;
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(a), "r"(b) : "memory");
}

// ---------------------------------------------------------------- storage traits
template <typename T> struct Store;

template <> struct Store<float> {
    static constexpr int kPerVec = 4;
    __device__ static __forceinline__ float get(const Vec16& v, int i) { return __uint_as_float(v.w[i]); }
    __device__ static __forceinline__ float load1(const float* p) { return CCK_DBG_OK(p, 4) ? *p : 0.0f; }
    __device__ static __forceinline__ void store1(float* p, float f) { if (CCK_DBG_OK(p, 4)) *p = f; }
    // value after one rounding to the storage type
    __device__ static __forceinline__ float round(float f) { return f; }
};

template <> struct Store<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    __device__ static __forceinline__ float get(const Vec16& v, int i) {
        const uint32_t w = v.w[i >> 1];
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    __device__ static __forceinline__ float load1(const __nv_bfloat16* p) {
        return CCK_DBG_OK(p, 2) ? __bfloat162float(*p) : 0.0f;
    }
    __device__ static __forceinline__ void store1(__nv_bfloat16* p, float f) {
        if (CCK_DBG_OK(p, 2)) *p = __float2bfloat16_rn(f);
    }
    __device__ static __forceinline__ float round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};

template <> struct Store<__half> {
    static constexpr int kPerVec = 8;
    __device__ static __forceinline__ float get(const Vec16& v, int i) {
        const uint32_t w = v.w[i >> 1];
        const __half_raw r{static_cast<unsigned short>((i & 1) ? (w >> 16) : (w & 0xffffu))};
        return __half2float(__half(r));
    }
    __device__ static __forceinline__ float load1(const __half* p) { return CCK_DBG_OK(p, 2) ? __half2float(*p) : 0.0f; }
    __device__ static __forceinline__ void store1(__half* p, float f) { if (CCK_DBG_OK(p, 2)) *p = __float2half_rn(f); }
    __device__ static __forceinline__ float round(float f) { return __half2float(__float2half_rn(f)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};

// Unpack a 16-byte vector into floats / pack floats (one rounding) into a vector.
template <typename T>
__device__ __forceinline__ void unpack(const Vec16& v, float (&f)[Store<T>::kPerVec]) {
#pragma unroll
    for (int i = 0; i < Store<T>::kPerVec; ++i) f[i] = Store<T>::get(v, i);
}
template <typename T>
__device__ __forceinline__ Vec16 pack(const float (&f)[Store<T>::kPerVec]) {
    Vec16 v;
    if constexpr (Store<T>::kPerVec == 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v.w[i] = __float_as_uint(f[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) v.w[i] = Store<T>::pack2(f[2 * i], f[2 * i + 1]);
    }
    return v;
}

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// CTA-wide reductions over THREADS threads (multiple of 32, <= 1024).  `slots`
// is a shared array of >= THREADS/32 floats.  All threads get the result; the
// trailing barrier makes `slots` reusable right away.
template <int THREADS, bool IS_MAX>
__device__ __forceinline__ float cta_reduce(float v, float* slots) {
    constexpr int kWarps = THREADS / 32;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if constexpr (kWarps == 1) return v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) slots[warp] = v;
    __syncthreads();
    float r = IS_MAX ? -INFINITY : 0.0f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) r = IS_MAX ? fmaxf(r, slots[i]) : r + slots[i];
    __syncthreads();
    return r;
}

// ---------------------------------------------------------------- SwiGLU element
// g * sigmoid(g) = g / (1 + 2^(-g*log2 e)); ex2.approx and the approximate divide are each
// good to ~2 ulp, far inside the 1e-4 / 1e-2 tolerances.
__device__ __forceinline__ float silu_f32(float g) {
    const float e = exp2f(-g * 1.4426950408889634f);
    return __fdividef(g, 1.0f + e);
}
// silu in fp32, rounded to the storage type, times `up`, rounded by the caller's store
// (the order of roundings of baselines/swiglu.py:109-112).
template <typename T>
__device__ __forceinline__ float glu1(float g, float u) {
    return Store<T>::round(silu_f32(g)) * u;
}

__host__ __device__ constexpr int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Function attributes (dynamic shared memory limit) and occupancy figures belong to a
// (function, device) pair: per-instantiation caches are indexed by the current device.
// One rotary pair, fp32: (a, b) are elements i and i + head_dim / 2 of a head, (c, s) = cos / sin of
// the position at i.  Every product and the sum / difference are rounded on their own (no fused
// multiply-add), which is the op chain of the eager baseline (baselines/rope.py:129-138) and does
// not depend on how the compiler would contract the expression in one kernel or another: the rope
// kernels and the GEMM epilogue that applies RoPE share this function and give the same bits.
__device__ __forceinline__ void rope_rotate(float a, float b, float c, float s, float& o1, float& o2) {
    o1 = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    o2 = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}

constexpr int kMaxDevices = 64;
inline int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

}  // namespace cck
