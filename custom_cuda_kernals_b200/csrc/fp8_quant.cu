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
//     FMA residual corrections (struct ExactDiv), two elements per packed fp32x2
//     instruction - 2.5 issue slots per element instead of a full division.  This file must not be compiled with
//     --use_fast_math.
//   * The row / tile is held in registers (token; small block problems) or in shared
//     memory filled by one TMA tile load (block) between the amax pass and the cast,
//     so HBM is read once.  Every load is one 16-byte vector per lane with
//     consecutive lanes on consecutive vectors (a warp reads 512 contiguous
//     bytes per instruction); the codes of one vector (8 for 16-bit inputs,
//     4 for fp32) go out as one 8- or 4-byte store, again contiguous per warp.
//
// HBM-bound: M*N*(sizeof(T) + 1) bytes per launch (+ scales).
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace cck {
namespace {

constexpr float kScaleFloor = 1e-12f;
constexpr int kMaxStatTiles = 1024;   // partial statistics per row a consumer kernel accepts
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
// whatever its last bits are.  The residuals are rounded toward -inf: an exact
// residual is unchanged by the rounding mode, except that an exact zero comes out
// as -0, and q + (-0) keeps q's own sign - so -0.0 / s stays -0.0 as IEEE
// division gives, at no extra instruction.  pair() does two quotients per
// instruction with the packed fp32x2 FMA of sm_100.
struct ExactDiv {
    float s, y;
    uint64_t neg_s2, y2;
    __device__ static __forceinline__ uint64_t pack2(float lo, float hi) {
        uint64_t r;
        asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
        return r;
    }
    __device__ static __forceinline__ ExactDiv make(float scale) {
        ExactDiv d;
        d.s = scale;
        d.y = __frcp_rn(scale);
        d.neg_s2 = pack2(-scale, -scale);
        d.y2 = pack2(d.y, d.y);
        return d;
    }
    __device__ __forceinline__ float operator()(float a) const {
        const float q0 = __fmul_rn(a, y);
        const float r0 = __fmaf_rd(-s, q0, a);
        const float q1 = __fmaf_rn(r0, y, q0);
        const float r1 = __fmaf_rd(-s, q1, a);
        return __fmaf_rn(r1, y, q1);
    }
    __device__ __forceinline__ void pair(float a, float b, float& qa, float& qb) const {
        const uint64_t ab = pack2(a, b);
        uint64_t q0, r0, q1, r1, q2;
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q0) : "l"(ab), "l"(y2));
        asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(r0) : "l"(neg_s2), "l"(q0), "l"(ab));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q1) : "l"(r0), "l"(y2), "l"(q0));
        asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(r1) : "l"(neg_s2), "l"(q1), "l"(ab));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q2) : "l"(r1), "l"(y2), "l"(q1));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(qa), "=f"(qb) : "l"(q2));
    }
};

template <bool E5M2>
__device__ __forceinline__ uint8_t quant1(float x, const ExactDiv& div) {
    return static_cast<uint8_t>(Fmt<E5M2>::cvt2(div(x), 0.0f) & 0xffu);
}

// One 16-byte vector of input -> kPer codes (8 bytes for 16-bit inputs, 4 for fp32).
template <typename T> struct Chunk {
    static constexpr int kPer = Store<T>::kPerVec;
    // largest magnitude in the vector
    __device__ static __forceinline__ float amax(const Vec16& v) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            __nv_bfloat162 m = __float2bfloat162_rn(0.0f);
#pragma unroll
            for (int i = 0; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v.w[i])));
            return fmaxf(__low2float(m), __high2float(m));
        } else if constexpr (std::is_same<T, __half>::value) {
            __half2 m = __float2half2_rn(0.0f);
#pragma unroll
            for (int i = 0; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __half2*>(&v.w[i])));
            return fmaxf(__low2float(m), __high2float(m));
        } else {
            float m = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) m = fmaxf(m, fabsf(__uint_as_float(v.w[i])));
            return m;
        }
    }
    template <bool E5M2>
    __device__ static __forceinline__ void quantise_store(const Vec16& v, const ExactDiv& div, uint8_t* dst) {
        float f[kPer];
#pragma unroll
        for (int e = 0; e < kPer; e += 2) div.pair(Store<T>::get(v, e), Store<T>::get(v, e + 1), f[e], f[e + 1]);
        const uint32_t w0 = Fmt<E5M2>::cvt2(f[0], f[1]) | (Fmt<E5M2>::cvt2(f[2], f[3]) << 16);
        if constexpr (kPer == 8) {
            const uint32_t w1 = Fmt<E5M2>::cvt2(f[4], f[5]) | (Fmt<E5M2>::cvt2(f[6], f[7]) << 16);
            st_stream8(dst, w0, w1);
        } else {
            asm volatile("st.global.cs.u32 [%0], %1;" :: "l"(dst), "r"(w0) : "memory");
        }
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
// One CTA per row; thread t owns vectors t, t + blockDim, ... (VPT of them, in registers).
template <typename T, bool E5M2, int VPT>
__global__ void __launch_bounds__(1024)
fp8_token_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                 int64_t n, int n_vec) {
    constexpr int kPer = Store<T>::kPerVec;
    __shared__ float slots[32];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * n;
    uint8_t* cr = codes + row * n;
    Vec16 v[VPT];
    const bool full = static_cast<int>(blockDim.x) * VPT == n_vec;   // no ragged last pass (the usual case)
    float m = 0.0f;
    if (full) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) v[j] = ld_stream(xr + static_cast<int64_t>(threadIdx.x + j * blockDim.x) * kPer);
#pragma unroll
        for (int j = 0; j < VPT; ++j) m = fmaxf(m, Chunk<T>::amax(v[j]));
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_vec) v[j] = ld_stream(xr + static_cast<int64_t>(i) * kPer);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (static_cast<int>(threadIdx.x + j * blockDim.x) < n_vec) m = fmaxf(m, Chunk<T>::amax(v[j]));
    }
    const float sc = scale_of<E5M2>(cta_max_dyn(m, slots));
    if (threadIdx.x == 0) scale[row] = sc;
    const ExactDiv div = ExactDiv::make(sc);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (full || i < n_vec) Chunk<T>::template quantise_store<E5M2>(v[j], div, cr + static_cast<int64_t>(i) * kPer);
    }
}

// The same quantiser for rows whose largest magnitude already exists as `n_tiles` partial maxima
// per row ([n_tiles][rows], written by the producing GEMM's epilogue): the row itself is not
// scanned, the threads share the loads of the partials and one CTA-wide maximum finishes.  A
// maximum does not depend on the order it is taken in, so codes and scales are bit for bit those
// of fp8_token_kernel.
template <typename T, bool E5M2, int VPT>
__global__ void __launch_bounds__(1024)
fp8_token_from_amax_kernel(const T* __restrict__ x, const float* __restrict__ amax, int n_tiles, int64_t rows,
                           uint8_t* __restrict__ codes, float* __restrict__ scale, int64_t n, int n_vec) {
    constexpr int kPer = Store<T>::kPerVec;
    __shared__ float slots[32];
    const int64_t row = blockIdx.x;
    const T* xr = x + row * n;
    uint8_t* cr = codes + row * n;
    Vec16 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) v[j] = ld_stream(xr + static_cast<int64_t>(i) * kPer);
    }
    // the row's partial maxima, spread over the threads (one load each where n_tiles <= CTA width)
    float m = 0.0f;
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) m = fmaxf(m, amax[static_cast<int64_t>(t) * rows + row]);
    const float sc = scale_of<E5M2>(cta_max_dyn(m, slots));
    if (threadIdx.x == 0) scale[row] = sc;
    const ExactDiv div = ExactDiv::make(sc);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) Chunk<T>::template quantise_store<E5M2>(v[j], div, cr + static_cast<int64_t>(i) * kPer);
    }
}

// packed product of two pairs of 16-bit values, each rounded once to the storage type
template <typename T>
__device__ __forceinline__ uint32_t mul2_16(uint32_t a, uint32_t b) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    } else {
        const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
}

// RMSNorm and per-token quantisation in one pass: codes, scale = fp8_quant(rmsnorm(x, w), "token"),
// bit for bit, without the normalised row ever going to HBM (it is read 2 bytes per element and
// written 1; the two-kernel chain moves 2 + 2 + 2 + 1).  The row lives in registers from the load to
// the store; the sum of squares is reduced exactly as rmsnorm_rowreg_kernel reduces it (same
// thread-to-vector map, same fp32 additions), or - when the producing GEMM left partial sums of
// squares ([n_tiles][rows]) - taken from those in tile order, as launch_rmsnorm_from_stats_fwd does.
// `y`, when not null, also receives the normalised row in the storage type.
template <typename T, bool E5M2, int VPT>
__global__ void __launch_bounds__(1024)
rmsnorm_fp8_token_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ sumsq, int n_tiles,
                         int64_t rows, T* __restrict__ y, uint8_t* __restrict__ codes, float* __restrict__ scale,
                         int cols, int n_vec, float eps) {
    constexpr int kPer = Store<T>::kPerVec;
    __shared__ float slots[32];
    const int64_t row = blockIdx.x;
    const Vec16* x16 = reinterpret_cast<const Vec16*>(x) + row * n_vec;
    const Vec16* w16 = reinterpret_cast<const Vec16*>(w);
    Vec16 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) v[j] = ld_stream(x16 + i);
    }
    float total;
    if (sumsq != nullptr) {
        // partials fetched once per CTA into shared memory, then added in tile order by every thread
        __shared__ float part[kMaxStatTiles];
        for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) part[t] = sumsq[static_cast<int64_t>(t) * rows + row];
        __syncthreads();
        total = 0.0f;
        for (int t = 0; t < n_tiles; ++t) total += part[t];
    } else {
        float sq = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (static_cast<int>(threadIdx.x + j * blockDim.x) < n_vec) {
                float a[kPer];
                unpack<T>(v[j], a);
#pragma unroll
                for (int e = 0; e < kPer; ++e) sq = fmaf(a[e], a[e], sq);
            }
        }
        sq = warp_sum(sq);                              // the reduction of rmsnorm_rowreg_kernel
        const int warps = blockDim.x >> 5;
        if (warps == 1) {
            total = sq;
        } else {
            if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = sq;
            __syncthreads();
            total = 0.0f;
            for (int i = 0; i < warps; ++i) total += slots[i];
            __syncthreads();                            // slots are reused by the maximum below
        }
    }
    const float inv = 1.0f / sqrtf(total / static_cast<float>(cols) + eps);
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            // round(x * inv) to the storage type, times weight in the storage type: two elements per
            // instruction - one packed conversion, one packed multiply (the product of two 16-bit
            // values is exact in fp32, so a packed multiply rounds exactly as multiply-then-convert)
            const Vec16 g = ld_cached(w16 + i);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t n2 = Store<T>::pack2(Store<T>::get(v[j], 2 * q) * inv, Store<T>::get(v[j], 2 * q + 1) * inv);
                v[j].w[q] = mul2_16<T>(n2, g.w[q]);
            }
            if (y != nullptr) st_stream(reinterpret_cast<Vec16*>(y) + row * n_vec + i, v[j]);
            m = fmaxf(m, Chunk<T>::amax(v[j]));
        }
    }
    const float sc = scale_of<E5M2>(cta_max_dyn(m, slots));
    if (threadIdx.x == 0) scale[row] = sc;
    const ExactDiv div = ExactDiv::make(sc);
    uint8_t* cr = codes + row * cols;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) Chunk<T>::template quantise_store<E5M2>(v[j], div, cr + static_cast<int64_t>(i) * kPer);
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
    const ExactDiv div = ExactDiv::make(sc);
    for (int64_t c = threadIdx.x; c < n; c += blockDim.x)
        codes[row * n + c] = quant1<E5M2>(Store<T>::load1(xr + c), div);
}

// ------------------------------------------------------------------ block granularity
// One CTA of 512 threads per 128x128 tile; a tile row is 128/kPer vectors, so a warp
// reads whole 256-byte (16-bit) or 512-byte (fp32) row segments; 4 (8) vectors per thread.
constexpr int kBlockThreads = 512;
template <typename T, bool E5M2>
__global__ void __launch_bounds__(kBlockThreads, sizeof(T) == 4 ? 2 : 3)
fp8_block_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes, float* __restrict__ scale,
                 int64_t m, int64_t n) {
    constexpr int kPer = Store<T>::kPerVec;
    constexpr int kVecPerRow = kTile / kPer;                        // 16 or 32
    constexpr int kVpt = kTile * kVecPerRow / kBlockThreads;        // 4 or 8
    __shared__ float slots[32];
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kTile, c0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const bool interior = r0 + kTile <= m && c0 + kTile <= n;      // no edge predicates needed
    Vec16 v[kVpt];
    int64_t off[kVpt];
    bool live[kVpt];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < kVpt; ++j) {
        const int id = threadIdx.x + j * kBlockThreads;
        const int64_t r = r0 + id / kVecPerRow, c = c0 + (id % kVecPerRow) * kPer;
        off[j] = r * n + c;
        live[j] = interior || (r < m && c < n);                     // n % kPer == 0 on this path
        if (live[j]) v[j] = ld_stream(x + off[j]);
    }
#pragma unroll
    for (int j = 0; j < kVpt; ++j)
        if (live[j]) mx = fmaxf(mx, Chunk<T>::amax(v[j]));
    const float sc = scale_of<E5M2>(cta_max_dyn(mx, slots));
    if (threadIdx.x == 0) scale[static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x] = sc;
    const ExactDiv div = ExactDiv::make(sc);
#pragma unroll
    for (int j = 0; j < kVpt; ++j)
        if (live[j]) Chunk<T>::template quantise_store<E5M2>(v[j], div, codes + off[j]);
}

// Same tile, staged by TMA: one thread issues a single 2-D tile load of the whole 128x128 tile
// (32 KB for 16-bit inputs, 64 KB for fp32) into shared memory, so a 128-thread CTA keeps a
// full tile in flight and 3-6 CTAs per SM keep 190 KB in flight without spending registers on
// it; the tile is then read from shared memory twice (amax pass, cast pass) with 16-byte
// conflict-free accesses.  TMA zero-fills the part of an edge tile that lies outside the
// matrix, which cannot change a maximum of magnitudes.  The wait is bounded; if it runs out
// the CTA sets bit 1 of the status word and writes nothing.
constexpr int kTmaThreads = 256;   // measured on B200, bf16 [8192,4096]: 128 threads 18.2 us, 256 17.4 us, 512 20.1 us
template <typename T, bool E5M2>
__global__ void __launch_bounds__(kTmaThreads)
fp8_block_tma_kernel(const __grid_constant__ CUtensorMap map, uint8_t* __restrict__ codes,
                     float* __restrict__ scale, int64_t m, int64_t n, unsigned int* status) {
    constexpr int kPer = Store<T>::kPerVec;
    constexpr int kVecPerRow = kTile / kPer;
    constexpr int kVecs = kTile * kVecPerRow;               // 2048 or 4096 vectors per tile
    extern __shared__ __align__(128) uint8_t tile[];
    __shared__ __align__(8) uint64_t bar_storage;
    __shared__ float slots[32];
    __shared__ int abort_flag;
    const uint32_t bar = ptx::smem_addr(&bar_storage);
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kTile, c0 = static_cast<int64_t>(blockIdx.x) * kTile;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(bar, 1);
        ptx::fence_barrier_init();
        ptx::mbar_arrive_expect_tx(bar, kTile * kTile * static_cast<uint32_t>(sizeof(T)));
        // c0 is a multiple of 128 elements: the copy starts on a 16-byte boundary
        ptx::tma_load_2d(ptx::smem_addr(tile), &map, bar, static_cast<int32_t>(c0), static_cast<int32_t>(r0));
    }
    __syncthreads();
    const bool ok = ptx::mbar_wait(bar, 0, &abort_flag, status);
    if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicOr(status, 2u);
        return;
    }
    const Vec16* t16 = reinterpret_cast<const Vec16*>(tile);
    float mx = 0.0f;
#pragma unroll 4
    for (int id = threadIdx.x; id < kVecs; id += kTmaThreads) mx = fmaxf(mx, Chunk<T>::amax(t16[id]));
    const float sc = scale_of<E5M2>(cta_max_dyn(mx, slots));
    if (threadIdx.x == 0) scale[static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x] = sc;
    const ExactDiv div = ExactDiv::make(sc);
    const bool interior = r0 + kTile <= m && c0 + kTile <= n;
#pragma unroll 2
    for (int id = threadIdx.x; id < kVecs; id += kTmaThreads) {
        const int64_t r = r0 + id / kVecPerRow, c = c0 + (id % kVecPerRow) * kPer;
        if (interior || (r < m && c < n)) Chunk<T>::template quantise_store<E5M2>(t16[id], div, codes + r * n + c);
    }
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
    const ExactDiv div = ExactDiv::make(sc);
    for (int id = threadIdx.x; id < kTile * kTile; id += 256) {
        const int64_t r = r0 + (id >> 7), c = c0 + (id & 127);
        if (r < m && c < n) codes[r * n + c] = quant1<E5M2>(Store<T>::load1(x + r * n + c), div);
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
        int64_t i = tid;
        for (; i + 3 * stride < n_vec; i += 4 * stride) {           // four loads in flight per thread
            Vec16 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = ld_cached(x + (i + j * stride) * kPer);   // default policy: the cast pass re-reads from L2
#pragma unroll
            for (int j = 0; j < 4; ++j) m = fmaxf(m, Chunk<T>::amax(v[j]));
        }
        for (; i < n_vec; i += stride) m = fmaxf(m, Chunk<T>::amax(ld_cached(x + i * kPer)));
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
    constexpr int kPer = Store<T>::kPerVec;
    const float sc = scale_of<E5M2>(__int_as_float(*amax_bits));
    const ExactDiv div = ExactDiv::make(sc);
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    if (tid == 0) scale[0] = sc;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t n_vec = total / kPer;
        int64_t i = tid;
        for (; i + 3 * stride < n_vec; i += 4 * stride) {
            Vec16 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = ld_stream(x + (i + j * stride) * kPer);
#pragma unroll
            for (int j = 0; j < 4; ++j) Chunk<T>::template quantise_store<E5M2>(v[j], div, codes + (i + j * stride) * kPer);
        }
        for (; i < n_vec; i += stride)
            Chunk<T>::template quantise_store<E5M2>(ld_stream(x + i * kPer), div, codes + i * kPer);
        done = n_vec * kPer;
    }
    for (int64_t i = done + tid; i < total; i += stride) codes[i] = quant1<E5M2>(Store<T>::load1(x + i), div);
}

// ------------------------------------------------------------------ host dispatch
template <typename T, bool E5M2>
cudaError_t run_token(const void* x, uint8_t* codes, float* scale, int64_t m, int64_t n, cudaStream_t s) {
    if (m > 0x7fffffffLL) return cudaErrorInvalidValue;
    const T* xp = static_cast<const T*>(x);
    const unsigned grid = static_cast<unsigned>(m);
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t n_vec = n / kPer;
    // codes of one vector are stored with one kPer-byte store: row starts must be kPer-byte aligned
    if (n % kPer == 0 && aligned16(x) && (reinterpret_cast<uintptr_t>(codes) % kPer) == 0 && n_vec <= 8 * 1024) {
        const int vpt = n_vec <= 4 * 1024 ? 4 : 8;
        int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, vpt), 32) * 32);
        if (threads < 32) threads = 32;
        const int nv = static_cast<int>(n_vec);
        if (vpt == 4) fp8_token_kernel<T, E5M2, 4><<<grid, threads, 0, s>>>(xp, codes, scale, n, nv);
        else fp8_token_kernel<T, E5M2, 8><<<grid, threads, 0, s>>>(xp, codes, scale, n, nv);
    } else {
        fp8_token_generic_kernel<T, E5M2><<<grid, 256, 0, s>>>(xp, codes, scale, n);
    }
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_rmsnorm_fp8(const void* x, const void* w, const float* sumsq, int64_t n_tiles, void* y, uint8_t* codes,
                            float* scale, int64_t rows, int64_t cols, float eps, cudaStream_t s) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t n_vec = cols / kPer;
    if (rows > 0x7fffffffLL || cols % kPer != 0 || n_vec > 8 * 1024 || !aligned16(x) || !aligned16(w) ||
        (y != nullptr && !aligned16(y)) || (reinterpret_cast<uintptr_t>(codes) % kPer) != 0 ||
        (sumsq != nullptr && (n_tiles <= 0 || n_tiles > kMaxStatTiles)))
        return cudaErrorInvalidValue;
    const int vpt = n_vec <= 4 * 1024 ? 4 : 8;         // the CTA shape of rmsnorm_rowreg_kernel
    int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, vpt), 32) * 32);
    if (threads < 32) threads = 32;
    const unsigned grid = static_cast<unsigned>(rows);
    const int nt = static_cast<int>(n_tiles), nc = static_cast<int>(cols), nv = static_cast<int>(n_vec);
    if (vpt == 4)
        rmsnorm_fp8_token_kernel<T, E5M2, 4><<<grid, threads, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(w), sumsq,
                                                                      nt, rows, static_cast<T*>(y), codes, scale, nc, nv, eps);
    else
        rmsnorm_fp8_token_kernel<T, E5M2, 8><<<grid, threads, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(w), sumsq,
                                                                      nt, rows, static_cast<T*>(y), codes, scale, nc, nv, eps);
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_token_from_amax(const void* x, const float* amax, int64_t n_tiles, uint8_t* codes, float* scale,
                                int64_t m, int64_t n, cudaStream_t s) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t n_vec = n / kPer;
    if (m > 0x7fffffffLL || n_tiles <= 0 || n_tiles > 4096 || amax == nullptr || n % kPer != 0 || !aligned16(x) ||
        (reinterpret_cast<uintptr_t>(codes) % kPer) != 0 || n_vec > 8 * 1024)
        return cudaErrorInvalidValue;
    const int vpt = n_vec <= 4 * 1024 ? 4 : 8;
    int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, vpt), 32) * 32);
    if (threads < 32) threads = 32;
    const unsigned grid = static_cast<unsigned>(m);
    const T* xp = static_cast<const T*>(x);
    const int nt = static_cast<int>(n_tiles), nv = static_cast<int>(n_vec);
    if (vpt == 4) fp8_token_from_amax_kernel<T, E5M2, 4><<<grid, threads, 0, s>>>(xp, amax, nt, m, codes, scale, n, nv);
    else fp8_token_from_amax_kernel<T, E5M2, 8><<<grid, threads, 0, s>>>(xp, amax, nt, m, codes, scale, n, nv);
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_block(const void* x, uint8_t* codes, float* scale, int64_t m, int64_t n, cudaStream_t s) {
    const int64_t gx = ceil_div64(n, kTile), gy = ceil_div64(m, kTile);
    if (gy > 65535 || gx > 0x7fffffffLL) return cudaErrorInvalidValue;
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    const T* xp = static_cast<const T*>(x);
    const bool vec_ok = n % Store<T>::kPerVec == 0 && aligned16(x) && (reinterpret_cast<uintptr_t>(codes) % 8) == 0;
    // TMA needs 16-byte aligned rows; tiny matrices are not worth a tensor map
    if (vec_ok && (n * sizeof(T)) % 16 == 0 && m * n >= (1 << 16) && m < (1LL << 31) && n < (1LL << 31) &&
        tc::encode_fn() != nullptr) {
        constexpr bool is32 = sizeof(T) == 4;
        const CUtensorMapDataType dt = is32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : (std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                              : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
        CUtensorMap map;
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * sizeof(T)};
        const cuuint32_t box[2] = {kTile, kTile};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = tc::encode_fn()(&map, dt, 2, const_cast<T*>(xp), dims, strides, box, estr,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        unsigned int* st = tc::status_word();
        if (r == CUDA_SUCCESS && st != nullptr) {
            constexpr int kSmem = kTile * kTile * static_cast<int>(sizeof(T));
            auto kern = fp8_block_tma_kernel<T, E5M2>;
            static bool configured[kMaxDevices] = {};
            const int slot = current_device_slot();
            if (slot < 0) return cudaErrorInvalidDevice;
            if (!configured[slot]) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
                if (e != cudaSuccess) return e;
                configured[slot] = true;
            }
            kern<<<grid, kTmaThreads, kSmem, s>>>(map, codes, scale, m, n, st);
            return cudaGetLastError();
        }
    }
    if (vec_ok)
        fp8_block_kernel<T, E5M2><<<grid, kBlockThreads, 0, s>>>(xp, codes, scale, m, n);
    else
        fp8_block_generic_kernel<T, E5M2><<<grid, 256, 0, s>>>(xp, codes, scale, m, n);
    return cudaGetLastError();
}

template <typename T, bool E5M2>
cudaError_t run_tensor(const void* x, uint8_t* codes, float* scale, int32_t* amax_bits, int64_t m, int64_t n,
                       cudaStream_t s) {
    const T* xp = static_cast<const T*>(x);
    const int64_t total = m * n;
    const bool vec_ok = aligned16(x) && (reinterpret_cast<uintptr_t>(codes) % 8) == 0;
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

// Per-token quantisation of a matrix whose row maxima the producing GEMM left as n_tiles partial
// maxima per row (launch_matmul_add_bias_stats_fwd: row_amax [n_tiles, m]).  Codes and scales are
// bit for bit those of launch_fp8_quant_token_fwd.  16-bit inputs, n a multiple of 8, 16-byte
// aligned x, 8-byte aligned codes; otherwise cudaErrorInvalidValue.  No counterpart in the reference.
extern "C" int32_t launch_fp8_quant_token_from_amax_fwd(const void* x, const float* row_amax, int64_t n_tiles,
                                                        uint8_t* x_fp8, float* scale, int64_t m, int64_t n,
                                                        int32_t dtype, int32_t fp8_format, void* stream) {
    using namespace cck;
    if (m <= 0 || n <= 0) return cudaSuccess;
    if (fp8_format != kF8E4M3 && fp8_format != kF8E5M2) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool e5 = fp8_format == kF8E5M2;
    switch (dtype) {
        case kF16:
            return e5 ? run_token_from_amax<__half, true>(x, row_amax, n_tiles, x_fp8, scale, m, n, s)
                      : run_token_from_amax<__half, false>(x, row_amax, n_tiles, x_fp8, scale, m, n, s);
        case kBF16:
            return e5 ? run_token_from_amax<__nv_bfloat16, true>(x, row_amax, n_tiles, x_fp8, scale, m, n, s)
                      : run_token_from_amax<__nv_bfloat16, false>(x, row_amax, n_tiles, x_fp8, scale, m, n, s);
        default:
            return cudaErrorInvalidValue;
    }
}

// x_fp8, scale = fp8_quant(rmsnorm(x, weight, eps), "token"), bit for bit, in one pass over x: the
// normalised row stays in registers between the norm and the quantiser (3 bytes of HBM traffic per
// element instead of 7).  row_sumsq, when not NULL, holds n_tiles partial sums of squares per row
// ([n_tiles, rows], from launch_matmul_add_bias_stats_fwd) and replaces the row reduction (the result
// then equals fp8_quant(rmsnorm_from_stats(...))).  y, when not NULL, also receives the normalised
// rows.  float16/bfloat16, cols a multiple of 8 and at most 65536, 16-byte aligned x, weight and y,
// 8-byte aligned x_fp8; otherwise cudaErrorInvalidValue.  No counterpart in the reference.
extern "C" int32_t launch_rmsnorm_fp8_quant_token_fwd(const void* x, const void* weight, const float* row_sumsq,
                                                      int64_t n_tiles, void* y, uint8_t* x_fp8, float* scale,
                                                      int64_t rows, int64_t cols, float eps, int32_t dtype,
                                                      int32_t fp8_format, void* stream) {
    using namespace cck;
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    if (fp8_format != kF8E4M3 && fp8_format != kF8E5M2) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool e5 = fp8_format == kF8E5M2;
    switch (dtype) {
        case kF16:
            return e5 ? run_rmsnorm_fp8<__half, true>(x, weight, row_sumsq, n_tiles, y, x_fp8, scale, rows, cols, eps, s)
                      : run_rmsnorm_fp8<__half, false>(x, weight, row_sumsq, n_tiles, y, x_fp8, scale, rows, cols, eps, s);
        case kBF16:
            return e5 ? run_rmsnorm_fp8<__nv_bfloat16, true>(x, weight, row_sumsq, n_tiles, y, x_fp8, scale, rows, cols, eps, s)
                      : run_rmsnorm_fp8<__nv_bfloat16, false>(x, weight, row_sumsq, n_tiles, y, x_fp8, scale, rows, cols, eps, s);
        default:
            return cudaErrorInvalidValue;
    }
}
