// Fused residual add + RMSNorm:
//   residual_out = x + residual;  y = residual_out * rsqrt(mean(residual_out^2) + eps) * weight
//
// Replaces the reference's csrc/kernels/rmsnorm_residual.cu:36-119, which
// walks every row twice with scalar loads.  Here a row is read from HBM exactly
// once: each thread issues all of its 16-byte loads of `x` and `residual`
// up front, keeps the summed row in registers across the reduction, and writes
// both outputs with 16-byte streaming stores.  One CTA per row; the CTA width is
// chosen so that every thread owns at most kVecPerThread vectors.
//
// Rounding follows the PyTorch baseline (baselines/rmsnorm_residual.py:130-136):
// the sum is rounded to the storage type first, the statistics are taken from
// the rounded sum in fp32, the normalised value is rounded to the storage type
// and then multiplied by `weight` in the storage type.
//
// HBM-bound: 4 tensors * rows * cols * sizeof(T) bytes per launch (+ weight once).
#include "common.cuh"

namespace cck {
namespace {

// CTA reduction for a runtime CTA width (multiple of 32).
__device__ __forceinline__ float cta_sum_dyn(float v, float* slots) {
    v = warp_sum(v);
    const int warps = blockDim.x >> 5;
    if (warps == 1) return v;
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    for (int i = 0; i < warps; ++i) r += slots[i];
    return r;
}

// kResidual = false is the plain RMSNorm used when the residual add has already been folded
// into the producing GEMM: `res` and `res_out` are not touched (2 tensors of traffic, not 4).
template <typename T, int VPT, bool kResidual>
__global__ void __launch_bounds__(1024)
rmsnorm_rowreg_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                      T* __restrict__ y, T* __restrict__ res_out, int cols, int n_vec, float eps) {
    constexpr int kPer = Store<T>::kPerVec;
    __shared__ float slots[32];
    const int64_t row_off = static_cast<int64_t>(blockIdx.x) * n_vec;
    const Vec16* x16 = reinterpret_cast<const Vec16*>(x) + row_off;
    const Vec16* r16 = reinterpret_cast<const Vec16*>(res) + row_off;
    const Vec16* w16 = reinterpret_cast<const Vec16*>(w);
    Vec16* y16 = reinterpret_cast<Vec16*>(y) + row_off;
    Vec16* o16 = reinterpret_cast<Vec16*>(res_out) + row_off;

    Vec16 xv[VPT], rv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            xv[j] = ld_stream(x16 + i);
            if constexpr (kResidual) rv[j] = ld_stream(r16 + i);
        }
    }

    // the rounded sum stays packed in the storage type (it is exact there)
    Vec16 sv[VPT];
    float sq = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            float a[kPer];
            if constexpr (kResidual) {
                float b[kPer];
                unpack<T>(xv[j], a);
                unpack<T>(rv[j], b);
#pragma unroll
                for (int e = 0; e < kPer; ++e) a[e] += b[e];
                sv[j] = pack<T>(a);
                st_stream(o16 + i, sv[j]);
            } else {
                sv[j] = xv[j];
            }
            unpack<T>(sv[j], a);
#pragma unroll
            for (int e = 0; e < kPer; ++e) sq = fmaf(a[e], a[e], sq);
        }
    }
    const float total = cta_sum_dyn(sq, slots);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(cols) + eps);

#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            float a[kPer], g[kPer];
            unpack<T>(sv[j], a);
            unpack<T>(ld_cached(w16 + i), g);
#pragma unroll
            for (int e = 0; e < kPer; ++e) a[e] = Store<T>::round(a[e] * inv) * g[e];
            st_stream(y16 + i, pack<T>(a));
        }
    }
}

// The norm of a row whose sum of squares already exists as `n_tiles` partial sums (written by the
// producing GEMM's epilogue, [n_tiles][rows]): the row is not reduced.  Each thread issues its VPT
// 16-byte loads of the row up front; meanwhile the CTA fetches the partials once into shared
// memory and every thread adds them in tile order (the same fp32 additions in every thread, so
// all hold the same factor), then scales its vectors.
constexpr int kMaxStatTiles = 1024;
template <typename T, int VPT>
__global__ void __launch_bounds__(1024)
rmsnorm_from_stats_kernel(const T* __restrict__ x, const float* __restrict__ sumsq, int n_tiles, int64_t rows,
                          const T* __restrict__ w, T* __restrict__ y, int cols, int n_vec, float eps) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t row = blockIdx.x;
    const Vec16* x16 = reinterpret_cast<const Vec16*>(x) + row * n_vec;
    const Vec16* w16 = reinterpret_cast<const Vec16*>(w);
    Vec16* y16 = reinterpret_cast<Vec16*>(y) + row * n_vec;
    Vec16 xv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) xv[j] = ld_stream(x16 + i);
    }
    // partials fetched once per CTA into shared memory, then added in tile order by every thread
    __shared__ float part[kMaxStatTiles];
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) part[t] = sumsq[static_cast<int64_t>(t) * rows + row];
    __syncthreads();
    float total = 0.0f;
    for (int t = 0; t < n_tiles; ++t) total += part[t];
    const float inv = 1.0f / sqrtf(total / static_cast<float>(cols) + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            float a[kPer], g[kPer];
            unpack<T>(xv[j], a);
            unpack<T>(ld_cached(w16 + i), g);
#pragma unroll
            for (int e = 0; e < kPer; ++e) a[e] = Store<T>::round(a[e] * inv) * g[e];
            st_stream(y16 + i, pack<T>(a));
        }
    }
}

template <typename T>
cudaError_t run_from_stats(const void* x, const float* sumsq, int64_t n_tiles, const void* w, void* y, int64_t rows,
                           int64_t cols, float eps, cudaStream_t stream) {
    constexpr int kPer = Store<T>::kPerVec;
    if (rows > 0x7fffffffLL || n_tiles <= 0 || n_tiles > kMaxStatTiles || sumsq == nullptr) return cudaErrorInvalidValue;
    const int64_t n_vec = cols / kPer;
    if (cols % kPer != 0 || n_vec > 8 * 1024 || !aligned16(x) || !aligned16(w) || !aligned16(y))
        return cudaErrorInvalidValue;
    const int vpt = n_vec <= 4 * 1024 ? 4 : 8;
    int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, vpt), 32) * 32);
    if (threads < 32) threads = 32;
    const unsigned grid = static_cast<unsigned>(rows);
    const T* xp = static_cast<const T*>(x);
    const T* wp = static_cast<const T*>(w);
    T* yp = static_cast<T*>(y);
    if (vpt == 4)
        rmsnorm_from_stats_kernel<T, 4><<<grid, threads, 0, stream>>>(xp, sumsq, static_cast<int>(n_tiles), rows, wp, yp,
                                                                      static_cast<int>(cols), static_cast<int>(n_vec), eps);
    else
        rmsnorm_from_stats_kernel<T, 8><<<grid, threads, 0, stream>>>(xp, sumsq, static_cast<int>(n_tiles), rows, wp, yp,
                                                                      static_cast<int>(cols), static_cast<int>(n_vec), eps);
    return cudaGetLastError();
}

// Any column count / alignment: scalar accesses, the row sum is written to
// residual_out in pass one and read back (by the thread that wrote it) in pass two.
template <typename T, bool kResidual>
__global__ void __launch_bounds__(256)
rmsnorm_generic_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                       T* __restrict__ y, T* res_out, int64_t cols, float eps) {
    __shared__ float slots[32];
    const int64_t off = static_cast<int64_t>(blockIdx.x) * cols;
    const T* summed = kResidual ? res_out : x;          // pass two re-reads the row from here
    float sq = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        float s = Store<T>::load1(x + off + c);
        if constexpr (kResidual) {
            s = Store<T>::round(s + Store<T>::load1(res + off + c));
            Store<T>::store1(res_out + off + c, s);
        }
        sq = fmaf(s, s, sq);
    }
    const float total = cta_sum_dyn(sq, slots);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(cols) + eps);
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float s = Store<T>::load1(summed + off + c);
        Store<T>::store1(y + off + c, Store<T>::round(s * inv) * Store<T>::load1(w + c));
    }
}

template <typename T, bool kResidual>
cudaError_t run(const void* x, const void* res, const void* w, void* y, void* res_out,
                int64_t rows, int64_t cols, float eps, cudaStream_t stream) {
    constexpr int kPer = Store<T>::kPerVec;
    const T* xp = static_cast<const T*>(x);
    const T* rp = static_cast<const T*>(res);
    const T* wp = static_cast<const T*>(w);
    T* yp = static_cast<T*>(y);
    T* op = static_cast<T*>(res_out);
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    const unsigned grid = static_cast<unsigned>(rows);
    const bool vec_ok = (cols % kPer == 0) && aligned16(x) && aligned16(w) && aligned16(y) &&
                        (!kResidual || (aligned16(res) && aligned16(res_out)));
    const int64_t n_vec = cols / kPer;
    if (vec_ok && n_vec <= 8 * 1024) {
        const int vpt = n_vec <= 4 * 1024 ? 4 : 8;
        int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, vpt), 32) * 32);
        if (threads < 32) threads = 32;
        if (vpt == 4)
            rmsnorm_rowreg_kernel<T, 4, kResidual><<<grid, threads, 0, stream>>>(
                xp, rp, wp, yp, op, static_cast<int>(cols), static_cast<int>(n_vec), eps);
        else
            rmsnorm_rowreg_kernel<T, 8, kResidual><<<grid, threads, 0, stream>>>(
                xp, rp, wp, yp, op, static_cast<int>(cols), static_cast<int>(n_vec), eps);
    } else {
        rmsnorm_generic_kernel<T, kResidual><<<grid, 256, 0, stream>>>(xp, rp, wp, yp, op, cols, eps);
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace cck

extern "C" int32_t launch_rmsnorm_residual_fwd(const void* x, const void* residual, const void* weight,
                                               void* y, void* residual_out, int64_t rows, int64_t cols,
                                               float eps, int32_t dtype, void* stream) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run<float, true>(x, residual, weight, y, residual_out, rows, cols, eps, s);
        case cck::kF16:  return cck::run<__half, true>(x, residual, weight, y, residual_out, rows, cols, eps, s);
        case cck::kBF16: return cck::run<__nv_bfloat16, true>(x, residual, weight, y, residual_out, rows, cols, eps, s);
        default:         return cudaErrorInvalidValue;
    }
}

// y = x * rsqrt(mean(x^2) + eps) * weight: the norm alone, for callers whose residual add already
// happened in the producing GEMM's epilogue (no counterpart in the reference).  Same rounding as
// launch_rmsnorm_residual_fwd with a zero residual, half the HBM traffic.
extern "C" int32_t launch_rmsnorm_fwd(const void* x, const void* weight, void* y, int64_t rows, int64_t cols,
                                      float eps, int32_t dtype, void* stream) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run<float, false>(x, nullptr, weight, y, nullptr, rows, cols, eps, s);
        case cck::kF16:  return cck::run<__half, false>(x, nullptr, weight, y, nullptr, rows, cols, eps, s);
        case cck::kBF16: return cck::run<__nv_bfloat16, false>(x, nullptr, weight, y, nullptr, rows, cols, eps, s);
        default:         return cudaErrorInvalidValue;
    }
}

// y = x * rsqrt(sum_t row_sumsq[t][row] / cols + eps) * weight: the norm of rows whose sums of squares
// the producing GEMM left as n_tiles partials per row (launch_matmul_add_bias_stats_fwd).  Same
// rounding chain as launch_rmsnorm_fwd; the statistics differ from that kernel's only in the order
// of the fp32 additions.  cols must be a multiple of the 16-byte vector width and at most 65536
// (16-bit types), pointers 16-byte aligned; otherwise cudaErrorInvalidValue.  No counterpart in the reference.
extern "C" int32_t launch_rmsnorm_from_stats_fwd(const void* x, const float* row_sumsq, int64_t n_tiles,
                                                 const void* weight, void* y, int64_t rows, int64_t cols, float eps,
                                                 int32_t dtype, void* stream) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF16:  return cck::run_from_stats<__half>(x, row_sumsq, n_tiles, weight, y, rows, cols, eps, s);
        case cck::kBF16: return cck::run_from_stats<__nv_bfloat16>(x, row_sumsq, n_tiles, weight, y, rows, cols, eps, s);
        default:         return cudaErrorInvalidValue;
    }
}

CCK_DEBUG_BOUNDS_EXPORT(rmsnorm)
