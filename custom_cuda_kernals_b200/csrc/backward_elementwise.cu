// Gradients of the two elementwise ops of the decoder block that have one (RoPE's is RoPE
// itself with the sine negated, so it needs no kernel).  The reference is forward-only
// (custom_cuda/kernels/linear_cross_entropy.py:11-18 names autograd as the missing piece);
// these follow the same conventions as the forward kernels: fp32 arithmetic, one rounding on
// store, 16-byte streaming accesses, every input read from HBM once.
//
//   swiglu:   y = silu(g) * u        d_g = dy * u * s * (1 + g * (1 - s)),  d_u = dy * silu(g),  s = sigmoid(g)
//             HBM-bound: 5 tensors * n * sizeof(T).
//   rmsnorm:  ro = x + r;  y = ro * rstd * w,  rstd = rsqrt(mean(ro^2) + eps)
//             with gy = dy * w:   d_ro = rstd * gy - ro * rstd^3 * mean(gy * ro)  (+ the gradient
//             that arrives through residual_out);  d_x = d_r = d_ro;  d_w = sum_rows dy * ro * rstd.
//             HBM-bound: 3 (4 with the residual_out gradient) tensors * rows * cols * sizeof(T).
#include "common.cuh"

namespace cck {
namespace {

// ------------------------------------------------------------------ swiglu
constexpr int kSwThreads = 256;
constexpr int kSwUnroll = 2;

__device__ __forceinline__ void swiglu_grad1(float g, float u, float dy, float& dg, float& du) {
    const float s = __fdividef(1.0f, 1.0f + exp2f(-g * 1.4426950408889634f));
    const float silu = g * s;
    du = dy * silu;
    dg = dy * u * (s + silu * (1.0f - s));
}

template <typename T>
__global__ void __launch_bounds__(kSwThreads)
swiglu_bwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dy,
                  T* __restrict__ dgate, T* __restrict__ dup, int64_t n_vec, int64_t n) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (kSwThreads * kSwUnroll) + threadIdx.x;
    const Vec16* g16 = reinterpret_cast<const Vec16*>(gate);
    const Vec16* u16 = reinterpret_cast<const Vec16*>(up);
    const Vec16* d16 = reinterpret_cast<const Vec16*>(dy);
    Vec16 gv[kSwUnroll], uv[kSwUnroll], dv[kSwUnroll];
#pragma unroll
    for (int j = 0; j < kSwUnroll; ++j) {
        const int64_t i = base + static_cast<int64_t>(j) * kSwThreads;
        if (i < n_vec) {
            gv[j] = ld_stream(g16 + i);
            uv[j] = ld_stream(u16 + i);
            dv[j] = ld_stream(d16 + i);
        }
    }
#pragma unroll
    for (int j = 0; j < kSwUnroll; ++j) {
        const int64_t i = base + static_cast<int64_t>(j) * kSwThreads;
        if (i < n_vec) {
            float g[kPer], u[kPer], d[kPer], og[kPer], ou[kPer];
            unpack<T>(gv[j], g);
            unpack<T>(uv[j], u);
            unpack<T>(dv[j], d);
#pragma unroll
            for (int e = 0; e < kPer; ++e) swiglu_grad1(g[e], u[e], d[e], og[e], ou[e]);
            st_stream(reinterpret_cast<Vec16*>(dgate) + i, pack<T>(og));
            st_stream(reinterpret_cast<Vec16*>(dup) + i, pack<T>(ou));
        }
    }
    if (blockIdx.x == gridDim.x - 1) {                 // ragged tail, fewer than one vector
        const int64_t t = n_vec * kPer + threadIdx.x;
        if (t < n) {
            float og, ou;
            swiglu_grad1(Store<T>::load1(gate + t), Store<T>::load1(up + t), Store<T>::load1(dy + t), og, ou);
            Store<T>::store1(dgate + t, og);
            Store<T>::store1(dup + t, ou);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kSwThreads)
swiglu_bwd_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dy,
                         T* __restrict__ dgate, T* __restrict__ dup, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kSwThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kSwThreads + threadIdx.x; i < n; i += stride) {
        float og, ou;
        swiglu_grad1(Store<T>::load1(gate + i), Store<T>::load1(up + i), Store<T>::load1(dy + i), og, ou);
        Store<T>::store1(dgate + i, og);
        Store<T>::store1(dup + i, ou);
    }
}

template <typename T>
cudaError_t run_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, int64_t n,
                           cudaStream_t s) {
    const T* g = static_cast<const T*>(gate);
    const T* u = static_cast<const T*>(up);
    const T* d = static_cast<const T*>(dy);
    T* og = static_cast<T*>(dgate);
    T* ou = static_cast<T*>(dup);
    if (aligned16(gate) && aligned16(up) && aligned16(dy) && aligned16(dgate) && aligned16(dup)) {
        const int64_t n_vec = n / Store<T>::kPerVec;
        const int64_t ctas = ceil_div64(n_vec, kSwThreads * kSwUnroll);
        swiglu_bwd_kernel<T><<<static_cast<unsigned>(ctas > 0 ? ctas : 1), kSwThreads, 0, s>>>(g, u, d, og, ou, n_vec, n);
    } else {
        const int64_t ctas = ceil_div64(n, kSwThreads);
        const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
        swiglu_bwd_scalar_kernel<T><<<static_cast<unsigned>(ctas < cap ? ctas : cap), kSwThreads, 0, s>>>(g, u, d, og, ou, n);
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------ rmsnorm + residual
constexpr int kRnVpt = 4;          // 16-byte vectors of each input a thread keeps in registers
constexpr int kRnMaxThreads = 256;
constexpr int kRnCtasPerSm = 8;   // upper bound on resident CTAs per SM (sizes the d_weight partials)

// Persistent CTAs, each walking rows blockIdx.x, blockIdx.x + gridDim.x, ...  A thread owns the
// same columns in every row.  Its slice of `weight` (as fp32) and of the CTA's partial d_weight
// live in shared memory as float4 planes [kPer / 4][n_vec] - plane q holds elements 4q..4q+3 of
// every vector, so a warp's 16-byte accesses are contiguous and only the owning thread touches
// a slot (no atomics, no barriers) - which keeps the register budget for the row itself: the
// dy / ro / d_ro vectors stay in registers between the reduction and the store.  Every CTA
// ends by writing its d_weight partial to dw_part[blockIdx.x][cols]; rmsnorm_dw_reduce_kernel
// sums the partials.
template <typename T, bool kHasDro>
__global__ void __launch_bounds__(kRnMaxThreads)
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ dro_in, const T* __restrict__ ro,
                   const T* __restrict__ w, T* __restrict__ dx, float* __restrict__ dw_part, int64_t rows,
                   int cols, int n_vec, float eps) {
    constexpr int kPer = Store<T>::kPerVec;
    constexpr int kPlanes = kPer / 4;
    extern __shared__ __align__(16) float4 planes[];
    float4* w4 = planes;                               // [kPlanes][n_vec]
    float4* dw4 = planes + kPlanes * n_vec;            // [kPlanes][n_vec]
    __shared__ float2 slots[32];
#pragma unroll
    for (int j = 0; j < kRnVpt; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
            float wf[kPer];
            unpack<T>(ld_cached(reinterpret_cast<const Vec16*>(w) + i), wf);
#pragma unroll
            for (int q = 0; q < kPlanes; ++q) {
                w4[q * n_vec + i] = make_float4(wf[4 * q], wf[4 * q + 1], wf[4 * q + 2], wf[4 * q + 3]);
                dw4[q * n_vec + i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    // software pipeline over rows: the next row's vectors are requested before this row is
    // reduced, so a CTA always has one row of loads in flight
    // (the residual_out gradient is only needed at the store, so it is requested at the top of
    // its own row's iteration and costs no second register set)
    Vec16 dv[kRnVpt], rv[kRnVpt], iv[kRnVpt], dn[kRnVpt], rn[kRnVpt];
    auto request = [&](int64_t row, Vec16 (&d)[kRnVpt], Vec16 (&r)[kRnVpt]) {
        const int64_t o = row * n_vec;
#pragma unroll
        for (int j = 0; j < kRnVpt; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_vec && row < rows) {
                d[j] = ld_stream(reinterpret_cast<const Vec16*>(dy) + o + i);
                r[j] = ld_stream(reinterpret_cast<const Vec16*>(ro) + o + i);
            }
        }
    };
    request(blockIdx.x, dv, rv);
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t off = row * n_vec;
        request(row + gridDim.x, dn, rn);
        if constexpr (kHasDro) {
#pragma unroll
            for (int j = 0; j < kRnVpt; ++j) {
                const int i = threadIdx.x + j * blockDim.x;
                if (i < n_vec) iv[j] = ld_stream(reinterpret_cast<const Vec16*>(dro_in) + off + i);
            }
        }
        float sq = 0.0f, gr = 0.0f;                    // sum ro^2, sum (dy * w) * ro
#pragma unroll
        for (int j = 0; j < kRnVpt; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_vec) {
                float d[kPer], r[kPer];
                unpack<T>(dv[j], d);
                unpack<T>(rv[j], r);
#pragma unroll
                for (int q = 0; q < kPlanes; ++q) {
                    const float4 wq = w4[q * n_vec + i];
                    const float wf[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sq = fmaf(r[4 * q + e], r[4 * q + e], sq);
                        gr = fmaf(d[4 * q + e] * wf[e], r[4 * q + e], gr);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            gr += __shfl_xor_sync(0xffffffffu, gr, o);
        }
        if (warps > 1) {
            if (lane == 0) slots[warp] = make_float2(sq, gr);
            __syncthreads();
            sq = 0.0f;
            gr = 0.0f;
            for (int i = 0; i < warps; ++i) {
                sq += slots[i].x;
                gr += slots[i].y;
            }
            __syncthreads();                           // slots are reused by the next row
        }
        const float rstd = 1.0f / sqrtf(sq * inv_cols + eps);
        const float coef = rstd * rstd * rstd * gr * inv_cols;
#pragma unroll
        for (int j = 0; j < kRnVpt; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n_vec) {
                float d[kPer], r[kPer], o[kPer];
                unpack<T>(dv[j], d);
                unpack<T>(rv[j], r);
#pragma unroll
                for (int q = 0; q < kPlanes; ++q) {
                    const float4 wq = w4[q * n_vec + i];
                    float4 acc = dw4[q * n_vec + i];
                    const float wf[4] = {wq.x, wq.y, wq.z, wq.w};
                    float af[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        o[4 * q + e] = fmaf(rstd * wf[e], d[4 * q + e], -coef * r[4 * q + e]);
                        af[e] = fmaf(d[4 * q + e] * rstd, r[4 * q + e], af[e]);
                    }
                    dw4[q * n_vec + i] = make_float4(af[0], af[1], af[2], af[3]);
                }
                if constexpr (kHasDro) {
                    float a[kPer];
                    unpack<T>(iv[j], a);
#pragma unroll
                    for (int e = 0; e < kPer; ++e) o[e] += a[e];
                }
                st_stream(reinterpret_cast<Vec16*>(dx) + off + i, pack<T>(o));
            }
        }
#pragma unroll
        for (int j = 0; j < kRnVpt; ++j) {
            dv[j] = dn[j];
            rv[j] = rn[j];
        }
    }
    float* part = dw_part + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
    for (int j = 0; j < kRnVpt; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n_vec) {
#pragma unroll
            for (int q = 0; q < kPlanes; ++q)
                *reinterpret_cast<float4*>(part + i * kPer + 4 * q) = dw4[q * n_vec + i];
        }
    }
}

// d_weight[c] = sum over the CTAs' partials.  A CTA owns 32 columns; its 8 warps take every
// eighth partial each (coalesced 128-byte reads, 8 independent loads in flight per thread)
// and meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ dw_part, int parts, int cols, T* __restrict__ dw) {
    __shared__ float partial[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float acc = 0.0f;
    if (c < cols) {
        int p = warp;
        for (; p + 56 < parts; p += 64) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = dw_part[static_cast<int64_t>(p + 8 * u) * cols + c];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += v[u];
        }
        for (; p < parts; p += 8) acc += dw_part[static_cast<int64_t>(p) * cols + c];
    }
    partial[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float total = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) total += partial[i][lane];
        Store<T>::store1(dw + c, total);
    }
}

inline int rmsnorm_bwd_ctas(int64_t rows, int per_sm = kRnCtasPerSm) {
    if (per_sm > kRnCtasPerSm) per_sm = kRnCtasPerSm;
    if (per_sm < 1) per_sm = 1;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * per_sm;
    return static_cast<int>(rows < cap ? rows : cap);
}

template <typename T>
cudaError_t run_rmsnorm_bwd(const void* dy, const void* dro_in, const void* ro, const void* w, void* dx, void* dw,
                            float* ws, int64_t rows, int64_t cols, float eps, cudaStream_t s) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t n_vec = cols / kPer;
    if (cols % kPer != 0 || n_vec > static_cast<int64_t>(kRnVpt) * kRnMaxThreads || !aligned16(dy) || !aligned16(ro) ||
        !aligned16(dx) || !aligned16(w) || !aligned16(ws) || (dro_in != nullptr && !aligned16(dro_in)))
        return cudaErrorInvalidValue;
    int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, kRnVpt), 32) * 32);
    if (threads < 32) threads = 32;
    int ctas = 0;
    const size_t smem = static_cast<size_t>(cols) * 2 * sizeof(float);   // weight + d_weight partial, fp32
    auto launch = [&](auto kernel) -> cudaError_t {
        // the row loop is persistent: launch exactly as many CTAs as can be resident at once
        // occupancy depends on (kernel, threads, smem) only: ask once per combination and device
        static thread_local struct { const void* fn; int threads; size_t smem; int dev; int per_sm; } memo[8] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        int per_sm = 0;
        const void* fn = reinterpret_cast<const void*>(kernel);
        for (const auto& m : memo)
            if (m.fn == fn && m.threads == threads && m.smem == smem && m.dev == dev) per_sm = m.per_sm;
        if (per_sm == 0) {
            // the limit is a property of the function, not of this launch: always raise it to the
            // largest row this kernel accepts, so a later launch with a wider row still fits
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kRnVpt * kRnMaxThreads * kPer * 2 * static_cast<int>(sizeof(float)));
            if (e != cudaSuccess) return e;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
            if (e != cudaSuccess) return e;
            if (per_sm < 1) return cudaErrorInvalidValue;
            static thread_local int next = 0;
            memo[next] = {fn, threads, smem, dev, per_sm};
            next = (next + 1) % 8;
        }
        ctas = rmsnorm_bwd_ctas(rows, per_sm);
        kernel<<<ctas, threads, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(dro_in),
                                           static_cast<const T*>(ro), static_cast<const T*>(w), static_cast<T*>(dx), ws,
                                           rows, static_cast<int>(cols), static_cast<int>(n_vec), eps);
        return cudaGetLastError();
    };
    cudaError_t e = dro_in != nullptr ? launch(rmsnorm_bwd_kernel<T, true>) : launch(rmsnorm_bwd_kernel<T, false>);
    if (e != cudaSuccess) return e;
    rmsnorm_dw_reduce_kernel<T><<<static_cast<unsigned>(ceil_div64(cols, 32)), 256, 0, s>>>(
        ws, ctas, static_cast<int>(cols), static_cast<T*>(dw));
    return cudaGetLastError();
}

}  // namespace
}  // namespace cck

// d_gate and d_up of y = silu(gate) * up for an upstream gradient dy, flat over n elements.
// No counterpart in the reference (forward-only).
extern "C" int32_t launch_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup,
                                     int64_t n, int32_t dtype, void* stream) {
    if (n <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run_swiglu_bwd<float>(gate, up, dy, dgate, dup, n, s);
        case cck::kF16:  return cck::run_swiglu_bwd<__half>(gate, up, dy, dgate, dup, n, s);
        case cck::kBF16: return cck::run_swiglu_bwd<__nv_bfloat16>(gate, up, dy, dgate, dup, n, s);
        default:         return cudaErrorInvalidValue;
    }
}

extern "C" int64_t cck_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return static_cast<int64_t>(cck::rmsnorm_bwd_ctas(rows)) * cols * static_cast<int64_t>(sizeof(float));
}

// Gradients of launch_rmsnorm_residual_fwd: dx (= d_x = d_residual, they are equal) and
// dweight, from dy, the saved residual_out, weight, and optionally the gradient d_residual_out
// that arrives through the second output (null when that output is unused downstream).
// workspace: cck_rmsnorm_bwd_workspace_bytes(rows, cols) bytes.  cols must be a multiple of the
// 16-byte vector width and at most 1024 vectors (8192 16-bit or 4096 fp32 columns); otherwise
// cudaErrorInvalidValue.
extern "C" int32_t launch_rmsnorm_residual_bwd(const void* dy, const void* d_residual_out, const void* residual_out,
                                               const void* weight, void* dx, void* dweight, void* workspace,
                                               int64_t workspace_bytes, int64_t rows, int64_t cols, float eps,
                                               int32_t dtype, void* stream) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    if (workspace == nullptr || workspace_bytes < cck_rmsnorm_bwd_workspace_bytes(rows, cols) || cols > 0x7fffffffLL)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* ws = static_cast<float*>(workspace);
    switch (dtype) {
        case cck::kF32:
            return cck::run_rmsnorm_bwd<float>(dy, d_residual_out, residual_out, weight, dx, dweight, ws, rows, cols, eps, s);
        case cck::kF16:
            return cck::run_rmsnorm_bwd<__half>(dy, d_residual_out, residual_out, weight, dx, dweight, ws, rows, cols, eps, s);
        case cck::kBF16:
            return cck::run_rmsnorm_bwd<__nv_bfloat16>(dy, d_residual_out, residual_out, weight, dx, dweight, ws, rows, cols,
                                                       eps, s);
        default:
            return cudaErrorInvalidValue;
    }
}
