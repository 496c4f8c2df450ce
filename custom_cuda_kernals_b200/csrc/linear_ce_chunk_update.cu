// Online-softmax update of per-row (max, sum-exp, target logit) with one
// materialised chunk of logits [N, chunk_v] covering vocabulary columns
// [v_start, v_start + chunk_v).
//
// Same contract as the reference's csrc/kernels/linear_cross_entropy.cu:29-133:
// accumulators are caller-initialised (-inf, 0, 0) and chunks arrive in any
// order of v_start (the update is order independent up to rounding).  This entry
// point exists for callers that already hold logits; the fused GEMM + softmax
// kernel in linear_cross_entropy.cu never materialises them.
//
// One CTA per row.  A row chunk of up to kThreads * kVecPerThread vectors is
// held in registers so it is read from HBM once; longer chunks fall back to two
// passes.  HBM-bound: N * chunk_v * sizeof(T) bytes per launch.
#include "common.cuh"

namespace cck {
namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;

template <typename T>
__global__ void __launch_bounds__(kThreads)
lce_chunk_kernel(const T* __restrict__ logits, const int64_t* __restrict__ targets, int64_t v_start,
                 int64_t chunk_v, float* __restrict__ run_max, float* __restrict__ run_sum,
                 float* __restrict__ tgt_logit, bool vec_ok) {
    constexpr int kPer = Store<T>::kPerVec;
    __shared__ float slots[kThreads / 32];
    const int64_t row = blockIdx.x;
    const T* lr = logits + row * chunk_v;
    const int64_t local_target = targets[row] - v_start;
    const int64_t n_vec = vec_ok ? chunk_v / kPer : 0;
    const bool in_regs = vec_ok && n_vec <= kThreads * kVecPerThread;

    Vec16 keep[kVecPerThread];
    float mx = -INFINITY;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kVecPerThread; ++j) {
            const int64_t i = threadIdx.x + j * kThreads;
            if (i < n_vec) keep[j] = ld_stream(lr + i * kPer);
        }
#pragma unroll
        for (int j = 0; j < kVecPerThread; ++j) {
            const int64_t i = threadIdx.x + j * kThreads;
            if (i < n_vec) {
#pragma unroll
                for (int e = 0; e < kPer; ++e) mx = fmaxf(mx, Store<T>::get(keep[j], e));
            }
        }
    } else {
        for (int64_t i = threadIdx.x; i < n_vec; i += kThreads) {
            const Vec16 v = ld_cached(lr + i * kPer);
#pragma unroll
            for (int e = 0; e < kPer; ++e) mx = fmaxf(mx, Store<T>::get(v, e));
        }
    }
    for (int64_t c = n_vec * kPer + threadIdx.x; c < chunk_v; c += kThreads)
        mx = fmaxf(mx, Store<T>::load1(lr + c));
    if (threadIdx.x == 0 && local_target >= 0 && local_target < chunk_v)
        tgt_logit[row] = Store<T>::load1(lr + local_target);

    const float chunk_max = cta_reduce<kThreads, true>(mx, slots);
    const float old_max = run_max[row];
    const float new_max = fmaxf(old_max, chunk_max);

    float sm = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kVecPerThread; ++j) {
            const int64_t i = threadIdx.x + j * kThreads;
            if (i < n_vec) {
#pragma unroll
                for (int e = 0; e < kPer; ++e) sm += expf(Store<T>::get(keep[j], e) - new_max);
            }
        }
    } else {
        for (int64_t i = threadIdx.x; i < n_vec; i += kThreads) {
            const Vec16 v = ld_cached(lr + i * kPer);
#pragma unroll
            for (int e = 0; e < kPer; ++e) sm += expf(Store<T>::get(v, e) - new_max);
        }
    }
    for (int64_t c = n_vec * kPer + threadIdx.x; c < chunk_v; c += kThreads)
        sm += expf(Store<T>::load1(lr + c) - new_max);
    const float chunk_sum = cta_reduce<kThreads, false>(sm, slots);

    if (threadIdx.x == 0) {
        // exp(-inf - finite) == 0, so the first chunk needs no special case
        run_sum[row] = run_sum[row] * expf(old_max - new_max) + chunk_sum;
        run_max[row] = new_max;
    }
}

template <typename T>
cudaError_t run(const void* logits, const int64_t* targets, int64_t v_start, int64_t n, int64_t chunk_v,
                float* run_max, float* run_sum, float* tgt, cudaStream_t s) {
    if (n > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bool vec_ok = aligned16(logits) && (chunk_v % Store<T>::kPerVec == 0);
    lce_chunk_kernel<T><<<static_cast<unsigned>(n), kThreads, 0, s>>>(
        static_cast<const T*>(logits), targets, v_start, chunk_v, run_max, run_sum, tgt, vec_ok);
    return cudaGetLastError();
}

}  // namespace
}  // namespace cck

extern "C" int32_t launch_linear_ce_chunk_update(const void* logits_chunk, const int64_t* targets,
                                                 int64_t v_start, int64_t n, int64_t chunk_v,
                                                 float* running_max, float* running_sum, float* target_logit,
                                                 int32_t dtype, void* stream) {
    if (n <= 0 || chunk_v <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:
            return cck::run<float>(logits_chunk, targets, v_start, n, chunk_v, running_max, running_sum, target_logit, s);
        case cck::kF16:
            return cck::run<__half>(logits_chunk, targets, v_start, n, chunk_v, running_max, running_sum, target_logit, s);
        case cck::kBF16:
            return cck::run<__nv_bfloat16>(logits_chunk, targets, v_start, n, chunk_v, running_max, running_sum, target_logit, s);
        default:
            return cudaErrorInvalidValue;
    }
}
