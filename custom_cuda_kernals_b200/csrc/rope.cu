// Rotary position embedding, half-split convention, q and k in one launch:
//   out[..., :D/2] = x1*cos - x2*sin;  out[..., D/2:] = x2*cos + x1*sin
// q [B,S,Hq,D], k [B,S,Hkv,D]; cos/sin [S,D/2] fp32; position = index along S.
//
// Replaces the reference's csrc/kernels/rope.cu:56-350 (one warp-sized block
// per 256-byte head row, table re-read for every head).  Here a CTA owns one
// sequence position: each thread loads its slice of that position's cos/sin
// row once into registers and then rotates the same slice of every head for
// kBatchPerCta batch entries, with all 16-byte loads of the two batch entries
// issued before the first use.  fp32 arithmetic, one rounding on store
// (baselines/rope.py:129-138).
//
// HBM-bound: 2 * (|q| + |k|) * sizeof(T) bytes per launch (tables stay in L2).
#include "common.cuh"

namespace cck {
namespace {

constexpr int kBatchPerCta = 2;

template <typename T>
__device__ __forceinline__ void rotate_store(const Vec16& lo, const Vec16& hi,
                                             const float* c, const float* s, T* out_lo, T* out_hi) {
    constexpr int kPer = Store<T>::kPerVec;
    float a[kPer], b[kPer], o1[kPer], o2[kPer];
    unpack<T>(lo, a);
    unpack<T>(hi, b);
#pragma unroll
    for (int e = 0; e < kPer; ++e) rope_rotate(a[e], b[e], c[e], s[e], o1[e], o2[e]);
    st_stream(out_lo, pack<T>(o1));
    st_stream(out_hi, pack<T>(o2));
}

template <typename T>
__global__ void __launch_bounds__(1024)
rope_kernel(const T* __restrict__ q, const T* __restrict__ k, const float* __restrict__ cos_t,
            const float* __restrict__ sin_t, T* __restrict__ q_out, T* __restrict__ k_out,
            int batch, int seq_len, int hq, int hkv, int head_dim, int64_t q_tok_stride, int64_t k_tok_stride) {
    constexpr int kPer = Store<T>::kPerVec;
    const int half = head_dim >> 1;
    const int hv = half / kPer;                 // 16-byte vectors per half row
    const int items = (hq + hkv) * hv;
    const int s_idx = blockIdx.x;
    const int b0 = blockIdx.y * kBatchPerCta;

    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int h = item / hv;
        const int j = item - h * hv;
        float c[kPer], sn[kPer];
        {
            const float* cp = cos_t + static_cast<int64_t>(s_idx) * half + j * kPer;
            const float* sp = sin_t + static_cast<int64_t>(s_idx) * half + j * kPer;
#pragma unroll
            for (int v = 0; v < kPer / 4; ++v) {
                const Vec16 cv = ld_cached(cp + 4 * v), sv = ld_cached(sp + 4 * v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    c[4 * v + e] = __uint_as_float(cv.w[e]);
                    sn[4 * v + e] = __uint_as_float(sv.w[e]);
                }
            }
        }
        const bool is_q = h < hq;
        const T* src = is_q ? q : k;
        T* dst = is_q ? q_out : k_out;
        const int heads = is_q ? hq : hkv;
        const int hh = is_q ? h : h - hq;

        const int64_t in_stride = is_q ? q_tok_stride : k_tok_stride;   // elements between tokens of the input
        Vec16 lo[kBatchPerCta], hi[kBatchPerCta];
        int64_t off[kBatchPerCta];
#pragma unroll
        for (int bb = 0; bb < kBatchPerCta; ++bb) {
            const int b = b0 + bb;
            const int64_t tok = static_cast<int64_t>(b) * seq_len + s_idx;
            off[bb] = (tok * heads + hh) * head_dim + j * kPer;           // outputs are contiguous
            if (b < batch) {
                const int64_t in = tok * in_stride + hh * head_dim + j * kPer;
                lo[bb] = ld_stream(src + in);
                hi[bb] = ld_stream(src + in + half);
            }
        }
#pragma unroll
        for (int bb = 0; bb < kBatchPerCta; ++bb)
            if (b0 + bb < batch)
                rotate_store<T>(lo[bb], hi[bb], c, sn, dst + off[bb], dst + off[bb] + half);
    }
}

// Any even head_dim / alignment: one element pair per thread, grid-stride.
template <typename T>
__global__ void __launch_bounds__(256)
rope_scalar_kernel(const T* __restrict__ q, const T* __restrict__ k, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, T* __restrict__ q_out, T* __restrict__ k_out,
                   int64_t tokens, int seq_len, int hq, int hkv, int head_dim, int64_t q_tok_stride,
                   int64_t k_tok_stride) {
    const int half = head_dim >> 1;
    const int64_t per_token = static_cast<int64_t>(hq + hkv) * half;
    const int64_t total = tokens * per_token;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t tok = idx / per_token;
        const int rem = static_cast<int>(idx - tok * per_token);
        const int h = rem / half, i = rem - h * half;
        const int s_idx = static_cast<int>(tok % seq_len);
        const float c = Store<float>::load1(cos_t + static_cast<int64_t>(s_idx) * half + i);
        const float sn = Store<float>::load1(sin_t + static_cast<int64_t>(s_idx) * half + i);
        const bool is_q = h < hq;
        const T* src = is_q ? q : k;
        T* dst = is_q ? q_out : k_out;
        const int hh = is_q ? h : h - hq;
        const int64_t o = (tok * (is_q ? hq : hkv) + hh) * head_dim + i;
        const int64_t in = tok * (is_q ? q_tok_stride : k_tok_stride) + static_cast<int64_t>(hh) * head_dim + i;
        const float a = Store<T>::load1(src + in), b = Store<T>::load1(src + in + half);
        float o1, o2;
        rope_rotate(a, b, c, sn, o1, o2);
        Store<T>::store1(dst + o, o1);
        Store<T>::store1(dst + o + half, o2);
    }
}

template <typename T>
cudaError_t run(const void* q, const void* k, const void* cos_t, const void* sin_t, void* q_out, void* k_out,
                int64_t batch, int64_t seq_len, int64_t hq, int64_t hkv, int64_t head_dim, int64_t q_tok_stride,
                int64_t k_tok_stride, cudaStream_t stream) {
    constexpr int kPer = Store<T>::kPerVec;
    const int64_t half = head_dim / 2;
    const bool vec_ok = (half % kPer == 0) && q_tok_stride % kPer == 0 && k_tok_stride % kPer == 0 && aligned16(q) && aligned16(k) && aligned16(cos_t) &&
                        aligned16(sin_t) && aligned16(q_out) && aligned16(k_out) &&
                        seq_len <= 0x7fffffffLL && ceil_div64(batch, kBatchPerCta) <= 65535;
    const float* cp = static_cast<const float*>(cos_t);
    const float* sp = static_cast<const float*>(sin_t);
    if (vec_ok) {
        const int64_t items = (hq + hkv) * (half / kPer);
        int threads = static_cast<int>(ceil_div64(items, 32) * 32);
        if (threads > 1024) threads = 1024;
        const dim3 grid(static_cast<unsigned>(seq_len), static_cast<unsigned>(ceil_div64(batch, kBatchPerCta)));
        rope_kernel<T><<<grid, threads, 0, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(k), cp, sp, static_cast<T*>(q_out),
            static_cast<T*>(k_out), static_cast<int>(batch), static_cast<int>(seq_len),
            static_cast<int>(hq), static_cast<int>(hkv), static_cast<int>(head_dim), q_tok_stride, k_tok_stride);
    } else {
        const int64_t total = batch * seq_len * (hq + hkv) * half;
        int64_t ctas = ceil_div64(total, 256);
        const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
        if (ctas > cap) ctas = cap;
        rope_scalar_kernel<T><<<static_cast<unsigned>(ctas), 256, 0, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(k), cp, sp, static_cast<T*>(q_out),
            static_cast<T*>(k_out), batch * seq_len, static_cast<int>(seq_len), static_cast<int>(hq),
            static_cast<int>(hkv), static_cast<int>(head_dim), q_tok_stride, k_tok_stride);
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace cck

namespace {
int32_t rope_dispatch(const void* q, const void* k, const void* cos_table, const void* sin_table, void* q_out,
                      void* k_out, int64_t batch, int64_t seq_len, int64_t n_q_heads, int64_t n_kv_heads,
                      int64_t head_dim, int64_t q_tok_stride, int64_t k_tok_stride, int32_t dtype, void* stream) {
    if (batch <= 0 || seq_len <= 0 || head_dim <= 0 || (n_q_heads + n_kv_heads) <= 0) return cudaSuccess;
    if (head_dim & 1) return cudaErrorInvalidValue;
    if (q_tok_stride < n_q_heads * head_dim || k_tok_stride < n_kv_heads * head_dim) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:
            return cck::run<float>(q, k, cos_table, sin_table, q_out, k_out, batch, seq_len, n_q_heads, n_kv_heads,
                                   head_dim, q_tok_stride, k_tok_stride, s);
        case cck::kF16:
            return cck::run<__half>(q, k, cos_table, sin_table, q_out, k_out, batch, seq_len, n_q_heads, n_kv_heads,
                                    head_dim, q_tok_stride, k_tok_stride, s);
        case cck::kBF16:
            return cck::run<__nv_bfloat16>(q, k, cos_table, sin_table, q_out, k_out, batch, seq_len, n_q_heads,
                                           n_kv_heads, head_dim, q_tok_stride, k_tok_stride, s);
        default:
            return cudaErrorInvalidValue;
    }
}
}  // namespace

extern "C" int32_t launch_rope_fwd(const void* q, const void* k, const void* cos_table, const void* sin_table,
                                   void* q_out, void* k_out, int64_t batch, int64_t seq_len,
                                   int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, int32_t dtype,
                                   void* stream) {
    return rope_dispatch(q, k, cos_table, sin_table, q_out, k_out, batch, seq_len, n_q_heads, n_kv_heads, head_dim,
                         n_q_heads * head_dim, n_kv_heads * head_dim, dtype, stream);
}

// Same rotation for inputs whose tokens are not packed: consecutive tokens of q (of k) are
// q_token_stride (k_token_stride) elements apart, e.g. q and k are column ranges of one fused
// QKV projection output.  Within a token the heads are contiguous; the outputs are contiguous.
extern "C" int32_t launch_rope_strided_fwd(const void* q, const void* k, const void* cos_table,
                                           const void* sin_table, void* q_out, void* k_out, int64_t batch,
                                           int64_t seq_len, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                                           int64_t q_token_stride, int64_t k_token_stride, int32_t dtype,
                                           void* stream) {
    return rope_dispatch(q, k, cos_table, sin_table, q_out, k_out, batch, seq_len, n_q_heads, n_kv_heads, head_dim,
                         q_token_stride, k_token_stride, dtype, stream);
}

CCK_DEBUG_BOUNDS_EXPORT(rope)
