// Mixture-of-experts neighbours of the decoder block: the top-k softmax router and the two
// row movers around the expert FFNs (gather into per-expert order, weighted combine back).
//
// Replaces the reference's csrc/kernels/moe_router.cu (one warp per token whatever the
// expert count) and csrc/kernels/token_permute.cu (one block per row, one 16-byte vector in
// flight per thread).  Here:
//   * router: a token is owned by a group of L = 1..32 lanes, L the smallest power of two with
//     8 * L >= experts, each lane holding 8 logits in registers - 8 experts is one THREAD per
//     token with a single 16-byte load, 256 experts a full warp.  Softmax statistics run on
//     xor-shuffles inside the group; each of the k arg-max rounds is one integer max-reduction
//     (redux.sync) when the group is a whole warp - on a packed (value, expert) key for 16-bit
//     logits, on the value followed by a ballot and a shuffle for fp32 - and a shuffle butterfly
//     otherwise; ties go to the lower expert id.
//   * gather: warps walk destination rows; a lane keeps four 16-byte vectors in flight and the
//     next row's index is fetched while the current row streams.
//   * combine: warps walk tokens, fp32 accumulators in registers, the token's indices and
//     weights fetched by one coalesced load and handed out by shuffles, two expert rows (8
//     vectors per lane) in flight.
// All three are HBM-bound; semantics follow baselines/moe_router.py:109-119 and
// baselines/token_permute.py:196-226.
#include "common.cuh"

namespace cck { namespace tc { unsigned int* status_word(); } }   // matmul_add_bias.cu: the per-device status word

namespace cck {
namespace {

// ------------------------------------------------------------------ router
constexpr int kRouterVals = 8;       // logits per lane
constexpr int kRouterThreads = 256;

// The 16 bits a 16-bit storage type holds for `f` (exact: `f` was read from that type), and back.
template <typename T> struct Bits16;
template <> struct Bits16<__nv_bfloat16> {
    __device__ static __forceinline__ uint32_t of(float f) { return __float_as_uint(f) >> 16; }
    __device__ static __forceinline__ float to_float(uint32_t b) { return __uint_as_float(b << 16); }
};
template <> struct Bits16<__half> {
    __device__ static __forceinline__ uint32_t of(float f) { return __half_as_ushort(__float2half_rn(f)); }
    __device__ static __forceinline__ float to_float(uint32_t b) {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
    }
};

template <typename T, int L>
__global__ void __launch_bounds__(kRouterThreads)
moe_router_kernel(const T* __restrict__ logits, float* __restrict__ topk_w, int64_t* __restrict__ topk_i,
                  int64_t n_tokens, int experts, int k, int renormalize, int vec_ok) {
    constexpr int kPer = Store<T>::kPerVec;
    const int sub = threadIdx.x % L;                                       // lane within the token's group
    const int64_t token = (static_cast<int64_t>(blockIdx.x) * kRouterThreads + threadIdx.x) / L;
    const bool live = token < n_tokens;
    const T* row = logits + (live ? token : 0) * experts;

    float v[kRouterVals];
#pragma unroll
    for (int i = 0; i < kRouterVals; ++i) v[i] = -INFINITY;
    if (live) {
        if (vec_ok) {                          // experts % 8 == 0: whole 16-byte vectors
            if (sub * kRouterVals < experts) {
#pragma unroll
                for (int q = 0; q < kRouterVals / kPer; ++q) {
                    float f[kPer];
                    unpack<T>(ld_stream(row + sub * kRouterVals + q * kPer), f);
#pragma unroll
                    for (int e = 0; e < kPer; ++e) v[q * kPer + e] = f[e];
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < kRouterVals; ++i) {
                const int e = sub * kRouterVals + i;
                if (e < experts) v[i] = Store<T>::load1(row + e);
            }
        }
    }
    // softmax statistics over the group
    float mx = v[0];
#pragma unroll
    for (int i = 1; i < kRouterVals; ++i) mx = fmaxf(mx, v[i]);
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kRouterVals; ++i) sum += __expf(v[i] - mx);         // exp(-inf) = 0 for the padding
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv_sum = 1.0f / sum;

    float picked = 0.0f;                        // sum of the selected probabilities
    // With k <= L, lane j of the group keeps the j-th result in registers: one coalesced store of
    // weights and ids per token at the end, renormalised on the way, instead of two narrow stores
    // per round and a global read-modify-write pass for the renormalisation.
    const bool in_regs = k <= L;
    float my_p = 0.0f;
    int my_e = 0;
    if constexpr (L == 32 && sizeof(T) == 2) {
        // 16-bit logits, whole warp per token: value and expert id fit one 32-bit key - the value's
        // bits made order-preserving in the high half, 255 - expert in the low byte, so that a
        // plain unsigned max picks the largest logit and, among equals, the lowest expert; keys
        // are unique.
        uint32_t key[kRouterVals];
#pragma unroll
        for (int i = 0; i < kRouterVals; ++i) {
            const int e = sub * kRouterVals + i;
            const uint32_t b = Bits16<T>::of(v[i]);
            const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
            key[i] = e < experts ? ((ord << 16) | static_cast<uint32_t>(255 - e)) : 0u;
        }
        // Each lane first sorts its eight keys (19 compare-exchanges); a round is then ONE
        // redux.sync over the lanes' current heads, and the lane that owned the winner moves its
        // list up by one - 10 instructions a round where scanning the eight keys took 24.
#define CCK_CE(a, b)                                         \
    {                                                        \
        const uint32_t hi = max(key[a], key[b]);             \
        key[b] = min(key[a], key[b]);                        \
        key[a] = hi;                                         \
    }
        CCK_CE(0, 1) CCK_CE(2, 3) CCK_CE(4, 5) CCK_CE(6, 7)
        CCK_CE(0, 2) CCK_CE(1, 3) CCK_CE(4, 6) CCK_CE(5, 7)
        CCK_CE(1, 2) CCK_CE(5, 6) CCK_CE(0, 4) CCK_CE(3, 7)
        CCK_CE(1, 5) CCK_CE(2, 6)
        CCK_CE(1, 4) CCK_CE(3, 6)
        CCK_CE(2, 4) CCK_CE(3, 5)
        CCK_CE(3, 4)
#undef CCK_CE
        auto decode = [&](uint32_t top, float& p, int& e) {
            const uint32_t ord = top >> 16;
            const float best = Bits16<T>::to_float((ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu));
            p = __expf(best - mx) * inv_sum;
            e = 255 - static_cast<int>(top & 0xffu);
        };
        if (in_regs) {
            // the rounds only move keys: lane j keeps the j-th winner's key and turns it into a
            // probability and an expert id once, after the loop
            uint32_t my_top = 0u;
            for (int j = 0; j < k; ++j) {
                const uint32_t top = __reduce_max_sync(0xffffffffu, key[0]);
                if (key[0] == top) {             // keys are unique: exactly one lane
#pragma unroll
                    for (int i = 0; i + 1 < kRouterVals; ++i) key[i] = key[i + 1];
                    key[kRouterVals - 1] = 0u;
                }
                if (sub == j) my_top = top;
            }
            decode(my_top, my_p, my_e);
            if (sub >= k) my_p = 0.0f;
            for (int j = 0; j < k; ++j) picked += __shfl_sync(0xffffffffu, my_p, j);   // in selection order
        } else {
            for (int j = 0; j < k; ++j) {
                const uint32_t top = __reduce_max_sync(0xffffffffu, key[0]);
                if (key[0] == top) {
#pragma unroll
                    for (int i = 0; i + 1 < kRouterVals; ++i) key[i] = key[i + 1];
                    key[kRouterVals - 1] = 0u;
                }
                float p;
                int e;
                decode(top, p, e);
                picked += p;
                if (live && sub == j % L) {
                    topk_w[token * k + j] = p;
                    topk_i[token * k + j] = e;
                }
            }
        }
    } else {
        // k rounds of arg-max; a selected logit is replaced by -inf in its owner's registers.
        // Equal logits go to the lower expert id: strict '>' keeps the first of a lane's values,
        // and across lanes the lower lane (= lower ids) wins.
        for (int j = 0; j < k; ++j) {
            float best = v[0];
            int best_i = 0;
    #pragma unroll
            for (int i = 1; i < kRouterVals; ++i)
                if (v[i] > best) {
                    best = v[i];
                    best_i = i;
                }
            int best_e;
            if constexpr (L == 32) {
                // whole warp: one integer max-reduction on an order-preserving key, one ballot for
                // the owner, one shuffle for the owner's slot - instead of ten shuffles.  (Sub-warp
                // groups keep the butterfly: redux.sync with one mask per group measured slower.)
                const uint32_t bits = __float_as_uint(best);
                const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
                const uint32_t top = __reduce_max_sync(0xffffffffu, key);
                const int owner = __ffs(__ballot_sync(0xffffffffu, key == top)) - 1;
                best_e = owner * kRouterVals + __shfl_sync(0xffffffffu, best_i, owner);
                best = __uint_as_float((top & 0x80000000u) ? (top & 0x7fffffffu) : ~top);
            } else {
                best_e = sub * kRouterVals + best_i;
    #pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                    if (ov > best || (ov == best && oe < best_e)) {
                        best = ov;
                        best_e = oe;
                    }
                }
            }
            if (best_e / kRouterVals == sub) {
    #pragma unroll
                for (int i = 0; i < kRouterVals; ++i)
                    if (i == best_e % kRouterVals) v[i] = -INFINITY;
            }
            const float p = __expf(best - mx) * inv_sum;
            picked += p;
            if (in_regs) {
                if (sub == j) {
                    my_p = p;
                    my_e = best_e;
                }
            } else if (live && sub == j % L) {
                topk_w[token * k + j] = p;
                topk_i[token * k + j] = best_e;
            }
        }
    }
    if (in_regs) {
        if (live && sub < k) {
            topk_w[token * k + sub] = renormalize ? my_p * (1.0f / picked) : my_p;
            topk_i[token * k + sub] = my_e;
        }
    } else if (renormalize && live) {
        const float inv = 1.0f / picked;
        for (int j = sub; j < k; j += L) topk_w[token * k + j] *= inv;      // each lane rescales what it wrote
    }
}

// The common large case on its own: 16-bit logits, 129..256 experts (a whole warp per token),
// k <= 32.  Same arithmetic as the packed-key path of moe_router_kernel; a warp handles TOK tokens
// at once with independent register sets, so that the dependent chain of one token (load, sort,
// k redux.sync rounds) fills the issue slots the other leaves empty.
template <typename T, int TOK>
__global__ void __launch_bounds__(kRouterThreads)
moe_router_packed_kernel(const T* __restrict__ logits, float* __restrict__ topk_w, int64_t* __restrict__ topk_i,
                         int64_t n_tokens, int experts, int k, int renormalize) {
    constexpr int kPer = Store<T>::kPerVec;
    static_assert(sizeof(T) == 2 && kRouterVals == kPer, "one 16-byte vector of 16-bit logits per lane");
    const int sub = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kRouterThreads + threadIdx.x) >> 5;
    float v[TOK][kRouterVals];
    uint32_t key[TOK][kRouterVals];
    bool live[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        const int64_t token = warp * TOK + t;
        live[t] = token < n_tokens;
#pragma unroll
        for (int i = 0; i < kRouterVals; ++i) v[t][i] = -INFINITY;
        if (live[t] && sub * kRouterVals < experts) unpack<T>(ld_stream(logits + token * experts + sub * kRouterVals), v[t]);
    }
    float mx[TOK], inv_sum[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        mx[t] = v[t][0];
#pragma unroll
        for (int i = 1; i < kRouterVals; ++i) mx[t] = fmaxf(mx[t], v[t][i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int t = 0; t < TOK; ++t) mx[t] = fmaxf(mx[t], __shfl_xor_sync(0xffffffffu, mx[t], o));
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kRouterVals; ++i) sum += __expf(v[t][i] - mx[t]);
        inv_sum[t] = sum;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int t = 0; t < TOK; ++t) inv_sum[t] += __shfl_xor_sync(0xffffffffu, inv_sum[t], o);
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        inv_sum[t] = 1.0f / inv_sum[t];
#pragma unroll
        for (int i = 0; i < kRouterVals; ++i) {
            const int e = sub * kRouterVals + i;
            const uint32_t b = Bits16<T>::of(v[t][i]);
            const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
            key[t][i] = e < experts ? ((ord << 16) | static_cast<uint32_t>(255 - e)) : 0u;
        }
#define CCK_CE(a, b)                                               \
    {                                                              \
        const uint32_t hi = max(key[t][a], key[t][b]);             \
        key[t][b] = min(key[t][a], key[t][b]);                     \
        key[t][a] = hi;                                            \
    }
        CCK_CE(0, 1) CCK_CE(2, 3) CCK_CE(4, 5) CCK_CE(6, 7)
        CCK_CE(0, 2) CCK_CE(1, 3) CCK_CE(4, 6) CCK_CE(5, 7)
        CCK_CE(1, 2) CCK_CE(5, 6) CCK_CE(0, 4) CCK_CE(3, 7)
        CCK_CE(1, 5) CCK_CE(2, 6)
        CCK_CE(1, 4) CCK_CE(3, 6)
        CCK_CE(2, 4) CCK_CE(3, 5)
        CCK_CE(3, 4)
#undef CCK_CE
    }
    uint32_t my_top[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) my_top[t] = 0u;
    for (int j = 0; j < k; ++j) {
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            const uint32_t top = __reduce_max_sync(0xffffffffu, key[t][0]);
            if (key[t][0] == top) {              // keys are unique: exactly one lane
#pragma unroll
                for (int i = 0; i + 1 < kRouterVals; ++i) key[t][i] = key[t][i + 1];
                key[t][kRouterVals - 1] = 0u;
            }
            if (sub == j) my_top[t] = top;
        }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        const uint32_t ord = my_top[t] >> 16;
        const float best = Bits16<T>::to_float((ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu));
        const float my_p = sub < k ? __expf(best - mx[t]) * inv_sum[t] : 0.0f;
        const int my_e = 255 - static_cast<int>(my_top[t] & 0xffu);
        float picked = 0.0f;
        for (int j = 0; j < k; ++j) picked += __shfl_sync(0xffffffffu, my_p, j);     // in selection order
        const int64_t token = warp * TOK + t;
        if (live[t] && sub < k) {
            topk_w[token * k + sub] = renormalize ? my_p * (1.0f / picked) : my_p;
            topk_i[token * k + sub] = my_e;
        }
    }
}

template <typename T>
cudaError_t run_router(const void* logits, float* w, int64_t* idx, int64_t n_tokens, int64_t experts, int64_t k,
                       int renorm, cudaStream_t s) {
    constexpr int kPer = Store<T>::kPerVec;
    const T* lg = static_cast<const T*>(logits);
    const int vec_ok = (experts % kRouterVals == 0 && aligned16(logits)) ? 1 : 0;
    int lanes = 1;
    while (lanes * kRouterVals < experts) lanes *= 2;
    const int64_t tokens_per_cta = kRouterThreads / lanes;
    const unsigned grid = static_cast<unsigned>(ceil_div64(n_tokens, tokens_per_cta));
    const int e = static_cast<int>(experts), kk = static_cast<int>(k);
    (void)kPer;
    if constexpr (sizeof(T) == 2) {
        if (lanes == 32 && vec_ok && kk <= 32) {
            constexpr int kTok = 2;       // measured at 16384 x 256 top-8: 1 token per warp 10.3 us, 2: 9.5, 4: 10.4
            const int64_t warps = ceil_div64(n_tokens, kTok);
            const unsigned g = static_cast<unsigned>(ceil_div64(warps, kRouterThreads / 32));
            moe_router_packed_kernel<T, kTok><<<g, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm);
            return cudaGetLastError();
        }
    }
    switch (lanes) {
        case 1:  moe_router_kernel<T, 1><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
        case 2:  moe_router_kernel<T, 2><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
        case 4:  moe_router_kernel<T, 4><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
        case 8:  moe_router_kernel<T, 8><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
        case 16: moe_router_kernel<T, 16><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
        default: moe_router_kernel<T, 32><<<grid, kRouterThreads, 0, s>>>(lg, w, idx, n_tokens, e, kk, renorm, vec_ok); break;
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------ gather
constexpr int kGatherThreads = 256;
constexpr int kGatherUnroll = 4;

// dst[i] = src[indices[i]] as raw 16-byte vectors (no arithmetic, so the element type is irrelevant)
__global__ void __launch_bounds__(kGatherThreads)
token_gather_vec_kernel(const Vec16* __restrict__ src, const int64_t* __restrict__ indices, Vec16* __restrict__ dst,
                        int64_t n_rows, int64_t n_vec) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kGatherThreads / 32);
    int64_t row = static_cast<int64_t>(blockIdx.x) * (kGatherThreads / 32) + (threadIdx.x >> 5);
    int64_t from = row < n_rows ? indices[row] : 0;
    for (; row < n_rows; row += warps) {
        const int64_t next = row + warps;
        const int64_t from_next = next < n_rows ? indices[next] : 0;       // fetched while this row streams
        const Vec16* s = src + from * n_vec;
        Vec16* d = dst + row * n_vec;
        for (int64_t i0 = lane; i0 < n_vec; i0 += 32 * kGatherUnroll) {
            Vec16 x[kGatherUnroll];
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i0 + 32 * u < n_vec) x[u] = ld_stream(s + i0 + 32 * u);
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i0 + 32 * u < n_vec) st_stream(d + i0 + 32 * u, x[u]);
        }
        from = from_next;
    }
}

// rows that are not whole aligned 16-byte vectors: element by element
template <typename T>
__global__ void __launch_bounds__(kGatherThreads)
token_gather_scalar_kernel(const T* __restrict__ src, const int64_t* __restrict__ indices, T* __restrict__ dst,
                           int64_t n_rows, int64_t hidden) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kGatherThreads / 32);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (kGatherThreads / 32) + (threadIdx.x >> 5); row < n_rows;
         row += warps) {
        const T* s = src + indices[row] * hidden;
        T* d = dst + row * hidden;
        for (int64_t c = lane; c < hidden; c += 32) d[c] = s[c];
    }
}

// One warp per row up to 64 waves of CTAs (the hardware hands out CTAs as SMs free up, which
// balances better than a fixed number of rows per warp); beyond that the warps loop.
inline unsigned warp_grid(int64_t rows) {
    const int64_t ctas = ceil_div64(rows, kGatherThreads / 32);
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 8 * 64;
    return static_cast<unsigned>(ctas < cap ? ctas : cap);
}

// ------------------------------------------------------------------ combine
constexpr int kCombineVpt = 4;
constexpr int kCombineMaxThreads = 256;

template <typename T>
__device__ __forceinline__ void fma_vec(float (&acc)[Store<T>::kPerVec], const Vec16& x, float w) {
    float f[Store<T>::kPerVec];
    unpack<T>(x, f);
#pragma unroll
    for (int e = 0; e < Store<T>::kPerVec; ++e) acc[e] = fmaf(w, f[e], acc[e]);
}

// combined[t] = sum_j weights[t, j] * expert_output[unpermute_index[t, j]], fp32 accumulation
// in index order.  Warps walk tokens (grid-stride).  Lane j of the warp holds the token's j-th
// (index, weight) pair - one coalesced load per token, handed out by shuffles - so no row load
// waits on an index of its own; a lane owns kCombineVpt vectors of the 32 * kCombineVpt-vector
// slab being reduced and keeps two expert rows (8 vectors) in flight.
template <typename T>
__global__ void __launch_bounds__(kCombineMaxThreads)
token_combine_vec_kernel(const T* __restrict__ expert_out, const int64_t* __restrict__ uidx,
                         const float* __restrict__ weights, T* __restrict__ combined, int64_t n_tokens, int k,
                         int64_t n_vec) {
    constexpr int kPer = Store<T>::kPerVec;
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kCombineMaxThreads / 32);
    const Vec16* base = reinterpret_cast<const Vec16*>(expert_out);
    for (int64_t token = static_cast<int64_t>(blockIdx.x) * (kCombineMaxThreads / 32) + (threadIdx.x >> 5);
         token < n_tokens; token += warps) {
        Vec16* out = reinterpret_cast<Vec16*>(combined) + token * n_vec;
        // the first 32 (index, weight) pairs are fetched once per token, not once per slab
        const int64_t first_row = lane < k ? __ldg(uidx + token * k + lane) : 0;
        const float first_w = lane < k ? __ldg(weights + token * k + lane) : 0.0f;
        for (int64_t slab = 0; slab < n_vec; slab += 32 * kCombineVpt) {     // warp-uniform: every lane shuffles
            const int64_t i0 = slab + lane;
            float acc[kCombineVpt][kPer];
#pragma unroll
            for (int u = 0; u < kCombineVpt; ++u)
#pragma unroll
                for (int e = 0; e < kPer; ++e) acc[u][e] = 0.0f;
            for (int j0 = 0; j0 < k; j0 += 32) {
                const int mine = j0 + lane;
                const int64_t my_row = j0 == 0 ? first_row : (mine < k ? __ldg(uidx + token * k + mine) : 0);
                const float my_w = j0 == 0 ? first_w : (mine < k ? __ldg(weights + token * k + mine) : 0.0f);
                const int in_chunk = k - j0 < 32 ? k - j0 : 32;
                for (int c = 0; c < in_chunk; c += 2) {
                    const bool two = c + 1 < in_chunk;
                    const int64_t row0 = __shfl_sync(0xffffffffu, my_row, c);
                    const int64_t row1 = __shfl_sync(0xffffffffu, my_row, two ? c + 1 : c);
                    const float w0 = __shfl_sync(0xffffffffu, my_w, c);
                    const float w1 = __shfl_sync(0xffffffffu, my_w, two ? c + 1 : c);
                    const Vec16* r0 = base + row0 * n_vec;
                    const Vec16* r1 = base + row1 * n_vec;
                    Vec16 a[kCombineVpt], b[kCombineVpt];
#pragma unroll
                    for (int u = 0; u < kCombineVpt; ++u) {
                        const int64_t i = i0 + 32 * u;
                        if (i < n_vec) {
                            a[u] = ld_stream(r0 + i);
                            if (two) b[u] = ld_stream(r1 + i);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kCombineVpt; ++u) {
                        const int64_t i = i0 + 32 * u;
                        if (i < n_vec) {
                            fma_vec<T>(acc[u], a[u], w0);
                            if (two) fma_vec<T>(acc[u], b[u], w1);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kCombineVpt; ++u) {
                const int64_t i = i0 + 32 * u;
                if (i < n_vec) st_stream(out + i, pack<T>(acc[u]));
            }
        }
    }
}

// Few choices per token (k <= 4, the usual top-2 / top-4): one CTA per token, a thread owns VPT
// vectors of the row and issues the loads of all k expert rows for them up front (k * VPT 16-byte
// loads in flight per thread, indices and weights read as broadcast loads), accumulates in index
// order and stores - the shape of the other row kernels here, at a third of the registers of the
// warp-per-token kernel above and therefore several times its resident warps.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024)
token_combine_row_kernel(const T* __restrict__ expert_out, const int64_t* __restrict__ uidx,
                         const float* __restrict__ weights, T* __restrict__ combined, int k, int n_vec) {
    constexpr int kPer = Store<T>::kPerVec;
    constexpr int kMaxK = 4;
    const int64_t token = blockIdx.x;
    const Vec16* base = reinterpret_cast<const Vec16*>(expert_out);
    int64_t row[kMaxK];
    float w[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
        row[j] = j < k ? __ldg(uidx + token * k + j) : 0;
        w[j] = j < k ? __ldg(weights + token * k + j) : 0.0f;
    }
    Vec16 x[kMaxK][VPT];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j)
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int i = threadIdx.x + u * blockDim.x;
            if (j < k && i < n_vec) x[j][u] = ld_stream(base + row[j] * n_vec + i);
        }
    Vec16* out = reinterpret_cast<Vec16*>(combined) + token * n_vec;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i >= n_vec) continue;
        float acc[kPer];
#pragma unroll
        for (int e = 0; e < kPer; ++e) acc[e] = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxK; ++j)
            if (j < k) fma_vec<T>(acc, x[j][u], w[j]);
        st_stream(out + i, pack<T>(acc));
    }
}

template <typename T>
__global__ void __launch_bounds__(kCombineMaxThreads)
token_combine_scalar_kernel(const T* __restrict__ expert_out, const int64_t* __restrict__ uidx,
                            const float* __restrict__ weights, T* __restrict__ combined, int k, int64_t hidden) {
    const int64_t token = blockIdx.x;
    for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < k; ++j)
            acc = fmaf(weights[token * k + j], Store<T>::load1(expert_out + uidx[token * k + j] * hidden + c), acc);
        Store<T>::store1(combined + token * hidden + c, acc);
    }
}

template <typename T>
cudaError_t run_combine(const void* expert_out, const int64_t* uidx, const float* weights, void* combined,
                        int64_t n_tokens, int64_t k, int64_t hidden, cudaStream_t s) {
    constexpr int kPer = Store<T>::kPerVec;
    if (n_tokens > 0x7fffffffLL || k > 0x7fffffffLL) return cudaErrorInvalidValue;
    const T* e = static_cast<const T*>(expert_out);
    T* c = static_cast<T*>(combined);
    if (hidden % kPer == 0 && aligned16(expert_out) && aligned16(combined)) {
        const int64_t n_vec = hidden / kPer;
        if (k <= 4 && n_vec <= 2048) {          // CTA per token, two vectors per thread
            int threads = static_cast<int>(ceil_div64(ceil_div64(n_vec, 2), 32) * 32);
            if (threads < 32) threads = 32;
            token_combine_row_kernel<T, 2><<<static_cast<unsigned>(n_tokens), threads, 0, s>>>(
                e, uidx, weights, c, static_cast<int>(k), static_cast<int>(n_vec));
            return cudaGetLastError();
        }
        token_combine_vec_kernel<T><<<warp_grid(n_tokens), kCombineMaxThreads, 0, s>>>(e, uidx, weights, c, n_tokens,
                                                                                     static_cast<int>(k), n_vec);
    } else {
        token_combine_scalar_kernel<T><<<static_cast<unsigned>(n_tokens), 128, 0, s>>>(e, uidx, weights, c, static_cast<int>(k), hidden);
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------ expert-parallel row exchange
// The same two row movers with one level of indirection: the destination (dispatch) or the
// source (combine) of a row is (rank, row) - a base pointer out of a table of `world` buffers,
// which in a multi-GPU run are the ranks' receive buffers mapped into this process (peer
// memory over NVLink), plus a row index.  The kernels only push or pull: nothing in them waits
// for another GPU; the caller separates the phases with stream-ordered barriers.  Every
// (rank, row) is checked against the table size and the buffers' capacity; a row that fails the
// check is skipped and bit 2 of the status word is set, so a wrong plan cannot fault a GPU.
constexpr unsigned int kStatusBadRoute = 4u;

__global__ void __launch_bounds__(kGatherThreads)
token_dispatch_kernel(const Vec16* __restrict__ src, const int64_t* __restrict__ src_row,
                      const int64_t* __restrict__ dst_rank, const int64_t* __restrict__ dst_row,
                      const int64_t* __restrict__ dst_bases, int world, int64_t capacity_rows, int64_t n_src_rows,
                      int64_t n, int64_t n_vec, unsigned int* status) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kGatherThreads / 32);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * (kGatherThreads / 32) + (threadIdx.x >> 5); i < n; i += warps) {
        const int64_t from = src_row[i], rank = dst_rank[i], to = dst_row[i];
        if (from < 0 || from >= n_src_rows || rank < 0 || rank >= world || to < 0 || to >= capacity_rows) {
            if (lane == 0) atomicOr(status, kStatusBadRoute);
            continue;
        }
        const Vec16* s = src + from * n_vec;
        Vec16* d = reinterpret_cast<Vec16*>(static_cast<uintptr_t>(dst_bases[rank])) + to * n_vec;
        for (int64_t i0 = lane; i0 < n_vec; i0 += 32 * kGatherUnroll) {
            Vec16 x[kGatherUnroll];
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i0 + 32 * u < n_vec) x[u] = ld_stream(s + i0 + 32 * u);
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i0 + 32 * u < n_vec) *(d + i0 + 32 * u) = x[u];      // plain store: the target may be peer memory
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kCombineMaxThreads)
token_combine_remote_kernel(const int64_t* __restrict__ src_bases, int world, int64_t capacity_rows,
                            const int64_t* __restrict__ src_rank, const int64_t* __restrict__ src_row,
                            const float* __restrict__ weights, T* __restrict__ combined, int64_t n_tokens, int k,
                            int64_t n_vec, unsigned int* status) {
    constexpr int kPer = Store<T>::kPerVec;
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kCombineMaxThreads / 32);
    for (int64_t token = static_cast<int64_t>(blockIdx.x) * (kCombineMaxThreads / 32) + (threadIdx.x >> 5);
         token < n_tokens; token += warps) {
        Vec16* out = reinterpret_cast<Vec16*>(combined) + token * n_vec;
        for (int64_t slab = 0; slab < n_vec; slab += 32 * kCombineVpt) {
            const int64_t i0 = slab + lane;
            float acc[kCombineVpt][kPer];
#pragma unroll
            for (int u = 0; u < kCombineVpt; ++u)
#pragma unroll
                for (int e = 0; e < kPer; ++e) acc[u][e] = 0.0f;
            for (int j = 0; j < k; ++j) {                                  // warp-uniform loads
                const int64_t rank = __ldg(src_rank + token * k + j), row = __ldg(src_row + token * k + j);
                const float w = __ldg(weights + token * k + j);
                if (rank < 0 || rank >= world || row < 0 || row >= capacity_rows) {
                    if (lane == 0 && slab == 0) atomicOr(status, kStatusBadRoute);
                    continue;
                }
                const Vec16* r = reinterpret_cast<const Vec16*>(static_cast<uintptr_t>(src_bases[rank])) + row * n_vec;
                Vec16 a[kCombineVpt];
#pragma unroll
                for (int u = 0; u < kCombineVpt; ++u)
                    if (i0 + 32 * u < n_vec) a[u] = *(r + i0 + 32 * u);      // plain load: the source may be peer memory
#pragma unroll
                for (int u = 0; u < kCombineVpt; ++u)
                    if (i0 + 32 * u < n_vec) fma_vec<T>(acc[u], a[u], w);
            }
#pragma unroll
            for (int u = 0; u < kCombineVpt; ++u)
                if (i0 + 32 * u < n_vec) st_stream(out + i0 + 32 * u, pack<T>(acc[u]));
        }
    }
}

// ---- the plan of one expert-parallel call, in one launch.
// From this rank's flattened top-k expert ids and the all-gathered count matrix
// counts[source][expert]: a STABLE counting sort of the (token, choice) pairs by expert (pairs
// of one expert keep their order), and for every pair the rank that owns its expert and the row
// it takes in that rank's receive buffer - blocks in source-rank order, inside a block sorted by
// expert.  One CTA walks the pairs 1024 at a time: a pair's position among the equal-expert
// pairs of its warp comes from match_any, the warps' counts are prefix-summed per expert in
// shared memory (32 x experts 16-bit cells), and a running per-expert base carries over to the
// next 1024.  meta[0] = rows this rank receives, meta[1] = the most any rank receives.
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxExperts = 256;   // the router's own limit
constexpr int kPlanMaxWorld = 32;

__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const int64_t* __restrict__ topk, const int64_t* __restrict__ counts, int64_t n, int k, int world,
               int experts, int rank, int64_t* __restrict__ src_row, int64_t* __restrict__ dst_rank,
               int64_t* __restrict__ dst_row, int64_t* __restrict__ pull_rank, int64_t* __restrict__ pull_row,
               int64_t* __restrict__ meta, unsigned int* status) {
    __shared__ int64_t per_rank[kPlanMaxWorld * kPlanMaxWorld];      // [source][destination]
    __shared__ int64_t seg_start[kPlanMaxWorld], first[kPlanMaxWorld];
    __shared__ int64_t expert_start[kPlanMaxExperts], base[kPlanMaxExperts];
    __shared__ uint16_t hist[32 * kPlanMaxExperts];                  // [warp][expert]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int epr = experts / world;
    for (int i = tid; i < world * world; i += kPlanThreads) {
        const int s = i / world, r = i - s * world;
        int64_t sum = 0;
        for (int e = 0; e < epr; ++e) sum += counts[static_cast<int64_t>(s) * experts + r * epr + e];
        per_rank[i] = sum;
    }
    __syncthreads();
    if (tid < world) {
        int64_t before = 0, mine_before = 0, total = 0;
        for (int s = 0; s < world; ++s) {
            if (s < rank) before += per_rank[s * world + tid];
            total += per_rank[s * world + tid];
        }
        for (int r = 0; r < tid; ++r) mine_before += per_rank[rank * world + r];
        seg_start[tid] = before;
        first[tid] = mine_before;
        base[tid] = total;                      // borrowed for the max below
    }
    __syncthreads();
    if (tid == 0) {
        int64_t worst = 0;
        for (int r = 0; r < world; ++r) worst = base[r] > worst ? base[r] : worst;
        meta[0] = base[rank];
        meta[1] = worst;
        int64_t run = 0;
        for (int e = 0; e < experts; ++e) {
            expert_start[e] = run;
            run += counts[static_cast<int64_t>(rank) * experts + e];
        }
    }
    __syncthreads();
    if (tid < experts) base[tid] = 0;
    for (int64_t p0 = 0; p0 < n; p0 += kPlanThreads) {
        for (int i = tid; i < 32 * experts; i += kPlanThreads) hist[i] = 0;
        const int64_t p = p0 + tid;
        int e = experts;                                             // sentinel: no pair / bad id
        if (p < n) {
            const int64_t v = topk[p];
            if (v >= 0 && v < experts) e = static_cast<int>(v);
            else atomicOr(status, kStatusBadRoute);
        }
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int ahead = __popc(peers & ((1u << lane) - 1u));
        __syncthreads();
        if (e < experts && ahead == 0) hist[warp * experts + e] = static_cast<uint16_t>(__popc(peers));
        __syncthreads();
        int64_t chunk_total = 0;
        if (tid < experts) {
            uint16_t run = 0;
            for (int w = 0; w < 32; ++w) {
                const uint16_t c = hist[w * experts + tid];
                hist[w * experts + tid] = run;
                run = static_cast<uint16_t>(run + c);
            }
            chunk_total = run;
        }
        __syncthreads();
        if (e < experts) {
            const int64_t slot = expert_start[e] + base[e] + hist[warp * experts + e] + ahead;
            const int r = e / epr;
            const int64_t row = seg_start[r] + (slot - first[r]);
            src_row[slot] = p / k;
            dst_rank[slot] = r;
            dst_row[slot] = row;
            pull_rank[p] = r;
            pull_row[p] = row;
        } else if (p < n) {
            pull_rank[p] = -1;                                       // the combine skips and reports it
            pull_row[p] = -1;
        }
        __syncthreads();
        if (tid < experts) base[tid] += chunk_total;
        __syncthreads();
    }
}

}  // namespace
}  // namespace cck

// csrc/includes/moe_router.h:20-29 of the reference: same signature and limits (at most 256
// experts, else cudaErrorInvalidValue; nothing launched for num_tokens <= 0).
extern "C" int32_t launch_moe_router_fwd(const void* logits, float* topk_weights, int64_t* topk_indices,
                                         int64_t num_tokens, int64_t num_experts, int64_t k, int32_t dtype,
                                         int32_t renormalize, void* stream) {
    if (num_tokens <= 0) return cudaSuccess;
    if (num_experts <= 0 || num_experts > 256 || k <= 0 || k > num_experts) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run_router<float>(logits, topk_weights, topk_indices, num_tokens, num_experts, k, renormalize, s);
        case cck::kF16:  return cck::run_router<__half>(logits, topk_weights, topk_indices, num_tokens, num_experts, k, renormalize, s);
        case cck::kBF16: return cck::run_router<__nv_bfloat16>(logits, topk_weights, topk_indices, num_tokens, num_experts, k, renormalize, s);
        default:         return cudaErrorInvalidValue;
    }
}

// csrc/includes/token_permute.h:17-24 of the reference.
extern "C" int32_t launch_token_gather_fwd(const void* src, const int64_t* indices, void* dst, int64_t n_dst_rows,
                                           int64_t hidden_dim, int32_t dtype, void* stream) {
    using namespace cck;
    if (n_dst_rows <= 0 || hidden_dim <= 0) return cudaSuccess;
    int64_t elem = 0;
    switch (dtype) {
        case kF32: elem = 4; break;
        case kF16: case kBF16: elem = 2; break;
        default: return cudaErrorInvalidValue;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t row_bytes = hidden_dim * elem;
    const unsigned grid = warp_grid(n_dst_rows);
    if (row_bytes % 16 == 0 && aligned16(src) && aligned16(dst)) {
        token_gather_vec_kernel<<<grid, kGatherThreads, 0, s>>>(static_cast<const Vec16*>(src), indices,
                                                                static_cast<Vec16*>(dst), n_dst_rows, row_bytes / 16);
    } else if (elem == 4) {
        token_gather_scalar_kernel<uint32_t><<<grid, kGatherThreads, 0, s>>>(
            static_cast<const uint32_t*>(src), indices, static_cast<uint32_t*>(dst), n_dst_rows, hidden_dim);
    } else {
        token_gather_scalar_kernel<uint16_t><<<grid, kGatherThreads, 0, s>>>(
            static_cast<const uint16_t*>(src), indices, static_cast<uint16_t*>(dst), n_dst_rows, hidden_dim);
    }
    return cudaGetLastError();
}

// csrc/includes/token_permute.h:32-41 of the reference.
extern "C" int32_t launch_token_combine_fwd(const void* expert_output, const int64_t* unpermute_index,
                                            const float* weights, void* combined, int64_t n_tokens, int64_t k,
                                            int64_t hidden_dim, int32_t dtype, void* stream) {
    if (n_tokens <= 0 || k <= 0 || hidden_dim <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case cck::kF32:  return cck::run_combine<float>(expert_output, unpermute_index, weights, combined, n_tokens, k, hidden_dim, s);
        case cck::kF16:  return cck::run_combine<__half>(expert_output, unpermute_index, weights, combined, n_tokens, k, hidden_dim, s);
        case cck::kBF16: return cck::run_combine<__nv_bfloat16>(expert_output, unpermute_index, weights, combined, n_tokens, k, hidden_dim, s);
        default:         return cudaErrorInvalidValue;
    }
}

// Expert-parallel dispatch: row src[src_row[i]] goes to row dst_row[i] of buffer dst_rank[i] of
// `dst_bases` (a device array of `world` base addresses - this rank's own receive buffer and its
// peers' mapped ones), for i < n.  Rows are `hidden_dim` elements of `dtype`; hidden_dim *
// element size must be a multiple of 16 and every buffer 16-byte aligned.  Routes outside
// [0, world) x [0, capacity_rows) or source rows outside [0, n_src_rows) are skipped and set bit
// 2 of the word `cck_take_device_status` returns.  No reference counterpart.
extern "C" int32_t launch_token_dispatch_fwd(const void* src, const int64_t* src_row, const int64_t* dst_rank,
                                             const int64_t* dst_row, const int64_t* dst_bases, int64_t world,
                                             int64_t capacity_rows, int64_t n_src_rows, int64_t n, int64_t hidden_dim,
                                             int32_t dtype, void* stream) {
    using namespace cck;
    if (n <= 0 || hidden_dim <= 0) return cudaSuccess;
    const int64_t elem = dtype == kF32 ? 4 : ((dtype == kF16 || dtype == kBF16) ? 2 : 0);
    if (elem == 0 || world <= 0 || world > 1024 || (hidden_dim * elem) % 16 != 0 || !aligned16(src)) return cudaErrorInvalidValue;
    unsigned int* st = cck::tc::status_word();
    if (!st) return cudaErrorMemoryAllocation;
    token_dispatch_kernel<<<warp_grid(n), kGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const Vec16*>(src), src_row, dst_rank, dst_row, dst_bases, static_cast<int>(world), capacity_rows,
        n_src_rows, n, hidden_dim * elem / 16, st);
    return cudaGetLastError();
}

// Expert-parallel combine: combined[t] = sum_j weights[t, j] * row src_row[t, j] of buffer
// src_rank[t, j] of `src_bases`, fp32 accumulation, one rounding.  Same checks as the dispatch.
extern "C" int32_t launch_token_combine_remote_fwd(const int64_t* src_bases, int64_t world, int64_t capacity_rows,
                                                   const int64_t* src_rank, const int64_t* src_row, const float* weights,
                                                   void* combined, int64_t n_tokens, int64_t k, int64_t hidden_dim,
                                                   int32_t dtype, void* stream) {
    using namespace cck;
    if (n_tokens <= 0 || k <= 0 || hidden_dim <= 0) return cudaSuccess;
    if (world <= 0 || world > 1024 || k > 0x7fffffffLL || !aligned16(combined)) return cudaErrorInvalidValue;
    unsigned int* st = cck::tc::status_word();
    if (!st) return cudaErrorMemoryAllocation;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = warp_grid(n_tokens);
    switch (dtype) {
        case kF32:
            if (hidden_dim % 4) return cudaErrorInvalidValue;
            token_combine_remote_kernel<float><<<grid, kCombineMaxThreads, 0, s>>>(
                src_bases, static_cast<int>(world), capacity_rows, src_rank, src_row, weights, static_cast<float*>(combined),
                n_tokens, static_cast<int>(k), hidden_dim / 4, st);
            break;
        case kF16:
            if (hidden_dim % 8) return cudaErrorInvalidValue;
            token_combine_remote_kernel<__half><<<grid, kCombineMaxThreads, 0, s>>>(
                src_bases, static_cast<int>(world), capacity_rows, src_rank, src_row, weights, static_cast<__half*>(combined),
                n_tokens, static_cast<int>(k), hidden_dim / 8, st);
            break;
        case kBF16:
            if (hidden_dim % 8) return cudaErrorInvalidValue;
            token_combine_remote_kernel<__nv_bfloat16><<<grid, kCombineMaxThreads, 0, s>>>(
                src_bases, static_cast<int>(world), capacity_rows, src_rank, src_row, weights,
                static_cast<__nv_bfloat16*>(combined), n_tokens, static_cast<int>(k), hidden_dim / 8, st);
            break;
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// The plan of one expert-parallel call (see ep_plan_kernel): topk = this rank's [n] flattened
// expert ids (n = tokens x k), counts = [world, experts] all-gathered per-expert counts.
// Outputs, all int64: src_row / dst_rank / dst_row [n] in expert-sorted slot order (the
// arguments of launch_token_dispatch_fwd), pull_rank / pull_row [n] in (token, choice) order
// (the arguments of launch_token_combine_remote_fwd), meta[2] = {rows this rank receives, most
// rows any rank receives}.  experts <= 256, world <= 32, experts % world == 0.  An id outside
// [0, experts) sets bit 2 of the status word and gets the route (-1, -1), which the movers skip;
// src_row / dst_* are then not fully written (zero them first if that can happen).
extern "C" int32_t launch_ep_plan(const int64_t* topk, const int64_t* counts, int64_t n, int64_t k, int64_t world,
                                  int64_t experts, int64_t rank, int64_t* src_row, int64_t* dst_rank, int64_t* dst_row,
                                  int64_t* pull_rank, int64_t* pull_row, int64_t* meta, void* stream) {
    using namespace cck;
    if (n < 0 || k <= 0 || world <= 0 || world > kPlanMaxWorld || experts <= 0 || experts > kPlanMaxExperts ||
        experts % world != 0 || rank < 0 || rank >= world)
        return cudaErrorInvalidValue;
    unsigned int* st = cck::tc::status_word();
    if (!st) return cudaErrorMemoryAllocation;
    ep_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        topk, counts, n, static_cast<int>(k), static_cast<int>(world), static_cast<int>(experts), static_cast<int>(rank),
        src_row, dst_rank, dst_row, pull_rank, pull_row, meta, st);
    return cudaGetLastError();
}
