// y = x @ weight^T + bias   (x [M,K], weight [N,K], bias [N] or null, y [M,N])
//
// Replaces the reference's csrc/kernels/matmul_add_bias.cu:53-222, a CUDA-core
// shared-memory GEMM.  Here f16/bf16 problems run on the 5th-generation tensor
// cores: TMA-fed, tcgen05.mma into TMEM, fp32 accumulation, bias added in fp32
// in the epilogue and one rounding to the storage type (gemm_tcgen05.cuh).
// An FP8 entry point (e4m3 operands, per-token and per-channel scales folded
// into the epilogue) has no counterpart in the reference.
// fp32 inputs, shapes TMA cannot address (K not a multiple of 8 elements) and
// problems below ~4 MFLOP use the CUDA-core kernel in gemm_simt.cuh.
//
// Tensor-bound: 2*M*N*K flops per launch.
#include <type_traits>

#include "gemm_simt.cuh"
#include "gemm_decode.cuh"
#include "gemm_splitk.cuh"

namespace cck {
namespace tc {

// Per-device status block (layout in ptx.cuh): error bits in the first word, the wait limit
// of the bounded mbarrier waits in bytes 8..15.
__device__ __align__(16) unsigned long long g_status_block[2] = {0ull, ptx::kDefaultWaitLimitNs};

// Address of the current device's status block.  The per-device cache is filled without a lock:
// two host threads making the first call on one device both store the same address.
unsigned int* status_word() {
    static unsigned int* ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_block) != cudaSuccess) return nullptr;
        ptr[dev] = static_cast<unsigned int*>(p);
    }
    return ptr[dev];
}

// ---- epilogue: + bias, round once, store
template <typename T>
struct EpiBias {
    struct Params {
        const T* bias;
        T* y;
        int64_t m, n;
        int vec_ok;     // rows of y start 16-byte aligned
    };
    struct Thread {};
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread&, const TileWork& w, float* scratch,
                                                      int lane, int) {
        const int64_t n0 = w.n0;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            scratch[lane + 32 * i] = (p.bias != nullptr && col < p.n) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread&, const TileWork& w, int row_in_tile,
                                                 int c0, float (&acc)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n0) + c0;
        if (row >= p.m || col >= p.n) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] += scratch[c0 + j];
        T* out = p.y + row * p.n + col;
        if (p.vec_ok && col + 32 <= p.n) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                Vec16 o;
#pragma unroll
                for (int q = 0; q < 4; ++q) o.w[q] = Store<T>::pack2(acc[8 * v + 2 * q], acc[8 * v + 2 * q + 1]);
                st_stream(out + 8 * v, o);
            }
        } else {
            for (int j = 0; j < 32 && col + j < p.n; ++j) Store<T>::store1(out + j, acc[j]);
        }
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// ---- epilogue: acc * a_scale[row] * w_scale[col] + bias, round once, store
template <typename T>
struct EpiScaledBias {
    struct Params {
        const float* a_scale;   // [M]
        const float* w_scale;   // [N]
        const T* bias;          // [N] or null
        T* y;
        int64_t m, n;
        int vec_ok;
    };
    struct Thread { float a_scale; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int row_in_tile) {
        const int64_t n0 = w.n0;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            const bool in = col < p.n;
            scratch[lane + 32 * i] = in ? p.w_scale[col] : 0.0f;
            scratch[kBN + lane + 32 * i] = (in && p.bias != nullptr) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        th.a_scale = row < p.m ? p.a_scale[row] : 0.0f;
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int row_in_tile,
                                                 int c0, float (&acc)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n0) + c0;
        if (row >= p.m || col >= p.n) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(acc[j] * th.a_scale, scratch[c0 + j], scratch[kBN + c0 + j]);
        T* out = p.y + row * p.n + col;
        if (p.vec_ok && col + 32 <= p.n) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                Vec16 o;
#pragma unroll
                for (int q = 0; q < 4; ++q) o.w[q] = Store<T>::pack2(acc[8 * v + 2 * q], acc[8 * v + 2 * q + 1]);
                st_stream(out + 8 * v, o);
            }
        } else {
            for (int j = 0; j < 32 && col + j < p.n; ++j) Store<T>::store1(out + j, acc[j]);
        }
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

template <typename T>
bool tc_applicable(const void* x, const void* w, int64_t m, int64_t k, int64_t n) {
    // rows must be 16-byte multiples for TMA; partial and even undersized tiles are fine (TMA
    // zero-fills outside the matrix, the epilogue masks), but below ~4 MFLOP the CUDA-core
    // kernel is as fast and skips building two tensor maps
    return k % 8 == 0 && aligned16(x) && aligned16(w) && 2 * m * n * k >= (1LL << 22) &&
           m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31);
}

template <typename T>
cudaError_t gemm_tc(const void* x, const void* w, const void* bias, void* y, int64_t m, int64_t k, int64_t n,
                    cudaStream_t s) {
    constexpr bool is_bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int m_tiles = static_cast<int>(ceil_div64(m, kBM)), n_tiles = static_cast<int>(ceil_div64(n, kBN));
    typename EpiBias<T>::Params ep{static_cast<const T*>(bias), static_cast<T*>(y), m, n,
                                   (n % 8 == 0 && aligned16(y)) ? 1 : 0};
    const uint32_t fmt = is_bf16 ? 1u : 0u;
    // Decode-sized batches: the weight rows take the M side of the instruction, the tokens the N
    // side, K split over a cluster (gemm_decode.cuh).
    if (m <= kDecMaxTokens && splitk_enabled(m))
        return launch_decode<T>(x, w, static_cast<const T*>(bias), static_cast<T*>(y), m, k, n, dt, fmt, s);
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 2, x, m, k, kBM);
    if (e != cudaSuccess) return e;
    // Too few full-width tiles to occupy the machine (small M, decode-sized batches): 128 x 64 tiles,
    // and while even those leave SMs idle, a cluster of 2-8 CTAs per tile that splits K
    // (gemm_splitk.cuh).  Measured on B200, K = N = 4096, device time per call: M = 128 full-width
    // 29 us, narrow 20 us; M = 256 26 / 21; from M = 512 on the full-width tiles win again.
    constexpr int kNarrow = 64;
    const int64_t wide_tiles = static_cast<int64_t>(m_tiles) * n_tiles;
    if (wide_tiles <= sm_count() / 2 && narrow_tiles_enabled()) {
        const int n_narrow = static_cast<int>(ceil_div64(n, kNarrow));
        const int splits = splitk_enabled(m) ? splitk_factor(static_cast<int64_t>(m_tiles) * n_narrow,
                                                            static_cast<int>(ceil_div64(k, 64))) : 1;
        if (splits > 1 || wide_tiles <= sm_count() / 4) {
            e = make_tmap(&tb, dt, 2, w, n, k, kNarrow);
            if (e != cudaSuccess) return e;
            const uint32_t idesc = ptx::instr_desc(fmt, fmt, kBM, kNarrow);
            if (splits > 1)
                return launch_splitk<T>(ta, tb, ep.bias, ep.y, m, n, m_tiles, n_narrow, k, idesc, ep.vec_ok, splits, s);
            SchedGemm::Params sp{m_tiles, n_narrow, m_tiles};
            const int64_t tiles = static_cast<int64_t>(sp.m_tiles) * sp.n_tiles;
            return launch<false, SchedGemm, EpiBias<T>, kNarrow>(ta, tb, sp, ep, k, idesc,
                                                                 static_cast<int>(tiles < sm_count() ? tiles : sm_count()), s);
        }
    }
    const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<false, SchedGemm, EpiBias<T>>() > 0;
    e = make_tmap(&tb, dt, 2, w, n, k, pair ? 128 : kBN);     // a CTA of a pair loads half of the B tile
    if (e != cudaSuccess) return e;
    if (pair) {
        const int m_pairs = (m_tiles + 1) / 2;
        SchedGemm::Params sp{m_pairs, n_tiles, raster_group(2 * kBM, k, 2, m_pairs)};
        return launch_pair<false, SchedGemm, EpiBias<T>>(ta, tb, sp, ep, k, ptx::instr_desc(fmt, fmt, 2 * kBM, kBN),
                                                         static_cast<int64_t>(sp.m_tiles) * sp.n_tiles, s);
    }
    SchedGemm::Params sp{m_tiles, n_tiles, raster_group(kBM, k, 2, m_tiles)};
    const int64_t tiles = static_cast<int64_t>(sp.m_tiles) * sp.n_tiles;
    const int ctas = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    return launch<false, SchedGemm, EpiBias<T>>(ta, tb, sp, ep, k, ptx::instr_desc(fmt, fmt, kBM, kBN), ctas, s);
}

}  // namespace tc
}  // namespace cck

extern "C" int32_t launch_matmul_add_bias_fwd(const void* x, const void* weight, const void* bias, void* y,
                                              int64_t m, int64_t k, int64_t n, int32_t dtype, void* stream) {
    using namespace cck;
    if (m <= 0 || n <= 0 || k <= 0) return cudaSuccess;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case kF32:
            return gemm_simt<float>(x, weight, bias, y, m, k, n, s);
        case kF16:
            return tc::tc_applicable<__half>(x, weight, m, k, n) ? tc::gemm_tc<__half>(x, weight, bias, y, m, k, n, s)
                                                                 : gemm_simt<__half>(x, weight, bias, y, m, k, n, s);
        case kBF16:
            return tc::tc_applicable<__nv_bfloat16>(x, weight, m, k, n)
                       ? tc::gemm_tc<__nv_bfloat16>(x, weight, bias, y, m, k, n, s)
                       : gemm_simt<__nv_bfloat16>(x, weight, bias, y, m, k, n, s);
        default:
            return cudaErrorInvalidValue;
    }
}

namespace cck {
namespace tc {

// FP8 GEMM on the tensor cores for any M and N (K a multiple of 16, 16-byte aligned operands):
// TMA zero-fills outside the matrices and the epilogue masks, so partial and undersized tiles
// need nothing special; few full-width tiles (decode-sized M) run on 128 x 64 tiles like the
// 16-bit path.
template <typename T>
cudaError_t gemm_fp8_tc(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_codes, const float* w_scale,
                        const void* bias, void* y, int64_t m, int64_t k, int64_t n, cudaStream_t s) {
    const int m_tiles = static_cast<int>(ceil_div64(m, kBM)), n_tiles = static_cast<int>(ceil_div64(n, kBN));
    typename EpiScaledBias<T>::Params ep{a_scale, w_scale, static_cast<const T*>(bias), static_cast<T*>(y), m, n,
                                         (n % 8 == 0 && aligned16(y)) ? 1 : 0};
    const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 1, a_codes, m, k, kBM);
    if (e != cudaSuccess) return e;
    constexpr int kNarrow = 64;
    const int64_t wide_tiles = static_cast<int64_t>(m_tiles) * n_tiles;
    if (wide_tiles <= sm_count() / 4 && narrow_tiles_enabled()) {
        e = make_tmap(&tb, dt, 1, w_codes, n, k, kNarrow);
        if (e != cudaSuccess) return e;
        SchedGemm::Params sp{m_tiles, static_cast<int>(ceil_div64(n, kNarrow)), m_tiles};
        const int64_t tiles = static_cast<int64_t>(sp.m_tiles) * sp.n_tiles;
        return launch<true, SchedGemm, EpiScaledBias<T>, kNarrow>(ta, tb, sp, ep, k, ptx::instr_desc(0u, 0u, kBM, kNarrow),
                                                                  static_cast<int>(tiles < sm_count() ? tiles : sm_count()), s);
    }
    const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<true, SchedGemm, EpiScaledBias<T>>() > 0;
    e = make_tmap(&tb, dt, 1, w_codes, n, k, pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    const int m_units = pair ? (m_tiles + 1) / 2 : m_tiles;
    SchedGemm::Params sp{m_units, n_tiles, raster_group(pair ? 2 * kBM : kBM, k, 1, m_units)};
    const int64_t tiles = static_cast<int64_t>(sp.m_tiles) * sp.n_tiles;
    const uint32_t idesc = ptx::instr_desc(0u, 0u, pair ? 2 * kBM : kBM, kBN);   // e4m3 x e4m3
    if (pair) return launch_pair<true, SchedGemm, EpiScaledBias<T>>(ta, tb, sp, ep, k, idesc, tiles, s);
    return launch<true, SchedGemm, EpiScaledBias<T>>(ta, tb, sp, ep, k, idesc,
                                                     static_cast<int>(tiles < sm_count() ? tiles : sm_count()), s);
}

}  // namespace tc
}  // namespace cck

// e4m3 operands with per-row scales.  Every shape runs, as with the 16-bit entry point (the
// reference's launcher has a fallback for every shape: csrc/kernels/matmul_add_bias.cu:170-180):
// K a multiple of 16 with 16-byte aligned operands and at least ~4 MFLOP go to the tensor
// cores, everything else to the CUDA-core kernel.
extern "C" int32_t launch_matmul_add_bias_fp8_fwd(const uint8_t* a_codes, const float* a_scale,
                                                  const uint8_t* w_codes, const float* w_scale, const void* bias,
                                                  void* y, int64_t m, int64_t k, int64_t n, int32_t out_dtype,
                                                  void* stream) {
    using namespace cck;
    if (m <= 0 || n <= 0 || k <= 0) return cudaSuccess;
    if (out_dtype != kBF16 && out_dtype != kF16) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = out_dtype == kBF16;
    const bool tensor_cores = k % 16 == 0 && aligned16(a_codes) && aligned16(w_codes) && 2 * m * n * k >= (1LL << 22) &&
                              m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31);
    if (tensor_cores)
        return bf ? tc::gemm_fp8_tc<__nv_bfloat16>(a_codes, a_scale, w_codes, w_scale, bias, y, m, k, n, s)
                  : tc::gemm_fp8_tc<__half>(a_codes, a_scale, w_codes, w_scale, bias, y, m, k, n, s);
    return bf ? gemm_fp8_simt<__nv_bfloat16>(a_codes, a_scale, w_codes, w_scale, bias, y, m, k, n, s)
              : gemm_fp8_simt<__half>(a_codes, a_scale, w_codes, w_scale, bias, y, m, k, n, s);
}

// Number of CTA pairs the bf16 GEMM can keep resident on the current device (0: the pair
// kernel is unavailable or disabled and every GEMM runs on the single-CTA kernel).
extern "C" int32_t cck_gemm_pair_capacity(void) {
    using namespace cck::tc;
    if (!pair_kernels_enabled()) return 0;
    return max_pairs<false, SchedGemm, EpiBias<__nv_bfloat16>>();
}

// Returns the tensor-core kernels' error word of the current device and clears
// it (bit 0: a bounded wait ran out).  Synchronises the device.
extern "C" int32_t cck_take_device_status(uint32_t* out) {
    unsigned int* st = cck::tc::status_word();
    if (!st || !out) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    unsigned int v = 0, zero = 0;
    e = cudaMemcpy(&v, st, sizeof(v), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    *out = v;
    return cudaMemcpy(st, &zero, sizeof(zero), cudaMemcpyHostToDevice);
}

// Sets the limit of every bounded device-side wait on the current device (nanoseconds, clamped
// to [1 us, 10 s]; the library starts with 2 s) and returns the previous one in *previous_ns
// (may be null).  Synchronises the device: kernels in flight keep the limit they started with.
extern "C" int32_t cck_set_wait_limit_ns(uint64_t limit_ns, uint64_t* previous_ns) {
    unsigned int* st = cck::tc::status_word();
    if (!st) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    unsigned long long old = 0, now = limit_ns < 1000ull ? 1000ull : (limit_ns > 10000000000ull ? 10000000000ull : limit_ns);
    e = cudaMemcpy(&old, st + 2, sizeof(old), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (previous_ns) *previous_ns = old;
    return cudaMemcpy(st + 2, &now, sizeof(now), cudaMemcpyHostToDevice);
}

// Self-test of the give-up path of the tensor-core kernels: one launch of a real GEMM kernel on
// ONE tile whose A tensor map is built with a 64-row box where the kernel counts on 128 rows of
// bytes, so the "stage full" mbarrier never completes and no MMA is ever issued.  The waiting
// roles run into the wait limit, raise the CTA's abort flag, the CTA waits for its copies in
// flight, frees its tensor memory, sets bit 0 of the status word and returns - no fault, no
// hang, the context stays usable.  Set a short limit (cck_set_wait_limit_ns, ~1 ms) first.
//   a [256, 64], b [256, 64] bf16 (row-major), y [256, 256] bf16 (left unwritten)
//   variant 0: gemm_kernel (one CTA)   1: gemm_pair_kernel (one CTA pair)   2: gemm_splitk_kernel (cluster of 2)
extern "C" int32_t launch_wait_limit_selftest(const void* a, const void* b, void* y, int32_t variant, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    using T = __nv_bfloat16;
    if (!a || !b || !y || !aligned16(a) || !aligned16(b) || !aligned16(y)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int64_t rows = 256, k = variant == 2 ? 128 : 64;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 2, a, variant == 2 ? 128 : rows, k, 64 /* the kernels expect kBM = 128 */);
    if (e != cudaSuccess) return e;
    EpiBias<T>::Params ep{nullptr, static_cast<T*>(y), rows, 256, 1};
    SchedGemm::Params sp{1, 1, 1};
    switch (variant) {
        case 0:
            e = make_tmap(&tb, dt, 2, b, rows, k, kBN);
            if (e != cudaSuccess) return e;
            return launch<false, SchedGemm, EpiBias<T>>(ta, tb, sp, ep, k, ptx::instr_desc(1u, 1u, kBM, kBN), 1, s);
        case 1:
            if (max_pairs<false, SchedGemm, EpiBias<T>>() <= 0) return cudaErrorNotSupported;
            e = make_tmap(&tb, dt, 2, b, rows, k, 128);
            if (e != cudaSuccess) return e;
            return launch_pair<false, SchedGemm, EpiBias<T>>(ta, tb, sp, ep, k, ptx::instr_desc(1u, 1u, 2 * kBM, kBN), 1, s);
        case 2:
            e = make_tmap(&tb, dt, 2, b, 128, k, 64);
            if (e != cudaSuccess) return e;
            return launch_splitk<T>(ta, tb, nullptr, static_cast<T*>(y), 128, 64, 1, 1, k, ptx::instr_desc(1u, 1u, kBM, 64),
                                    1, 2, s);
        default:
            return cudaErrorInvalidValue;
    }
}
