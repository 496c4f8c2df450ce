// Fused linear + cross entropy: per-row softmax statistics of
//   logits = hidden [N,H] @ weight[v0:v1, H]^T
// without ever writing the logits to memory.
//
// Replaces the reference's Python chunk loop (custom_cuda/kernels/
// linear_cross_entropy.py:56-67: one cuBLAS GEMM per 4096-column chunk, the
// chunk written to HBM and read twice by csrc/kernels/linear_cross_entropy.cu:
// 29-75).  Here the tcgen05 mainloop of gemm_tcgen05.cuh leaves each 128x256
// logits tile in TMEM and the epilogue folds it straight into running per-row
// (max, sum of exp, target logit) registers - one thread owns one row, so the
// online softmax needs no cross-thread traffic.  The logits stay fp32 (the
// reference rounds them to bf16 first).
//
// Work decomposition: the vocabulary tiles are cut into `splits` contiguous
// ranges; a unit = (row tile, split); units are dealt round-robin to the persistent
// CTAs (or CTA pairs) in groups of row tiles (grouped_unit in gemm_tcgen05.cuh) so
// that the workers running at the same time share a few hidden-state panels and a
// few weight ranges that fit the L2 together.  Each unit writes one partial triple per
// row into the caller's workspace [splits][3][N]; lce_merge_kernel reduces them
// to row_stats [3][N] for this vocabulary slice.  A vocabulary-sharded run
// all-gathers row_stats across ranks and calls launch_lce_finalize on the stack.
//
// Tensor-bound: 2*N*H*V flops per launch.
#include <type_traits>

#include "gemm_tcgen05.cuh"

namespace cck {
namespace tc {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__host__ __device__ inline int split_begin(int split, int splits, int n_tiles) {
    return static_cast<int>((static_cast<int64_t>(split) * n_tiles) / splits);
}

struct SchedLce {
    struct Params { int m_tiles, n_tiles, splits, group; };
    struct Iter {
        Params p;
        int unit, step, units, nt, nt_end, nt_begin, split, m_tile;
        __device__ Iter(const Params& q, int worker, int workers)
            : p(q), unit(worker - workers), step(workers), units(q.m_tiles * q.splits),
              nt(0), nt_end(0), nt_begin(0), split(0), m_tile(0) {}
        __device__ bool next(TileWork& w) {
            while (nt >= nt_end) {
                unit += step;
                if (unit >= units) return false;
                grouped_unit(unit, p.m_tiles, p.splits, p.group, m_tile, split);
                nt_begin = nt = split_begin(split, p.splits, p.n_tiles);
                nt_end = split_begin(split + 1, p.splits, p.n_tiles);
            }
            w.m_tile = m_tile;
            w.n_tile = nt;
            w.split = split;
            w.first = nt == nt_begin;
            w.last = nt + 1 == nt_end;
            ++nt;
            return true;
        }
    };
};

struct EpiLce {
    struct Params {
        const int64_t* targets;   // [N] global class ids (or ignore_index)
        float* partials;          // [splits][3][N]
        int64_t n_rows;
        int64_t v_count;          // rows of this weight slice
        int64_t v_start;          // global id of the slice's first row
    };
    struct Thread {
        float mx, sm, tg;
        int64_t tgt_local;
    };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float*, int,
                                                      int row_in_tile) {
        if (w.first) {
            th.mx = -INFINITY;
            th.sm = 0.0f;
            th.tg = 0.0f;
            const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
            th.tgt_local = row < p.n_rows ? p.targets[row] - p.v_start : -1;
        }
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int, int c0,
                                                 float (&acc)[32], const float*) {
        const int64_t col0 = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (col0 >= p.v_count) return;
        const int valid = p.v_count - col0 < 32 ? static_cast<int>(p.v_count - col0) : 32;
        const int64_t t_off = th.tgt_local - col0;
        if (t_off >= 0 && t_off < valid) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j == t_off) th.tg = acc[j];
        }
        float cmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (j >= valid) acc[j] = -INFINITY;
            cmax = fmaxf(cmax, acc[j]);
        }
        const float new_max = fmaxf(th.mx, cmax);
        const float shift = new_max * kLog2e;
        float add = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) add += ex2_approx(fmaf(acc[j], kLog2e, -shift));
        th.sm = fmaf(th.sm, ex2_approx((th.mx - new_max) * kLog2e), add);
        th.mx = new_max;
    }
    __device__ static __forceinline__ void tile_end(const Params& p, Thread& th, const TileWork& w, int row_in_tile) {
        if (!w.last) return;
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        if (row >= p.n_rows) return;
        float* base = p.partials + static_cast<int64_t>(w.split) * 3 * p.n_rows + row;
        base[0] = th.mx;
        base[p.n_rows] = th.sm;
        base[2 * p.n_rows] = th.tg;
    }
};

// ---- backward helper: d(loss)/d(logits) for a block of rows, written in the storage type.
//   dl[i, j] = (exp(l_ij - lse_i) - [j == target_i]) * grad_scale   (0 for ignored rows)
// The logits tile is recomputed by the same mainloop and turned into its gradient in the
// epilogue; the caller then forms d_hidden = dl @ W and d_weight += dl^T @ hidden with the GEMM.
template <typename T>
struct EpiDlogits {
    struct Params {
        const int64_t* targets;   // [n]
        const float* lse;         // [n] log-sum-exp of each row's logits (from the forward statistics)
        T* dl;                    // [n, v]
        int64_t n, v;
        int64_t ignore_index;
        float grad_scale;
        int vec_ok;
    };
    struct Thread {
        float neg_lse2;           // -lse * log2(e)
        float scale;              // grad_scale, or 0 for an ignored row
        int64_t target;
    };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float*, int,
                                                      int row_in_tile) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        th.target = -1;
        th.scale = 0.0f;
        th.neg_lse2 = 0.0f;
        if (row < p.n) {
            th.target = p.targets[row];
            th.scale = th.target == p.ignore_index ? 0.0f : p.grad_scale;
            th.neg_lse2 = -p.lse[row] * kLog2e;
        }
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float*) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.n || col >= p.v) return;
        const int64_t t_off = th.target - col;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float prob = ex2_approx(fmaf(acc[j], kLog2e, th.neg_lse2));
            acc[j] = (prob - (j == t_off ? 1.0f : 0.0f)) * th.scale;
        }
        T* out = p.dl + row * p.v + col;
        if (p.vec_ok && col + 32 <= p.v) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                Vec16 o;
#pragma unroll
                for (int i = 0; i < 4; ++i) o.w[i] = Store<T>::pack2(acc[8 * q + 2 * i], acc[8 * q + 2 * i + 1]);
                st_stream(out + 8 * q, o);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < p.v) Store<T>::store1(out + j, acc[j]);
        }
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// partials [splits][3][N] -> row_stats [3][N]
__global__ void __launch_bounds__(256)
lce_merge_kernel(const float* __restrict__ partials, int splits, int64_t n, float* __restrict__ row_stats) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (row >= n) return;
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, partials[(static_cast<int64_t>(s) * 3) * n + row]);
    float sm = 0.0f, tg = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float* b = partials + (static_cast<int64_t>(s) * 3) * n + row;
        sm += b[n] * expf(b[0] - mx);
        tg += b[2 * n];
    }
    row_stats[row] = mx;
    row_stats[n + row] = sm;
    row_stats[2 * n + row] = tg;
}

// stats [shards][3][N] -> per-row loss (0 for ignored rows) and {sum of losses, number of valid rows}
__global__ void __launch_bounds__(1024)
lce_finalize_kernel(const float* __restrict__ stats, const int64_t* __restrict__ targets, int64_t n, int shards,
                    int64_t ignore_index, float* __restrict__ loss_rows, float* __restrict__ reduce_out) {
    __shared__ double sum_slots[32];
    __shared__ double cnt_slots[32];
    double acc = 0.0, cnt = 0.0;
    for (int64_t row = threadIdx.x; row < n; row += 1024) {
        float mx = -INFINITY;
        for (int g = 0; g < shards; ++g) mx = fmaxf(mx, stats[(static_cast<int64_t>(g) * 3) * n + row]);
        float sm = 0.0f, tg = 0.0f;
        for (int g = 0; g < shards; ++g) {
            const float* b = stats + (static_cast<int64_t>(g) * 3) * n + row;
            sm += b[n] * expf(b[0] - mx);
            tg += b[2 * n];
        }
        const bool valid = targets[row] != ignore_index;
        const float loss = valid ? (mx + logf(sm) - tg) : 0.0f;
        if (loss_rows) loss_rows[row] = loss;
        acc += static_cast<double>(loss);
        cnt += valid ? 1.0 : 0.0;
    }
    for (int o = 16; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
        cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    }
    if ((threadIdx.x & 31) == 0) {
        sum_slots[threadIdx.x >> 5] = acc;
        cnt_slots[threadIdx.x >> 5] = cnt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, c = 0.0;
        for (int i = 0; i < 32; ++i) {
            a += sum_slots[i];
            c += cnt_slots[i];
        }
        reduce_out[0] = static_cast<float>(a);
        reduce_out[1] = static_cast<float>(c);
    }
}

// Number of vocabulary splits: minimise the makespan of the round-robin unit
// assignment, ceil(units / ctas) * ceil(n_tiles / splits), over 1..64 splits.
inline int choose_splits(int m_tiles, int n_tiles, int ctas) {
    int best = 1;
    int64_t best_cost = -1;
    const int cap = n_tiles < 64 ? n_tiles : 64;
    for (int s = 1; s <= cap; ++s) {
        const int64_t units = static_cast<int64_t>(s) * m_tiles;
        const int64_t cost = ceil_div64(units, ctas) * ceil_div64(n_tiles, s);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

}  // namespace tc
}  // namespace cck

namespace cck {
namespace tc {
// How one launch is laid out: CTA pairs (256-row units) when the problem has at least two
// row tiles and pairs can be scheduled, else single CTAs (128-row units).
struct LcePlan {
    bool pair;
    int m_units, n_tiles, splits, workers;
};
inline LcePlan lce_plan(int64_t n, int64_t v_count) {
    LcePlan p;
    const int m_tiles = static_cast<int>(ceil_div64(n, kBM));
    p.n_tiles = static_cast<int>(ceil_div64(v_count, kBN));
    const int pairs = (m_tiles >= 2 && pair_kernels_enabled()) ? max_pairs<false, SchedLce, EpiLce>() : 0;
    p.pair = pairs > 0;
    p.m_units = p.pair ? (m_tiles + 1) / 2 : m_tiles;
    p.workers = p.pair ? pairs : sm_count();
    p.splits = choose_splits(p.m_units, p.n_tiles, p.workers);
    return p;
}
}  // namespace tc
}  // namespace cck

extern "C" int64_t cck_lce_num_splits(int64_t n, int64_t v_count) {
    if (n <= 0 || v_count <= 0) return 1;
    return cck::tc::lce_plan(n, v_count).splits;
}

extern "C" int64_t cck_lce_workspace_bytes(int64_t n, int64_t v_count) {
    if (n <= 0 || v_count <= 0) return 0;
    return cck_lce_num_splits(n, v_count) * 3 * n * static_cast<int64_t>(sizeof(float));
}

extern "C" int32_t launch_linear_cross_entropy_fwd(const void* hidden, const void* weight, const int64_t* targets,
                                                   int64_t v_start, int64_t n, int64_t h, int64_t v_count,
                                                   float* row_stats, void* workspace, int64_t workspace_bytes,
                                                   int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (n <= 0 || v_count <= 0 || h <= 0) return cudaSuccess;
    if (dtype != kBF16 && dtype != kF16) return cudaErrorInvalidValue;
    if (h % 8 != 0 || !aligned16(hidden) || !aligned16(weight) || n >= (1LL << 31) || v_count >= (1LL << 31) ||
        h >= (1LL << 31))
        return cudaErrorInvalidValue;
    const LcePlan plan = lce_plan(n, v_count);
    if (workspace == nullptr || workspace_bytes < static_cast<int64_t>(plan.splits) * 3 * n * 4) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool is_bf16 = dtype == kBF16;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 2, hidden, n, h, kBM);
    if (e != cudaSuccess) return e;
    e = make_tmap(&tb, dt, 2, weight, v_count, h, plan.pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    SchedLce::Params sp{plan.m_units, plan.n_tiles, plan.splits,
                        raster_group(plan.pair ? 2 * kBM : kBM, h, 2, plan.m_units)};
    EpiLce::Params ep{targets, static_cast<float*>(workspace), n, v_count, v_start};
    const int64_t units = static_cast<int64_t>(plan.m_units) * plan.splits;
    const uint32_t fmt = is_bf16 ? 1u : 0u;
    if (plan.pair) {
        e = launch_pair<false, SchedLce, EpiLce>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, 2 * kBM, kBN), units, s);
    } else {
        const int ctas = static_cast<int>(units < plan.workers ? units : plan.workers);
        e = launch<false, SchedLce, EpiLce>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, kBM, kBN), ctas, s);
    }
    if (e != cudaSuccess) return e;
    lce_merge_kernel<<<static_cast<unsigned>(ceil_div64(n, 256)), 256, 0, s>>>(
        static_cast<const float*>(workspace), plan.splits, n, row_stats);
    return cudaGetLastError();
}

extern "C" int32_t launch_lce_finalize(const float* stats, const int64_t* targets, int64_t n, int64_t n_shards,
                                       int64_t ignore_index, float* loss_rows, float* reduce_out, void* stream) {
    if (n_shards <= 0 || reduce_out == nullptr) return cudaErrorInvalidValue;
    cck::tc::lce_finalize_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        stats, targets, n, static_cast<int>(n_shards), ignore_index, loss_rows, reduce_out);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ variant that allocates nothing
// Some hosts cannot hand this library a workspace: an inference server whose
// memory pool already owns every byte of device memory, or a latency-critical
// loop that must not call cudaMalloc (it synchronises the whole device).  For
// them the per-split partial statistics live in this fixed array instead, which
// every GPU that loads the library holds until the process exits.
namespace {
constexpr int64_t kNoAllocScratchBytes = 6ll << 20;   // 6 MiB: e.g. 8192 rows x 64 splits
static __device__ __align__(256) float g_lce_noalloc_scratch[kNoAllocScratchBytes / sizeof(float)];

// In host code the array's name only stands for the symbol; its device address has
// to be asked for, once per device, with that device current.
float* noalloc_scratch_ptr(cudaError_t* err) {
    static float* ptr[64] = {};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    if (!ptr[dev]) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_lce_noalloc_scratch);
        if (*err != cudaSuccess) return nullptr;
        ptr[dev] = static_cast<float*>(p);
    }
    return ptr[dev];
}
}  // namespace

extern "C" int64_t cck_lce_noalloc_max_workspace_bytes(void) { return kNoAllocScratchBytes; }

// Same computation and same result as launch_linear_cross_entropy_fwd, but the
// workspace is the library's own fixed 6 MiB device array, so the call makes no
// cudaMalloc / cudaFree and needs no workspace argument.
//   * Problems whose workspace need, cck_lce_workspace_bytes(n, v_count), exceeds
//     cck_lce_noalloc_max_workspace_bytes() are refused with cudaErrorInvalidValue
//     before anything is launched.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress); make that first call outside any stream capture.
//   * All calls on a device share the one array.  Nothing in it has to start at
//     zero - every partial that is read has been written by the same call - but two
//     calls that overlap on the GPU (different streams) race on it: serialise them.
extern "C" int32_t launch_linear_cross_entropy_fwd_noalloc(const void* hidden, const void* weight,
                                                           const int64_t* targets, int64_t v_start, int64_t n,
                                                           int64_t h, int64_t v_count, float* row_stats,
                                                           int32_t dtype, void* stream) {
    if (n <= 0 || v_count <= 0 || h <= 0) return cudaSuccess;
    if (cck_lce_workspace_bytes(n, v_count) > kNoAllocScratchBytes) return cudaErrorInvalidValue;
    cudaError_t err = cudaSuccess;
    float* scratch = noalloc_scratch_ptr(&err);
    if (scratch == nullptr) return err;
    return launch_linear_cross_entropy_fwd(hidden, weight, targets, v_start, n, h, v_count, row_stats, scratch,
                                           kNoAllocScratchBytes, dtype, stream);
}

// d(loss)/d(logits) of rows [0, n) against the whole vocabulary [0, v), in the storage type
// (no counterpart in the reference, which is forward-only).  lse[i] = max_i + log(sumexp_i) from
// the forward statistics; grad_scale = upstream gradient (x 1/valid_rows for a mean reduction).
extern "C" int32_t launch_lce_dlogits_fwd(const void* hidden, const void* weight, const int64_t* targets,
                                          const float* lse, int64_t n, int64_t h, int64_t v, int64_t ignore_index,
                                          float grad_scale, void* dlogits, int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (n <= 0 || v <= 0 || h <= 0) return cudaSuccess;
    if (dtype != kBF16 && dtype != kF16) return cudaErrorInvalidValue;
    if (h % 8 != 0 || !aligned16(hidden) || !aligned16(weight) || n >= (1LL << 31) || v >= (1LL << 31) || h >= (1LL << 31))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int m_tiles = static_cast<int>(ceil_div64(n, kBM)), n_tiles = static_cast<int>(ceil_div64(v, kBN));
    const int vec_ok = (v % 8 == 0 && aligned16(dlogits)) ? 1 : 0;
    auto run = [&](auto tag) -> cudaError_t {
        using T = decltype(tag);
        using Epi = EpiDlogits<T>;
        constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
        const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const uint32_t fmt = is_bf16 ? 1u : 0u;
        typename Epi::Params ep{targets, lse, static_cast<T*>(dlogits), n, v, ignore_index, grad_scale, vec_ok};
        const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<false, SchedGemm, Epi>() > 0;
        CUtensorMap ta, tb;
        cudaError_t e = make_tmap(&ta, dt, 2, hidden, n, h, kBM);
        if (e != cudaSuccess) return e;
        e = make_tmap(&tb, dt, 2, weight, v, h, pair ? 128 : kBN);
        if (e != cudaSuccess) return e;
        if (pair) {
            const int m_pairs = (m_tiles + 1) / 2;
            SchedGemm::Params sp{m_pairs, n_tiles, raster_group(2 * kBM, h, 2, m_pairs)};
            return launch_pair<false, SchedGemm, Epi>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, 2 * kBM, kBN),
                                                      static_cast<int64_t>(m_pairs) * n_tiles, s);
        }
        SchedGemm::Params sp{m_tiles, n_tiles, raster_group(kBM, h, 2, m_tiles)};
        const int64_t tiles = static_cast<int64_t>(m_tiles) * n_tiles;
        return launch<false, SchedGemm, Epi>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, kBM, kBN),
                                             static_cast<int>(tiles < sm_count() ? tiles : sm_count()), s);
    };
    return dtype == kBF16 ? run(__nv_bfloat16{}) : run(__half{});
}
