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

// kStore: also write the fp32 logits tile to `logits` [N, v_count] (the gradient path reads
// it back once instead of running the contraction a second time).
template <bool kStore>
struct EpiLceT {
    struct Params {
        const int64_t* targets;   // [N] global class ids (or ignore_index)
        float* partials;          // [splits][3][N]
        int64_t n_rows;
        int64_t v_count;          // rows of this weight slice
        int64_t v_start;          // global id of the slice's first row
        float* logits;            // kStore only
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
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int row_in_tile,
                                                 int c0, float (&acc)[32], const float*) {
        const int64_t col0 = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (col0 >= p.v_count) return;
        const int valid = p.v_count - col0 < 32 ? static_cast<int>(p.v_count - col0) : 32;
        if constexpr (kStore) {
            const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
            if (row < p.n_rows) {
                float* out = p.logits + row * p.v_count + col0;
                if (valid == 32) {       // written once, read once by the gradient pass: keep it out of the way in L2
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        Vec16 o;
                        o.w[0] = __float_as_uint(acc[4 * q]);
                        o.w[1] = __float_as_uint(acc[4 * q + 1]);
                        o.w[2] = __float_as_uint(acc[4 * q + 2]);
                        o.w[3] = __float_as_uint(acc[4 * q + 3]);
                        st_stream(out + 4 * q, o);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j < valid) out[j] = acc[j];
                }
            }
        }
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

using EpiLce = EpiLceT<false>;

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

namespace cck {
namespace tc {
template <bool kStore>
cudaError_t lce_forward(const void* hidden, const void* weight, const int64_t* targets, int64_t v_start, int64_t n,
                        int64_t h, int64_t v_count, float* row_stats, void* workspace, int64_t workspace_bytes,
                        float* logits, int32_t dtype, cudaStream_t s) {
    using Epi = EpiLceT<kStore>;
    if (n <= 0 || v_count <= 0 || h <= 0) return cudaSuccess;
    if (dtype != kBF16 && dtype != kF16) return cudaErrorInvalidValue;
    if (h % 8 != 0 || !aligned16(hidden) || !aligned16(weight) || n >= (1LL << 31) || v_count >= (1LL << 31) ||
        h >= (1LL << 31))
        return cudaErrorInvalidValue;
    if (kStore && (logits == nullptr || !aligned16(logits) || v_count % 4 != 0)) return cudaErrorInvalidValue;
    const LcePlan plan = lce_plan(n, v_count);
    if (workspace == nullptr || workspace_bytes < static_cast<int64_t>(plan.splits) * 3 * n * 4) return cudaErrorInvalidValue;
    const bool is_bf16 = dtype == kBF16;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 2, hidden, n, h, kBM);
    if (e != cudaSuccess) return e;
    e = make_tmap(&tb, dt, 2, weight, v_count, h, plan.pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    SchedLce::Params sp{plan.m_units, plan.n_tiles, plan.splits,
                        raster_group(plan.pair ? 2 * kBM : kBM, h, 2, plan.m_units)};
    typename Epi::Params ep{targets, static_cast<float*>(workspace), n, v_count, v_start, logits};
    const int64_t units = static_cast<int64_t>(plan.m_units) * plan.splits;
    const uint32_t fmt = is_bf16 ? 1u : 0u;
    if (plan.pair) {
        e = launch_pair<false, SchedLce, Epi>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, 2 * kBM, kBN), units, s);
    } else {
        const int ctas = static_cast<int>(units < plan.workers ? units : plan.workers);
        e = launch<false, SchedLce, Epi>(ta, tb, sp, ep, h, ptx::instr_desc(fmt, fmt, kBM, kBN), ctas, s);
    }
    if (e != cudaSuccess) return e;
    lce_merge_kernel<<<static_cast<unsigned>(ceil_div64(n, 256)), 256, 0, s>>>(
        static_cast<const float*>(workspace), plan.splits, n, row_stats);
    return cudaGetLastError();
}

// ---- d(loss)/d(logits) from stored fp32 logits, written row-major AND transposed.
//   dl[i, j] = (exp(l_ij - lse_i) - [j == target_i]) * grad_scale   (0 for ignored rows)
// One CTA owns a 64-row x 128-column tile.
//   Pass 0: 64 threads put each row's (-lse * log2 e, scale) in shared memory.
//   Pass 1: a warp walks 8 rows, a lane owns four adjacent columns (16-byte loads, all 8 in
//           flight before the first use), stores the four rounded values to dl (8 bytes per
//           lane) and to a shared tile in which row r sits in slot r/4 + 16 * (r % 4).
//   Pass 1b: the one element per row that carries the "- 1" of its target column is patched
//           by one thread per row, in dl and in the shared tile (the main loop stays free of
//           per-row 64-bit target arithmetic).
//   Pass 2: a lane owns one row QUAD of two adjacent columns - slots q, q + 16, q + 32, q + 48
//           - and writes 8 bytes per column to dl_t: 16 lanes cover 128 contiguous bytes; the
//           other half-warp works on the next column pair, which keeps the shared-memory
//           reads (even word pitch) conflict-free.
// HBM-bound: 4 (read) + 2 + 2 (writes) bytes per logit.
constexpr int kDlRows = 64;
constexpr int kDlCols = 128;
constexpr int kDlPitchW = kDlCols / 2 + 2;   // 32-bit words per slot; even, so 8-byte stores stay aligned

template <typename T>
__global__ void __launch_bounds__(256)
lce_dlogits_from_logits_kernel(const float* __restrict__ logits, const int64_t* __restrict__ targets,
                               const float* __restrict__ lse, int64_t n, int64_t v, int64_t ignore_index,
                               float grad_scale, T* __restrict__ dl, T* __restrict__ dl_t, int64_t ld_t) {
    __shared__ __align__(16) uint32_t tile[kDlRows * kDlPitchW];
    __shared__ float2 row_par[kDlRows];               // (-lse * log2 e, scale)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col0 = static_cast<int64_t>(blockIdx.x) * kDlCols;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kDlRows;
    const int64_t col = col0 + 4 * lane;
    const bool col_ok = col < v;                      // v % 4 == 0: all four columns or none

    float4 lg[8];
    const float* src = logits + (row0 + warp * 8) * v + col;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        lg[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (row0 + warp * 8 + i < n && col_ok) {
            const Vec16 x = ld_stream(src + i * v);
            lg[i] = make_float4(__uint_as_float(x.w[0]), __uint_as_float(x.w[1]), __uint_as_float(x.w[2]),
                                __uint_as_float(x.w[3]));
        }
    }
    int64_t my_target = -1;                           // threads 0..63: target column of row `threadIdx.x`
    if (threadIdx.x < kDlRows) {
        const int64_t row = row0 + threadIdx.x;
        float2 par = make_float2(0.0f, 0.0f);
        if (row < n) {
            const int64_t t = targets[row];
            par = make_float2(-lse[row] * kLog2e, t == ignore_index ? 0.0f : grad_scale);
            if (t != ignore_index && t >= col0 && t < col0 + kDlCols && t < v) my_target = t;
        }
        row_par[threadIdx.x] = par;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = warp * 8 + i;
        const float2 par = row_par[r];
        const float a = ex2_approx(fmaf(lg[i].x, kLog2e, par.x)) * par.y;
        const float b = ex2_approx(fmaf(lg[i].y, kLog2e, par.x)) * par.y;
        const float c = ex2_approx(fmaf(lg[i].z, kLog2e, par.x)) * par.y;
        const float d = ex2_approx(fmaf(lg[i].w, kLog2e, par.x)) * par.y;
        const uint32_t p0 = Store<T>::pack2(a, b), p1 = Store<T>::pack2(c, d);
        if (row0 + r < n && col_ok) st_stream8(dl + (row0 + r) * v + col, p0, p1);
        if (dl_t != nullptr) {
            const int slot = (r >> 2) + 16 * (r & 3);
            *reinterpret_cast<uint2*>(&tile[slot * kDlPitchW + 2 * lane]) = make_uint2(p0, p1);
        }
    }
    __syncthreads();
    if (my_target >= 0) {                             // the target column's element: (p - 1) * scale
        const int r = threadIdx.x;
        const float2 par = row_par[r];
        const float l = logits[(row0 + r) * v + my_target];
        T val;
        Store<T>::store1(&val, (ex2_approx(fmaf(l, kLog2e, par.x)) - 1.0f) * par.y);
        dl[(row0 + r) * v + my_target] = val;
        const int c = static_cast<int>(my_target - col0);
        if (dl_t != nullptr) reinterpret_cast<T*>(&tile[((r >> 2) + 16 * (r & 3)) * kDlPitchW])[c] = val;
    }
    if (dl_t == nullptr) return;                      // row-major output only (the GEMMs that follow read it as stored)
    __syncthreads();
    const int quad = lane & 15, half = lane >> 4;
    const int64_t rq = row0 + 4 * quad;               // first row of this lane's quad
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int cw = warp * 8 + 2 * i + half;       // column-pair index within the tile
        const int64_t c = col0 + 2 * cw;
        if (c >= v || rq >= n) continue;
        const uint32_t w0 = tile[quad * kDlPitchW + cw], w1 = tile[(quad + 16) * kDlPitchW + cw];
        const uint32_t w2 = tile[(quad + 32) * kDlPitchW + cw], w3 = tile[(quad + 48) * kDlPitchW + cw];
        const uint32_t lo01 = __byte_perm(w0, w1, 0x5410), lo23 = __byte_perm(w2, w3, 0x5410);   // column c
        const uint32_t hi01 = __byte_perm(w0, w1, 0x7632), hi23 = __byte_perm(w2, w3, 0x7632);   // column c + 1
        T* out = dl_t + c * ld_t + rq;
        if (rq + 4 <= n) {
            st_stream8(out, lo01, lo23);
            st_stream8(out + ld_t, hi01, hi23);
        } else {
            const uint32_t lo[2] = {lo01, lo23}, hi[2] = {hi01, hi23};
            uint16_t* o16 = reinterpret_cast<uint16_t*>(out);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (rq + k < n) {
                    o16[k] = static_cast<uint16_t>(lo[k >> 1] >> (16 * (k & 1)));
                    o16[ld_t + k] = static_cast<uint16_t>(hi[k >> 1] >> (16 * (k & 1)));
                }
        }
    }
}

// ---- out[c, r] = in[r, c] for 2-byte elements (any 16-bit type), out's row pitch ld_out >= rows;
// out[c, rows..ld_out) is zero-filled.  The gradient GEMMs contract over the row index, so
// their operands have to be row-contiguous: this makes hidden^T and W^T.  Same tiling and
// shared-memory slot layout as lce_dlogits_from_logits_kernel (64 x 128 tile, 8-byte loads,
// 8-byte stores in 128-byte runs).  HBM-bound: 4 bytes per element.
__global__ void __launch_bounds__(256)
transpose16_kernel(const uint16_t* __restrict__ in, int64_t rows, int64_t cols, uint16_t* __restrict__ out,
                   int64_t ld_out) {
    __shared__ __align__(16) uint32_t tile[kDlRows * kDlPitchW];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col0 = static_cast<int64_t>(blockIdx.x) * kDlCols;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kDlRows;
    const int64_t col = col0 + 4 * lane;
    uint2 x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = row0 + warp * 8 + i;
        x[i] = make_uint2(0u, 0u);
        if (row < rows && col < cols)
            asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                         : "=r"(x[i].x), "=r"(x[i].y)
                         : "l"(in + row * cols + col));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = warp * 8 + i;
        *reinterpret_cast<uint2*>(&tile[((r >> 2) + 16 * (r & 3)) * kDlPitchW + 2 * lane]) = x[i];
    }
    __syncthreads();
    const int quad = lane & 15, half = lane >> 4;
    const int64_t rq = row0 + 4 * quad;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int cw = warp * 8 + 2 * i + half;
        const int64_t c = col0 + 2 * cw;
        if (c >= cols || rq >= ld_out) continue;
        const uint32_t w0 = tile[quad * kDlPitchW + cw], w1 = tile[(quad + 16) * kDlPitchW + cw];
        const uint32_t w2 = tile[(quad + 32) * kDlPitchW + cw], w3 = tile[(quad + 48) * kDlPitchW + cw];
        // rows beyond `rows` were loaded as zeros, so the padding comes out as zeros
        uint16_t* o = out + c * ld_out + rq;
        st_stream8(o, __byte_perm(w0, w1, 0x5410), __byte_perm(w2, w3, 0x5410));
        st_stream8(o + ld_out, __byte_perm(w0, w1, 0x7632), __byte_perm(w2, w3, 0x7632));
    }
}
}  // namespace tc
}  // namespace cck

extern "C" int32_t launch_linear_cross_entropy_fwd(const void* hidden, const void* weight, const int64_t* targets,
                                                   int64_t v_start, int64_t n, int64_t h, int64_t v_count,
                                                   float* row_stats, void* workspace, int64_t workspace_bytes,
                                                   int32_t dtype, void* stream) {
    return cck::tc::lce_forward<false>(hidden, weight, targets, v_start, n, h, v_count, row_stats, workspace,
                                       workspace_bytes, nullptr, dtype, static_cast<cudaStream_t>(stream));
}

// The same launch that also leaves the fp32 logits in `logits` [n, v_count] (v_count % 4 == 0,
// 16-byte aligned) for launch_lce_dlogits_from_logits.  No counterpart in the reference.
extern "C" int32_t launch_linear_cross_entropy_fwd_store(const void* hidden, const void* weight,
                                                         const int64_t* targets, int64_t v_start, int64_t n,
                                                         int64_t h, int64_t v_count, float* row_stats,
                                                         void* workspace, int64_t workspace_bytes, float* logits,
                                                         int32_t dtype, void* stream) {
    return cck::tc::lce_forward<true>(hidden, weight, targets, v_start, n, h, v_count, row_stats, workspace,
                                      workspace_bytes, logits, dtype, static_cast<cudaStream_t>(stream));
}

// d(loss)/d(logits) from stored logits: dlogits [n, v] and, unless dlogits_t is NULL, its
// transpose dlogits_t [v, ld_t] (ld_t >= n, a multiple of 4; columns n..ld_t of dlogits_t are
// not written), both in the storage type.  `targets` index the columns of `logits` (a value outside [0, v) selects none);
// v % 4 == 0.
extern "C" int32_t launch_lce_dlogits_from_logits(const float* logits, const int64_t* targets, const float* lse,
                                                  int64_t n, int64_t v, int64_t ignore_index, float grad_scale,
                                                  void* dlogits, void* dlogits_t, int64_t ld_t, int32_t dtype,
                                                  void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (n <= 0 || v <= 0) return cudaSuccess;
    if (dtype != kBF16 && dtype != kF16) return cudaErrorInvalidValue;
    if (v % 4 != 0 || !aligned16(logits) || (reinterpret_cast<uintptr_t>(dlogits) & 7u)) return cudaErrorInvalidValue;
    if (dlogits_t != nullptr && (ld_t < n || ld_t % 4 != 0 || (reinterpret_cast<uintptr_t>(dlogits_t) & 7u)))
        return cudaErrorInvalidValue;
    const int64_t gx = ceil_div64(v, kDlCols), gy = ceil_div64(n, kDlRows);
    if (gy > 65535) return cudaErrorInvalidValue;
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == kBF16)
        lce_dlogits_from_logits_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
            logits, targets, lse, n, v, ignore_index, grad_scale, static_cast<__nv_bfloat16*>(dlogits),
            static_cast<__nv_bfloat16*>(dlogits_t), ld_t);
    else
        lce_dlogits_from_logits_kernel<__half><<<grid, 256, 0, s>>>(
            logits, targets, lse, n, v, ignore_index, grad_scale, static_cast<__half*>(dlogits),
            static_cast<__half*>(dlogits_t), ld_t);
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
// to be asked for, once per device, with that device current.  The per-device cache is
// filled without a lock: host threads that make the first call on one device at the same
// time each look the address up and store the same value, so no thread reads a wrong one.
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

// out[c, r] = in[r, c] for a contiguous [rows, cols] matrix of 2-byte elements; out is
// [cols, ld_out] with ld_out >= rows, and out[:, rows..ld_out) is set to zero.  cols % 4 == 0,
// ld_out % 4 == 0, both pointers 8-byte aligned.  No counterpart in the reference.
extern "C" int32_t launch_transpose_2byte(const void* in, int64_t rows, int64_t cols, void* out, int64_t ld_out,
                                          void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    if (cols % 4 != 0 || ld_out < rows || ld_out % 4 != 0 || (reinterpret_cast<uintptr_t>(in) & 7u) ||
        (reinterpret_cast<uintptr_t>(out) & 7u))
        return cudaErrorInvalidValue;
    const int64_t gx = ceil_div64(cols, kDlCols), gy = ceil_div64(ld_out, kDlRows);
    if (gy > 65535) return cudaErrorInvalidValue;
    transpose16_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(in), rows, cols,
                                                              static_cast<uint16_t*>(out), ld_out);
    return cudaGetLastError();
}
