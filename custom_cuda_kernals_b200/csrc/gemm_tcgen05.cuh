// Persistent, warp-specialised tcgen05 GEMM mainloop for sm_100a, shared by
// matmul_add_bias (bf16/fp16/fp8) and the fused linear + cross-entropy kernel.
//
//   D[128 x 256] (fp32, in TMEM) = A[128 x K] * B[256 x K]^T,  A and B both K-major.
//
// One CTA per SM, 192 threads:
//   warp 0  (one lane)  TMA producer: 128-byte-wide K slabs of A (128 rows) and
//                       B (256 rows) into a 4-stage shared-memory ring, 128-byte
//                       swizzle, completion by mbarrier transaction bytes.
//   warp 1  (one lane)  MMA issuer: four tcgen05.mma (K = 32 bytes each) per
//                       stage into one of two 256-column TMEM accumulators;
//                       tcgen05.commit releases the stage / publishes the tile.
//   warps 2-5           epilogue: tcgen05.ld of the finished accumulator (each
//                       thread owns one output row) while the MMA warp already
//                       fills the other accumulator.
// Tiles come from a scheduler policy, the epilogue from an epilogue policy.
// gemm_kernel is that single-CTA form; gemm_pair_kernel further down runs the same
// roles on a pair of CTAs that share a 256 x 256 tile (cta_group::2) and is the
// default.  Every CTA fetches its own operand tiles; no load is shared across CTAs.
// All waits are bounded; a time-out sets bit 0 of *status and the CTA leaves.
//
// Operand layouts (kMajors): by default A [M,K] and B [N,K] are both K-major (rows contiguous
// along K: activations [tokens, features], nn.Linear weights [out, in]).  Bit 0 (kAMn) / bit 1
// (kBMn) of kMajors switch an operand to MN-major: it is stored as [K, M] (or [K, N]) row-major
// - the transpose of the above - and is fed to the tensor cores as stored, through 64 x 64
// TMA boxes and MN-major shared-memory descriptors, so gradient GEMMs (dX = dY W, dW = dY^T X)
// need no transposed copies of their operands.  16-bit types only.
#pragma once

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace cck {
namespace tc {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kRowBytes = 128;                 // K slab width in bytes (= swizzle span)
constexpr int kStages = 4;
constexpr int kABytes = kBM * kRowBytes;       // 16 KiB
constexpr int kBBytes = kBN * kRowBytes;       // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes; // 48 KiB
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr int kTmemCols = 512;                 // two 256-column fp32 accumulators
constexpr int kScratchFloatsPerWarp = 2 * kBN; // per-epilogue-warp staging (bias / scales)
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ +
                           kEpiWarps * kScratchFloatsPerWarp * 4;
constexpr int kAMn = 1, kBMn = 2;              // kMajors bits: operand stored [K, M] / [K, N]
constexpr int kMnBoxBytes = 64 * kRowBytes;    // one 64 (MN) x 64 (K) box of an MN-major operand: 8 KiB

struct TileWork {
    int m_tile, n_tile;
    int n0;             // first output column of the tile (n_tile x the kernel's tile width)
    int split;          // LCE: vocabulary split this tile belongs to
    bool first, last;   // first / last tile of a unit (a unit = tiles sharing epilogue row state)
};

// Row units (128-row tiles, or 256-row tiles of a CTA pair) are walked in groups of `group`
// units: inside a group the row unit varies fastest, then the column tile.  The workers that
// run at the same time therefore touch `group` A panels and workers/group B panels - a roughly
// square patch whose operands stay in the 126 MB L2 - instead of every A panel of the matrix.
__host__ __device__ inline void grouped_unit(int t, int m_units, int other, int group, int& m, int& o) {
    const int span = group * other;
    const int g = t / span;
    const int r = t - g * span;
    const int left = m_units - g * group;
    const int gm = left < group ? left : group;
    o = r / gm;
    m = g * group + (r - o * gm);
}
// Units per group so that one group's A panels take about 48 MB of L2 (4..32 units).
inline int raster_group(int64_t rows_per_unit, int64_t k_elems, int elem_bytes, int m_units) {
    const int64_t panel = rows_per_unit * k_elems * elem_bytes;
    int64_t g = panel > 0 ? (48ll << 20) / panel : 32;
    if (g < 4) g = 4;
    if (g > 32) g = 32;
    return static_cast<int>(g < m_units ? g : m_units);
}

// ---- scheduler: plain GEMM
struct SchedGemm {
    struct Params { int m_tiles, n_tiles, group; };
    struct Iter {
        int t, step, total;
        Params p;
        __device__ Iter(const Params& q, int worker, int workers)
            : t(worker), step(workers), total(q.m_tiles * q.n_tiles), p(q) {}
        __device__ bool next(TileWork& w) {
            if (t >= total) return false;
            grouped_unit(t, p.m_tiles, p.n_tiles, p.group, w.m_tile, w.n_tile);
            w.split = 0;
            w.first = w.last = true;
            t += step;
            return true;
        }
    };
};

// Reads one finished 128 x 256 accumulator (this thread's row) out of tensor memory and hands
// it to the epilogue policy, 32 columns at a time.  A policy with kPairedHalves pairs column j
// of the tile's first half with column j of its second half (gate / up of a fused SwiGLU GEMM)
// - or, with kPairStride = 64, column j of a 128-column head with column j + 64 (RoPE) - and gets
// both 32-column pieces at once.
template <class Epi, class = void> struct PairedHalves { static constexpr bool value = false; };
template <class Epi> struct PairedHalves<Epi, std::enable_if_t<Epi::kPairedHalves>> { static constexpr bool value = true; };
// Distance in columns between the two members of a pair: half the tile unless the policy says
// otherwise with kPairStride (64: column j of every 128-column head with column j + 64, RoPE).
template <class Epi, class = void> struct PairStride { static constexpr int value = kBN / 2; };
template <class Epi> struct PairStride<Epi, std::void_t<decltype(Epi::kPairStride)>> { static constexpr int value = Epi::kPairStride; };

template <class Epi, int BN = kBN>
__device__ __forceinline__ void drain_tile(const typename Epi::Params& ep, typename Epi::Thread& th, const TileWork& w,
                                           int row_in_tile, uint32_t t0, float* scratch) {
    if constexpr (PairedHalves<Epi>::value) {
        static_assert(BN == kBN, "paired halves need the full-width tile");
#pragma unroll 1
        constexpr int kStride = PairStride<Epi>::value;
        for (int c = 0; c < kBN / 64; ++c) {
            const int lo_col = (c * 32 / kStride) * 2 * kStride + (c * 32) % kStride;
            float lo[32], hi[32];
            ptx::tmem_ld32(t0 + lo_col, lo);
            ptx::tmem_ld32(t0 + lo_col + kStride, hi);
            Epi::chunk2(ep, th, w, row_in_tile, lo_col, lo, hi, scratch);
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            float acc[32];
            ptx::tmem_ld32(t0 + c * 32, acc);
            Epi::chunk(ep, th, w, row_in_tile, c * 32, acc, scratch);
        }
    }
}

// ---- kernel
// BN = 256 is the throughput shape.  BN = 64 is for problems with too few 128 x 256 tiles to
// occupy the machine (small M: decode-sized batches): four times as many CTAs pull the weight
// matrix, 24 KB stages let the ring run 8 deep, and the two accumulators take 128 TMEM columns.
template <int BN> struct TileShape {
    static constexpr int kStagesN = BN == kBN ? kStages : 8;
    static constexpr int kBBytesN = BN * kRowBytes;
    static constexpr int kStageBytesN = kABytes + kBBytesN;
    static constexpr int kTmemColsN = 2 * BN;
    static constexpr int kSmemBytesN = kStagesN * kStageBytesN + 1024 + 256 + kEpiWarps * kScratchFloatsPerWarp * 4;
};

// One K slab of one operand into shared memory at `dst`: a single box for a K-major operand,
// `mn_extent / 64` boxes of 64 x 64 for an MN-major one (x = M / N coordinate, y = K coordinate).
template <bool kMn, bool kPairLoad>
__device__ __forceinline__ void load_slab(uint32_t dst, const CUtensorMap* map, uint32_t bar, int kb, int elems_per_slab,
                                          int mn0, int mn_extent) {
    if constexpr (!kMn) {
        if constexpr (kPairLoad) ptx::tma_load_2d_pair(dst, map, bar, kb * elems_per_slab, mn0);
        else                     ptx::tma_load_2d(dst, map, bar, kb * elems_per_slab, mn0);
    } else {
        for (int j = 0; j < mn_extent / 64; ++j) {
            if constexpr (kPairLoad) ptx::tma_load_2d_pair(dst + j * kMnBoxBytes, map, bar, mn0 + 64 * j, kb * 64);
            else                     ptx::tma_load_2d(dst + j * kMnBoxBytes, map, bar, mn0 + 64 * j, kb * 64);
        }
    }
}
template <bool kMn>
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
    if constexpr (kMn) return ptx::smem_desc_mn_sw128(saddr, kMnBoxBytes);
    else               return ptx::smem_desc_k_sw128(saddr);
}
// what one 16-element K step adds to the descriptor's start-address field
template <bool kMn> __host__ __device__ constexpr uint64_t k_step() { return kMn ? (2048 >> 4) : (32 >> 4); }

template <bool kFp8, class Sched, class Epi, int BN = kBN, int kMajors = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const typename Sched::Params sp, const typename Epi::Params ep, int k_blocks, uint32_t idesc,
            unsigned int* status) {
    constexpr int kStages = TileShape<BN>::kStagesN;          // shadow the full-width constants
    constexpr int kStageBytes = TileShape<BN>::kStageBytesN;
    constexpr int kTmemCols = TileShape<BN>::kTmemColsN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;            // stage ring, 1024-byte aligned
    uint8_t* gen = smem_raw + (base - raw);
    const uint32_t bar0 = base + kStages * kStageBytes;       // mbarriers, 8 bytes each
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
    uint8_t* misc = gen + kStages * kStageBytes + 8 * (2 * kStages + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
    float* scratch = reinterpret_cast<float*>(gen + kStages * kStageBytes + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kElemsPerSlab = kFp8 ? 128 : 64;
    constexpr bool kAIsMn = (kMajors & kAMn) != 0, kBIsMn = (kMajors & kBMn) != 0;
    static_assert(!kFp8 || kMajors == 0, "MN-major operands are for 16-bit types");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), kEpiWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            typename Sched::Iter it(sp, blockIdx.x, gridDim.x);
            TileWork w;
            while (ok && it.next(w)) {
                const int m0 = w.m_tile * kBM, n0 = w.n_tile * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    const uint32_t a_dst = base + stage * kStageBytes;
                    load_slab<kAIsMn, false>(a_dst, &tmap_a, full_bar(stage), kb, kElemsPerSlab, m0, kBM);
                    load_slab<kBIsMn, false>(a_dst + kABytes, &tmap_b, full_bar(stage), kb, kElemsPerSlab, n0, BN);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc_iter = 0;
            bool ok = true;
            typename Sched::Iter it(sp, blockIdx.x, gridDim.x);
            TileWork w;
            while (ok && it.next(w)) {
                const int buf = acc_iter & 1;
                const uint32_t acc_phase = (acc_iter >> 1) & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, status)) break;
                ptx::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, status)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_src = base + stage * kStageBytes;
                    const uint64_t da = operand_desc<kAIsMn>(a_src);
                    const uint64_t db = operand_desc<kBIsMn>(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {        // 4 x 32 bytes of K per slab
                        const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                        if (kFp8) ptx::mma_f8(d, da + k_step<kAIsMn>() * k, db + k_step<kBIsMn>() * k, idesc, acc);
                        else      ptx::mma_f16(d, da + k_step<kAIsMn>() * k, db + k_step<kBIsMn>() * k, idesc, acc);
                    }
                    ptx::mma_commit(empty_bar(stage));   // stage reusable once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::mma_commit(tfull_bar(buf));  // accumulator complete
                ++acc_iter;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                     // TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        float* my_scratch = scratch + (warp - 2) * kScratchFloatsPerWarp;
        typename Epi::Thread th;
        int acc_iter = 0;
        typename Sched::Iter it(sp, blockIdx.x, gridDim.x);
        TileWork w;
        while (it.next(w)) {
            w.n0 = w.n_tile * BN;
            const int buf = acc_iter & 1;
            const uint32_t acc_phase = (acc_iter >> 1) & 1;
            __syncwarp();
            Epi::tile_begin(ep, th, w, my_scratch, lane, row_in_tile);
            __syncwarp();
            const bool got = ptx::mbar_wait(tfull_bar(buf), acc_phase, abort_flag, status);
            if (!__all_sync(0xffffffffu, got)) break;
            ptx::tc_fence_after_sync();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            drain_tile<Epi, BN>(ep, th, w, row_in_tile, t0, my_scratch);
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
            Epi::tile_end(ep, th, w, row_in_tile);
            ++acc_iter;
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // give copies / MMAs that may still be in flight a bounded time to land
        const unsigned long long t0 = ptx::globaltimer();
        while (ptx::globaltimer() - t0 < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicOr(status, 1u);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ CTA-pair variant
// Two CTAs on the SMs of one TPC (a cluster of 2) share one 256 x 256 output tile:
// CTA r loads rows [128r, 128r+128) of the A tile and rows [128r, 128r+128) of the B
// tile (32 KB per stage instead of 48 KB, so the ring is 6 stages deep), one thread of
// the leader CTA (rank 0) issues tcgen05.mma.cta_group::2 with M = 256, and each CTA's
// tensor memory receives its own 128 accumulator rows - which the CTA's epilogue warps
// drain exactly as in the single-CTA kernel (its tile is m_tile = 2 * pair_tile + r).
// Per MMA each SM reads 4 KB of A and 4 KB of B from its shared memory instead of
// 4 + 8 KB: the operand traffic that limits the single-CTA kernel is cut by a third.
// Cross-CTA signalling: both CTAs' TMA loads count their bytes on the leader's `full`
// barrier; the leader's commits arrive on both CTAs' `empty` and `tmem full` barriers;
// the peer's epilogue warps arrive on the leader's `tmem empty` barrier.  No load is
// multicast; the only remote accesses are barrier arrivals and the MMA itself.
constexpr int kPairStages = 6;
constexpr int kPairBBytes = 128 * kRowBytes;                    // this CTA's half of B: 16 KiB
constexpr int kPairStageBytes = kABytes + kPairBBytes;          // 32 KiB
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256 + kEpiWarps * kScratchFloatsPerWarp * 4;

template <bool kFp8, class Sched, class Epi, int kMajors = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const typename Sched::Params sp, const typename Epi::Params ep, int k_blocks, uint32_t idesc,
                 unsigned int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    const uint32_t bar0 = base + kPairStages * kPairStageBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kPairStages + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kPairStages + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kPairStages + 2 + b); };
    uint8_t* misc = gen + kPairStages * kPairStageBytes + 8 * (2 * kPairStages + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
    float* scratch = reinterpret_cast<float*>(gen + kPairStages * kPairStageBytes + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    constexpr int kElemsPerSlab = kFp8 ? 128 : 64;
    constexpr bool kAIsMn = (kMajors & kAMn) != 0, kBIsMn = (kMajors & kBMn) != 0;
    static_assert(!kFp8 || kMajors == 0, "MN-major operands are for 16-bit types");

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);                 // used in the leader only
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), 2 * kEpiWarps);   // used in the leader only: both CTAs' epilogues
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {                                        // the same warp in both CTAs
        ptx::tmem_alloc_pair(ptx::smem_addr(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();                                  // barriers of both CTAs initialised before any remote arrival
    ptx::cluster_wait();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            typename Sched::Iter it(sp, pair_id, pairs);
            TileWork w;
            while (ok && it.next(w)) {
                const int m0 = (w.m_tile * 2 + static_cast<int>(rank)) * kBM;
                const int n0 = w.n_tile * kBN + static_cast<int>(rank) * 128;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status)) { ok = false; break; }
                    const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), 0);
                    if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);
                    const uint32_t a_dst = base + stage * kPairStageBytes;
                    load_slab<kAIsMn, true>(a_dst, &tmap_a, leader_full, kb, kElemsPerSlab, m0, kBM);
                    load_slab<kBIsMn, true>(a_dst + kABytes, &tmap_b, leader_full, kb, kElemsPerSlab, n0, 128);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc_iter = 0;
            bool ok = true;
            typename Sched::Iter it(sp, pair_id, pairs);
            TileWork w;
            while (ok && it.next(w)) {
                const int buf = acc_iter & 1;
                const uint32_t acc_phase = (acc_iter >> 1) & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, status)) break;
                ptx::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * kBN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, status)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_src = base + stage * kPairStageBytes;
                    const uint64_t da = operand_desc<kAIsMn>(a_src);
                    const uint64_t db = operand_desc<kBIsMn>(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                        if (kFp8) ptx::mma_f8_pair(d, da + k_step<kAIsMn>() * k, db + k_step<kBIsMn>() * k, idesc, acc);
                        else      ptx::mma_f16_pair(d, da + k_step<kAIsMn>() * k, db + k_step<kBIsMn>() * k, idesc, acc);
                    }
                    ptx::mma_commit_pair(ptx::map_to_cta(empty_bar(stage), 0));   // stage free in both CTAs
                    ptx::mma_commit_pair(ptx::map_to_cta(empty_bar(stage), 1));
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    ptx::mma_commit_pair(ptx::map_to_cta(tfull_bar(buf), 0));     // accumulators complete in both CTAs
                    ptx::mma_commit_pair(ptx::map_to_cta(tfull_bar(buf), 1));
                }
                ++acc_iter;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        float* my_scratch = scratch + (warp - 2) * kScratchFloatsPerWarp;
        typename Epi::Thread th;
        int acc_iter = 0;
        typename Sched::Iter it(sp, pair_id, pairs);
        TileWork w;
        while (it.next(w)) {
            w.m_tile = w.m_tile * 2 + static_cast<int>(rank);
            w.n0 = w.n_tile * kBN;
            const int buf = acc_iter & 1;
            const uint32_t acc_phase = (acc_iter >> 1) & 1;
            __syncwarp();
            Epi::tile_begin(ep, th, w, my_scratch, lane, row_in_tile);
            __syncwarp();
            const bool got = ptx::mbar_wait(tfull_bar(buf), acc_phase, abort_flag, status);
            if (!__all_sync(0xffffffffu, got)) break;
            ptx::tc_fence_after_sync();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
            drain_tile<Epi>(ep, th, w, row_in_tile, t0, my_scratch);
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(buf), 0));
            Epi::tile_end(ep, th, w, row_in_tile);
            ++acc_iter;
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = ptx::globaltimer();
        while (ptx::globaltimer() - t0 < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicOr(status, 1u);
        __syncthreads();
    }
    // neither CTA may leave (or free tensor memory) while the other can still reach into it
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ host side
// Row-major [rows, cols] matrix of `elem_bytes`-wide elements; box = 128 bytes x box_rows, 128-byte swizzle.
inline cudaError_t make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* ptr,
                             int64_t rows, int64_t cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * elem_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// MN-major operand: the matrix is stored [k_rows, mn_cols] row-major; box = 64 (MN, 128 bytes) x 64 (K).
inline cudaError_t make_tmap_mn(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, int64_t k_rows,
                                int64_t mn_cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(mn_cols), static_cast<cuuint64_t>(k_rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(mn_cols) * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// CCK_GEMM_SINGLE_CTA=1 in the environment keeps every GEMM on the single-CTA kernel.
inline bool pair_kernels_enabled() {
    static const bool on = [] {
        const char* v = getenv("CCK_GEMM_SINGLE_CTA");
        return !(v && v[0] == '1');
    }();
    return on;
}

// CCK_GEMM_NO_NARROW=1 keeps small problems on the full-width tiles.
inline bool narrow_tiles_enabled() {
    static const bool on = [] {
        const char* v = getenv("CCK_GEMM_NO_NARROW");
        return !(v && v[0] == '1');
    }();
    return on;
}

// Split-K over a thread-block cluster for problems with too few output tiles to pull the weight
// matrix at speed.  Default: on for decode-sized batches (M <= 128 rows: gemm_decode.cuh, weight
// rows on the M side of the instruction), off above.  CCK_GEMM_SPLITK=1 extends it to every problem
// that leaves SMs idle (gemm_splitk.cuh), CCK_GEMM_SPLITK=0 turns it off.  Why not everywhere: the
// other kernels add a row's products in one fixed order whatever M and N are, so a row shard or a
// column shard of a problem gives bit for bit the rows / columns of the whole; partial sums over K
// slices are added in another order, so where split-K runs that invariance does not hold (results
// are still deterministic run to run).
inline int splitk_mode() {
    static const int mode = [] {
        const char* v = getenv("CCK_GEMM_SPLITK");
        return (v && (v[0] == '0' || v[0] == '1')) ? v[0] - '0' : -1;
    }();
    return mode;
}
inline bool splitk_enabled(int64_t m_rows) {
    const int mode = splitk_mode();
    return mode == 1 || (mode < 0 && m_rows <= 128);
}

inline int sm_count() {
    static int cached_per_device[kMaxDevices] = {};
    const int slot = current_device_slot();
    if (slot < 0) return kNumSMs;
    int& n = cached_per_device[slot];
    if (n <= 0) {
        int v = 0;
        n = (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, slot) == cudaSuccess && v > 0) ? v : kNumSMs;
    }
    return n;
}

template <bool kFp8, class Sched, class Epi, int BN = kBN, int kMajors = 0>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const typename Sched::Params& sp,
                   const typename Epi::Params& ep, int64_t k_elems, uint32_t idesc, int ctas, cudaStream_t s) {
    auto kern = gemm_kernel<kFp8, Sched, Epi, BN, kMajors>;
    constexpr int kSmemBytes = TileShape<BN>::kSmemBytesN;
    static bool configured[kMaxDevices] = {};   // per instantiation and device
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    if (!configured[slot]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[slot] = true;
    }
    unsigned int* st = status_word();
    if (!st) return cudaErrorMemoryAllocation;
    const int slab = kFp8 ? 128 : 64;
    const int k_blocks = static_cast<int>((k_elems + slab - 1) / slab);
    kern<<<ctas, kThreads, kSmemBytes, s>>>(ta, tb, sp, ep, k_blocks, idesc, st);
    return cudaGetLastError();
}

// Number of CTA pairs that can be resident at once (at most one pair per TPC).
template <bool kFp8, class Sched, class Epi, int kMajors = 0>
int max_pairs() {
    static int cached_per_device[kMaxDevices] = {};
    const int slot = current_device_slot();
    if (slot < 0) return 0;
    int& cached = cached_per_device[slot];
    if (cached > 0) return cached;
    auto kern = gemm_pair_kernel<kFp8, Sched, Epi, kMajors>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
        (void)cudaGetLastError();
        cudaLaunchAttribute attr;                 // some runtimes want the cluster shape spelled out
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
            (void)cudaGetLastError();
            return 0;
        }
    }
    cached = clusters;
    return cached;
}

// `pair_tiles` = number of 256-row x 256-column tiles (or units) to spread over the pairs.
template <bool kFp8, class Sched, class Epi, int kMajors = 0>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const typename Sched::Params& sp,
                        const typename Epi::Params& ep, int64_t k_elems, uint32_t idesc, int64_t pair_tiles,
                        cudaStream_t s) {
    const int cap = max_pairs<kFp8, Sched, Epi, kMajors>();
    if (cap <= 0) return cudaErrorLaunchOutOfResources;
    unsigned int* st = status_word();
    if (!st) return cudaErrorMemoryAllocation;
    const int pairs = static_cast<int>(pair_tiles < cap ? pair_tiles : cap);
    const int slab = kFp8 ? 128 : 64;
    const int k_blocks = static_cast<int>((k_elems + slab - 1) / slab);
    gemm_pair_kernel<kFp8, Sched, Epi, kMajors><<<2 * pairs, kThreads, kPairSmemBytes, s>>>(ta, tb, sp, ep, k_blocks, idesc, st);
    return cudaGetLastError();
}

}  // namespace tc
}  // namespace cck
