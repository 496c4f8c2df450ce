// Decode-sized GEMM: y[M,N] = x[M,K] @ W[N,K]^T + bias for a handful of tokens (M <= 128).
//
// With so few rows the job is to stream the weight matrix once, at the HBM rate, through as
// many SMs as possible - the arithmetic is negligible.  The roles of the operands are therefore
// swapped with respect to gemm_tcgen05.cuh: the WEIGHT rows are the M side of the tensor-core
// instruction (a CTA owns 128 consecutive output features and streams their 128 x K slab of W in
// 16 KB stages), the tokens are the N side (tcgen05.mma with N = 16, 32, 64 or 128; the x slab of a
// stage is 2-16 KB and stays in L2), and the accumulator is y^T: TMEM lane = output feature,
// column = token.  Eight stages of W are in flight per CTA (six with 128 tokens), one CTA per SM.  When N / 128 tiles
// do not fill the machine, a thread-block cluster of 2-8 CTAs shares a tile and splits K; the
// partial accumulators (128 x BT fp32, at most 64 KB per CTA) are summed through distributed
// shared memory as a reduce-scatter - every CTA of the cluster sums and stores its share of the
// tokens, adding the ranks' partials in rank order - no workspace, no atomics, deterministic,
// re-entrant across streams.  The epilogue adds the bias and stores the transpose: for one token, the 32
// lanes of a warp hold 32 consecutive output features, i.e. 64 contiguous bytes of y.
//
// Waits are the bounded ones of ptx.cuh; the cluster barriers are reached by every thread on
// every path; if any CTA of a cluster gave up, none of them stores anything for the tile and bit 0
// of the status word is set.  Sums over K slices are added in another order than the other GEMM
// kernels use, so these results agree with theirs to rounding, not bit for bit.
#pragma once

#include "gemm_splitk.cuh"

namespace cck {
namespace tc {

constexpr int kDecMaxTokens = 128;

template <int BT> struct DecShape {
    static_assert(BT == 16 || BT == 32 || BT == 64 || BT == 128, "token tile of 16, 32, 64 or 128");
    static constexpr int kStages = BT <= 64 ? 8 : 6;
    static constexpr int kTmemCols = BT <= 64 ? 64 : 128;
    static constexpr int kXBytes = BT * kRowBytes;                 // 2, 4, 8 or 16 KiB
    static constexpr int kStageBytes = kABytes + kXBytes;          // W slab + x slab
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

template <typename T, int BT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const T* __restrict__ bias, const T* __restrict__ residual, T* __restrict__ y, int64_t m, int64_t n,
                   int k_blocks, uint32_t idesc, unsigned int* status) {
    constexpr int kStageBytes = DecShape<BT>::kStageBytes;
    constexpr int kDecStages = DecShape<BT>::kStages;
    constexpr int kDecTmemCols = DecShape<BT>::kTmemCols;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    const uint32_t bar0 = base + kDecStages * kStageBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kDecStages + s); };
    const uint32_t tfull_bar = bar0 + 8u * (2 * kDecStages);
    uint8_t* misc = gen + kDecStages * kStageBytes + 8 * (2 * kDecStages + 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank(), splits = cluster_nctarank();
    const int n_tile = blockIdx.x / splits;                        // 128 output features
    const int kb0 = static_cast<int>((static_cast<int64_t>(rank) * k_blocks) / splits);
    const int kb1 = static_cast<int>((static_cast<int64_t>(rank + 1) * k_blocks) / splits);   // k_blocks >= splits

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDecStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_x);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kDecTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    constexpr int kChunks = BT <= 32 ? 1 : BT / 32;                 // 32-column TMEM reads per row
    float acc[kChunks][32];                                         // this thread's output feature, all tokens
    bool have_acc = false;
    if (warp == 0) {
        if (lane == 0) {                                            // ---- TMA producer
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status)) break;
                ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                const uint32_t w_dst = base + stage * kStageBytes;
                ptx::tma_load_2d(w_dst, &tmap_w, full_bar(stage), kb * 64, n_tile * kBM);
                ptx::tma_load_2d(w_dst + kABytes, &tmap_x, full_bar(stage), kb * 64, 0);
                if (++stage == kDecStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                            // ---- MMA issuer: D[128 features x BT tokens]
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, status)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t w_src = base + stage * kStageBytes;
                const uint64_t dw = ptx::smem_desc_k_sw128(w_src);
                const uint64_t dx = ptx::smem_desc_k_sw128(w_src + kABytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    ptx::mma_f16(tmem_base, dw + 2 * k, dx + 2 * k, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
                ptx::mma_commit(empty_bar(stage));
                if (++stage == kDecStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) ptx::mma_commit(tfull_bar);
        }
    } else {
        // ---- epilogue, part 1: this CTA's partial out of tensor memory
        const int quarter = warp & 3;
        const bool got = ptx::mbar_wait(tfull_bar, 0u, abort_flag, status);
        if (__all_sync(0xffffffffu, got)) {
            ptx::tc_fence_after_sync();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) ptx::tmem_ld32(t0 + 32 * c, acc[c]);
            have_acc = true;
            if (splits > 1) {
                // park it as BT / 4 float4 planes [plane][feature] (plane q = tokens 4q..4q+3):
                // consecutive features are 16 bytes apart, so this store and the remote loads of
                // part 2 are contiguous across a warp
                float4* part = reinterpret_cast<float4*>(gen);
                const int row = quarter * 32 + lane;
#pragma unroll
                for (int q = 0; q < BT / 4; ++q) {
                    const int c = q / 8, j = 4 * (q % 8);
                    part[q * kBM + row] = make_float4(acc[c][j], acc[c][j + 1], acc[c][j + 2], acc[c][j + 3]);
                }
            }
        }
    }

    ptx::cluster_arrive();                                          // every thread of every CTA, on every path
    ptx::cluster_wait();

    if (warp >= 2) {
        // ---- epilogue, part 2: the sum over the cluster, bias, rounding, transposed store.  The
        // token planes are dealt over the CTAs of the cluster (a reduce-scatter through distributed
        // shared memory): every CTA sums its planes over all ranks, in rank order, and stores them.
        bool all_ok = have_acc && !*abort_flag;
        const uint32_t flag_local = ptx::smem_addr(const_cast<int*>(abort_flag));
        for (uint32_t r = 0; r < splits; ++r)
            if (r != rank) all_ok = all_ok && ld_cluster_u32(ptx::map_to_cta(flag_local, r)) == 0u;
        if (!all_ok && threadIdx.x == 64) atomicOr(status, 1u);
        const int row_in_tile = (warp & 3) * 32 + lane;
        const int64_t feature = static_cast<int64_t>(n_tile) * kBM + row_in_tile;
        if (all_ok && feature < n) {
            const float b = bias != nullptr ? Store<T>::load1(bias + feature) : 0.0f;
            // + bias, rounded; with a residual: + residual[t, feature], rounded again - the roundings of
            // the bias epilogue followed by an elementwise add in the storage type
            auto put = [&](int64_t at, float sum) {
                if (residual == nullptr) Store<T>::store1(y + at, sum + b);
                else Store<T>::store1(y + at, Store<T>::round(sum + b) + Store<T>::load1(residual + at));
            };
            if (splits == 1) {
#pragma unroll
                for (int t = 0; t < BT; ++t)
                    if (t < m) put(static_cast<int64_t>(t) * n + feature, acc[t / 32][t % 32]);
            } else {
                constexpr int kPlanes = BT / 4;
                const int q0 = static_cast<int>(rank) * kPlanes / static_cast<int>(splits);
                const int q1 = (static_cast<int>(rank) + 1) * kPlanes / static_cast<int>(splits);
                for (int q = q0; q < q1 && 4 * q < m; ++q) {
                    const int64_t at = static_cast<int64_t>(4 * q) * n + feature;
                    float res[4] = {0.0f, 0.0f, 0.0f, 0.0f};        // fetched first: they travel while the partials are summed
                    if (residual != nullptr) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (4 * q + j < m) res[j] = Store<T>::load1(residual + at + j * n);
                    }
                    const uint32_t off = static_cast<uint32_t>((q * kBM + row_in_tile) * 16);
                    float4 sum = ld_cluster_f4(ptx::map_to_cta(base, 0) + off);
                    for (uint32_t r = 1; r < splits; ++r) {
                        const float4 v = ld_cluster_f4(ptx::map_to_cta(base, r) + off);
                        sum.x += v.x;
                        sum.y += v.y;
                        sum.z += v.z;
                        sum.w += v.w;
                    }
                    const float out[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (4 * q + j < m)
                            Store<T>::store1(y + at + j * n, residual == nullptr ? out[j] + b : Store<T>::round(out[j] + b) + res[j]);
                }
            }
        }
    }

    ptx::cluster_arrive();                                          // every CTA's shared memory outlives its peers' reads
    ptx::cluster_wait();

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = ptx::globaltimer();
        while (ptx::globaltimer() - t0 < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicOr(status, 1u);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kDecTmemCols);
    }
}

// K split for `tiles` 128-feature tiles: the largest power of two (up to 8) that keeps every CTA
// resident at once (one per SM) and leaves each CTA at least four 64-element slabs.  Clusters that
// run in more than one wave were measured and are not used: 86 tiles (N = 11008) as clusters of 5
// in 3 waves - the shortest schedule on paper, 0.6 of the unsplit time - took 35.5 us against 21.3 us
// unsplit.
inline int decode_split(int64_t tiles, int k_blocks) {
    int s = 1;
    while (s < kSkMaxSplit && tiles * (2 * s) <= sm_count() && k_blocks / (2 * s) >= 4) s *= 2;
    return s;
}

template <typename T, int BT>
cudaError_t launch_decode_bt(const CUtensorMap& tw, const CUtensorMap& tx, const T* bias, const T* residual, T* y,
                             int64_t m, int64_t n, int64_t k_elems, uint32_t fmt, cudaStream_t s) {
    auto kern = gemm_decode_kernel<T, BT>;
    constexpr int kSmem = DecShape<BT>::kSmemBytes;
    static bool configured[kMaxDevices] = {};
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    if (!configured[slot]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return e;
        configured[slot] = true;
    }
    unsigned int* st = status_word();
    if (!st) return cudaErrorMemoryAllocation;
    const int n_tiles = static_cast<int>(ceil_div64(n, kBM));
    const int k_blocks = static_cast<int>((k_elems + 63) / 64);
    const int splits = decode_split(n_tiles, k_blocks);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(n_tiles) * splits);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(splits);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const uint32_t idesc = ptx::instr_desc(fmt, fmt, kBM, BT);
    return cudaLaunchKernelEx(&cfg, kern, tw, tx, bias, residual, y, m, n, k_blocks, idesc, st);
}

// x [m <= 128, k], W [n, k], 16-bit; k % 8 == 0 and 16-byte aligned operands (the caller checked).
// residual [m, n] (optional) is added after the bias epilogue's rounding.
template <typename T>
cudaError_t launch_decode(const void* x, const void* w, const T* bias, T* y, int64_t m, int64_t k, int64_t n,
                          CUtensorMapDataType dt, uint32_t fmt, cudaStream_t s, const T* residual = nullptr) {
    const int bt = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
    CUtensorMap tw, tx;
    cudaError_t e = make_tmap(&tw, dt, 2, w, n, k, kBM);
    if (e != cudaSuccess) return e;
    e = make_tmap(&tx, dt, 2, x, m, k, bt);
    if (e != cudaSuccess) return e;
    switch (bt) {
        case 16: return launch_decode_bt<T, 16>(tw, tx, bias, residual, y, m, n, k, fmt, s);
        case 32: return launch_decode_bt<T, 32>(tw, tx, bias, residual, y, m, n, k, fmt, s);
        case 64: return launch_decode_bt<T, 64>(tw, tx, bias, residual, y, m, n, k, fmt, s);
        default: return launch_decode_bt<T, 128>(tw, tx, bias, residual, y, m, n, k, fmt, s);
    }
}

}  // namespace tc
}  // namespace cck
