// Split-K GEMM for decode-sized problems: y[M,N] = x[M,K] @ W[N,K]^T + bias with so few output
// tiles that one CTA per tile leaves most of the GPU idle and the weight matrix arrives at a
// fraction of the HBM rate.  A thread-block CLUSTER of S CTAs shares one 128 x 64 output tile:
// CTA r of the cluster contracts the r-th slice of K into its own tensor memory (same TMA ->
// mbarrier ring -> tcgen05.mma pipeline as gemm_tcgen05.cuh), then the partial accumulators
// meet on chip - every non-leader CTA parks its 128 x 64 fp32 partial in its own shared
// memory (the stage ring is free by then), a cluster barrier publishes them, and the leader's
// epilogue threads read them through distributed shared memory, add them in rank order to
// their own accumulator, add the bias, round once and store.  No workspace, no atomics: the
// result does not depend on timing, and launches on different streams do not share state.
//
// Waits: the mbarrier waits are the bounded ones of ptx.cuh; the two cluster barriers are
// reached by every thread of every CTA on every path (a role that gave up still arrives).
// If any CTA of the cluster gave up, the leader stores nothing for that tile and bit 0 of the
// status word is set.
#pragma once

#include "gemm_tcgen05.cuh"

namespace cck {
namespace tc {

constexpr int kSkBN = 64;
constexpr int kSkStages = 4;
constexpr int kSkStageBytes = kABytes + kSkBN * kRowBytes;       // 24 KiB
constexpr int kSkSmemBytes = kSkStages * kSkStageBytes + 1024 + 256;
constexpr int kSkMaxSplit = 8;

__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t cluster_addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const T* __restrict__ bias, T* __restrict__ y, int64_t m, int64_t n, int n_tiles, int k_blocks,
                   uint32_t idesc, int vec_ok, unsigned int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);
    const uint32_t bar0 = base + kSkStages * kSkStageBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kSkStages + s); };
    const uint32_t tfull_bar = bar0 + 8u * (2 * kSkStages);
    uint8_t* misc = gen + kSkStages * kSkStageBytes + 8 * (2 * kSkStages + 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank(), splits = cluster_nctarank();
    const int tile = blockIdx.x / splits;
    const int m_tile = tile / n_tiles, n_tile = tile - m_tile * n_tiles;
    const int kb0 = static_cast<int>((static_cast<int64_t>(rank) * k_blocks) / splits);
    const int kb1 = static_cast<int>((static_cast<int64_t>(rank + 1) * k_blocks) / splits);   // kb1 > kb0: k_blocks >= splits

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSkStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kSkBN);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    float acc[2][32];                                  // this epilogue thread's row of the tile
    bool have_acc = false;
    if (warp == 0) {
        if (lane == 0) {                               // ---- TMA producer
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status)) break;
                ptx::mbar_arrive_expect_tx(full_bar(stage), kSkStageBytes);
                const uint32_t a_dst = base + stage * kSkStageBytes;
                ptx::tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * 64, m_tile * kBM);
                ptx::tma_load_2d(a_dst + kABytes, &tmap_b, full_bar(stage), kb * 64, n_tile * kSkBN);
                if (++stage == kSkStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                               // ---- MMA issuer
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag, status)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t a_src = base + stage * kSkStageBytes;
                const uint64_t da = ptx::smem_desc_k_sw128(a_src);
                const uint64_t db = ptx::smem_desc_k_sw128(a_src + kABytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    ptx::mma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
                ptx::mma_commit(empty_bar(stage));
                if (++stage == kSkStages) { stage = 0; phase ^= 1u; }
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
            ptx::tmem_ld32(t0, acc[0]);
            ptx::tmem_ld32(t0 + 32, acc[1]);
            have_acc = true;
            if (rank != 0) {
                // park it as 16 float4 planes [plane][row]: consecutive rows are 16 bytes apart, so
                // both this store and the leader's remote load are contiguous across a warp
                float4* part = reinterpret_cast<float4*>(gen);
                const int row = quarter * 32 + lane;
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        part[(c * 8 + q) * kBM + row] =
                            make_float4(acc[c][4 * q], acc[c][4 * q + 1], acc[c][4 * q + 2], acc[c][4 * q + 3]);
            }
        }
    }

    // every thread of every CTA of the cluster, on every path
    ptx::cluster_arrive();
    ptx::cluster_wait();

    // a peer whose wait ran out parked nothing: its abort flag (raised before it arrived at the
    // barrier above) tells the leader to leave the tile unwritten and report instead
    bool peers_ok = true;
    if (rank == 0 && warp >= 2) {
        const uint32_t flag_local = ptx::smem_addr(const_cast<int*>(abort_flag));
        for (uint32_t r = 1; r < splits; ++r) peers_ok = peers_ok && ld_cluster_u32(ptx::map_to_cta(flag_local, r)) == 0u;
        if (!peers_ok && threadIdx.x == 64) atomicOr(status, 1u);
    }
    if (rank == 0 && warp >= 2 && have_acc && !*abort_flag && peers_ok) {
        // ---- epilogue, part 2 (leader): add the peers' partials in rank order, bias, round, store
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t part_local = base;              // same offset in every CTA of the cluster
        for (uint32_t r = 1; r < splits; ++r) {
            const uint32_t remote = ptx::map_to_cta(part_local, r);
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float4 v = ld_cluster_f4(remote + static_cast<uint32_t>(((c * 8 + q) * kBM + row_in_tile) * 16));
                    acc[c][4 * q] += v.x;
                    acc[c][4 * q + 1] += v.y;
                    acc[c][4 * q + 2] += v.z;
                    acc[c][4 * q + 3] += v.w;
                }
        }
        const int64_t row = static_cast<int64_t>(m_tile) * kBM + row_in_tile;
        if (row < m) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int64_t col = static_cast<int64_t>(n_tile) * kSkBN + 32 * c;
                if (col >= n) continue;
                if (bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col + j < n) acc[c][j] += Store<T>::load1(bias + col + j);
                }
                T* out = y + row * n + col;
                if (vec_ok && col + 32 <= n) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        Vec16 o;
#pragma unroll
                        for (int q = 0; q < 4; ++q) o.w[q] = Store<T>::pack2(acc[c][8 * v + 2 * q], acc[c][8 * v + 2 * q + 1]);
                        st_stream(out + 8 * v, o);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col + j < n) Store<T>::store1(out + j, acc[c][j]);
                }
            }
        }
    }

    // the peers' shared memory must outlive the leader's reads
    ptx::cluster_arrive();
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
        ptx::tmem_dealloc(tmem_base, kSkBN);
    }
}

// Split factor for a problem of `tiles` 128 x 64 output tiles and `k_blocks` 64-element K slabs:
// the largest power of two (2, 4, 8) that keeps every CTA resident at once (two per SM) and
// leaves each CTA at least four slabs; 1 = do not split.
inline int splitk_factor(int64_t tiles, int k_blocks) {
    int s = 1;
    while (s < kSkMaxSplit && tiles * (2 * s) <= 2 * static_cast<int64_t>(sm_count()) && k_blocks / (2 * s) >= 4) s *= 2;
    return s;
}

template <typename T>
cudaError_t launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const T* bias, T* y, int64_t m, int64_t n,
                          int m_tiles, int n_tiles, int64_t k_elems, uint32_t idesc, int vec_ok, int splits,
                          cudaStream_t s) {
    auto kern = gemm_splitk_kernel<T>;
    static bool configured[kMaxDevices] = {};
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    if (!configured[slot]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemBytes);
        if (e != cudaSuccess) return e;
        configured[slot] = true;
    }
    unsigned int* st = status_word();
    if (!st) return cudaErrorMemoryAllocation;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(m_tiles) * n_tiles * splits);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSkSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(splits);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const int k_blocks = static_cast<int>((k_elems + 63) / 64);
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, bias, y, m, n, n_tiles, k_blocks, idesc, vec_ok, st);
}

}  // namespace tc
}  // namespace cck
