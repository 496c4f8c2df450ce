// GEMMs of the decoder block with the neighbouring elementwise op folded into the
// epilogue (no counterpart in the reference, which runs these as separate kernels:
// examples/llama_block.py:168-172 computes gate_proj, up_proj, swiglu, down_proj and
// the residual add one after the other).
//
//   matmul_swiglu:             y[M,F]  = silu(x @ Wg^T) * (x @ Wu^T)
//   matmul_add_bias_residual:  y[M,N]  = x @ W^T + bias + residual
//
// Both reuse the tcgen05 mainloop of gemm_tcgen05.cuh.  For the SwiGLU form the gate
// and up weights are interleaved in blocks of 128 output features (rows [256j, 256j+128)
// of the fused weight are gate rows [128j, 128j+128), the next 128 rows the matching up
// rows), so one 256-column accumulator tile holds gate columns in its first half and the
// matching up columns in its second half; in the CTA-pair kernel CTA 0 loads the gate
// half and CTA 1 the up half.  The epilogue rounds exactly where the unfused chain
// rounds (GEMM output to the storage type, silu to the storage type, product to the
// storage type; GEMM output to the storage type before the residual add), so the fused
// results equal the unfused ones bit for bit.
//
// Tensor-bound; what the fusion removes is HBM traffic: 2*M*F*sizeof(T) written and
// read again for gate/up, M*N*sizeof(T) written and read again for the residual add.
#include <type_traits>

#include "gemm_decode.cuh"

namespace cck {
namespace tc {

template <typename T>
__device__ __forceinline__ void store32(T* out, const float (&v)[32], int64_t col, int64_t n, int vec_ok) {
    if (vec_ok && col + 32 <= n) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            Vec16 o;
#pragma unroll
            for (int i = 0; i < 4; ++i) o.w[i] = Store<T>::pack2(v[8 * q + 2 * i], v[8 * q + 2 * i + 1]);
            st_stream(out + 8 * q, o);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < n) Store<T>::store1(out + j, v[j]);
    }
}

// ---- epilogue: y = silu(gate) * up, gate = first half of the tile, up = second half
template <typename T>
struct EpiSwiGLU {
    static constexpr bool kPairedHalves = true;
    struct Params {
        T* y;
        int64_t m, f;      // y is [m, f]
        int vec_ok;
    };
    struct Thread {};
    __device__ static __forceinline__ void tile_begin(const Params&, Thread&, const TileWork&, float*, int, int) {}
    __device__ static __forceinline__ void chunk2(const Params& p, Thread&, const TileWork& w, int row_in_tile, int c0,
                                                  float (&gate)[32], float (&up)[32], const float*) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * (kBN / 2) + c0;
        if (row >= p.m || col >= p.f) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) gate[j] = glu1<T>(Store<T>::round(gate[j]), Store<T>::round(up[j]));
        store32<T>(p.y + row * p.f + col, gate, col, p.f, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// ---- epilogue: y = rope(round(acc + bias)) on the columns below rope_cols, round(acc + bias) on the rest
// One projection for q, k and v with the rotary embedding applied where the accumulator is read:
// rows are tokens (row = sequence * seq_len + position), columns are 128-wide heads, element j of
// a head is rotated with element j + 64 (half-split convention, as in rope.cu).  The projection is
// rounded to the storage type before the rotation, so the result equals rope(matmul_add_bias(...))
// bit for bit.
template <typename T>
struct EpiBiasRope {
    static constexpr bool kPairedHalves = true;
    static constexpr int kPairStride = 64;
    struct Params {
        const T* bias;           // [N] or null
        const float* cos_t;      // [seq_len, 64]
        const float* sin_t;
        T* y;                    // [M, N]
        int64_t m, n, rope_cols; // n and rope_cols are multiples of 128
        int seq_len;
        int vec_ok;
    };
    struct Thread { int pos; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int row_in_tile) {
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = static_cast<int64_t>(w.n0) + lane + 32 * i;
            scratch[lane + 32 * i] = (p.bias != nullptr && col < p.n) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
        th.pos = static_cast<int>((static_cast<int64_t>(w.m_tile) * kBM + row_in_tile) % p.seq_len);
    }
    __device__ static __forceinline__ void chunk2(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                  float (&lo)[32], float (&hi)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n0) + c0;          // a head never straddles n: n % 128 == 0
        if (row >= p.m || col >= p.n) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            lo[j] = Store<T>::round(lo[j] + scratch[c0 + j]);
            hi[j] = Store<T>::round(hi[j] + scratch[c0 + 64 + j]);
        }
        if (col < p.rope_cols) {
            const int64_t t = static_cast<int64_t>(th.pos) * 64 + (c0 & 63);
            const float4* cp = reinterpret_cast<const float4*>(p.cos_t + t);
            const float4* sp = reinterpret_cast<const float4*>(p.sin_t + t);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 c = __ldg(cp + q), sn = __ldg(sp + q);
                rope_rotate(lo[4 * q], hi[4 * q], c.x, sn.x, lo[4 * q], hi[4 * q]);
                rope_rotate(lo[4 * q + 1], hi[4 * q + 1], c.y, sn.y, lo[4 * q + 1], hi[4 * q + 1]);
                rope_rotate(lo[4 * q + 2], hi[4 * q + 2], c.z, sn.z, lo[4 * q + 2], hi[4 * q + 2]);
                rope_rotate(lo[4 * q + 3], hi[4 * q + 3], c.w, sn.w, lo[4 * q + 3], hi[4 * q + 3]);
            }
        }
        T* out = p.y + row * p.n + col;
        store32<T>(out, lo, col, p.n, p.vec_ok);
        store32<T>(out + 64, hi, col + 64, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// ---- epilogue: y = round(acc + bias) + residual
template <typename T>
struct EpiBiasResidual {
    struct Params {
        const T* bias;       // [n] or null
        const T* residual;   // [m, n]
        T* y;
        int64_t m, n;
        int vec_ok;
    };
    struct Thread {};
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread&, const TileWork& w, float* scratch,
                                                      int lane, int) {
        const int64_t n0 = static_cast<int64_t>(w.n_tile) * kBN;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            scratch[lane + 32 * i] = (p.bias != nullptr && col < p.n) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread&, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
        const T* res = p.residual + row * p.n + col;
        if (p.vec_ok && col + 32 <= p.n) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float r[8];
                unpack<T>(ld_stream(res + 8 * q), r);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[8 * q + i] = Store<T>::round(acc[8 * q + i] + scratch[c0 + 8 * q + i]) + r[i];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < p.n) acc[j] = Store<T>::round(acc[j] + scratch[c0 + j]) + Store<T>::load1(res + j);
        }
        store32<T>(p.y + row * p.n + col, acc, col, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// ---- epilogue: y = round(acc + bias) (+ residual), and per (row, 256-column tile) statistics of
// the STORED values: sum of squares and largest magnitude.  A row of y spans several tiles, which
// different CTAs compute, so the row-wide reduction is left to the consumer: the statistics go to
// [n_tiles][m] side buffers (tile-major: a warp's 32 rows are 128 contiguous bytes) and the
// RMSNorm / per-token FP8 quantiser that follows reads n_tiles floats per row instead of reducing
// the row itself (launch_rmsnorm_from_stats_fwd, launch_fp8_quant_token_from_amax_fwd).
// Summation order is fixed - columns ascending inside a tile, one fp32 FMA chain per row - so the
// statistics do not depend on the schedule.
template <typename T>
struct EpiBiasResidualStats {
    struct Params {
        const T* bias;       // [n] or null
        const T* residual;   // [m, n] or null
        T* y;
        float* sumsq;        // [n_tiles, m] or null
        float* amax;         // [n_tiles, m] or null
        int64_t m, n;
        int vec_ok;
    };
    struct Thread { float sumsq, amax; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int) {
        const int64_t n0 = static_cast<int64_t>(w.n_tile) * kBN;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            scratch[lane + 32 * i] = (p.bias != nullptr && col < p.n) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
        th.sumsq = 0.0f;
        th.amax = 0.0f;
    }
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
        const bool whole = p.vec_ok && col + 32 <= p.n;
        if (p.residual != nullptr) {
            const T* res = p.residual + row * p.n + col;
            if (whole) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float r[8];
                    unpack<T>(ld_stream(res + 8 * q), r);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        acc[8 * q + i] = Store<T>::round(acc[8 * q + i] + scratch[c0 + 8 * q + i]) + r[i];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col + j < p.n) acc[j] = Store<T>::round(acc[j] + scratch[c0 + j]) + Store<T>::load1(res + j);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] += scratch[c0 + j];
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            acc[j] = Store<T>::round(acc[j]);                  // what the store below writes
            if (whole || col + j < p.n) {
                th.sumsq = fmaf(acc[j], acc[j], th.sumsq);
                th.amax = fmaxf(th.amax, fabsf(acc[j]));
            }
        }
        store32<T>(p.y + row * p.n + col, acc, col, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params& p, Thread& th, const TileWork& w, int row_in_tile) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        if (row >= p.m) return;
        const int64_t at = static_cast<int64_t>(w.n_tile) * p.m + row;
        if (p.sumsq != nullptr) p.sumsq[at] = th.sumsq;
        if (p.amax != nullptr) p.amax[at] = th.amax;
    }
};

// ---- epilogue: y_f32 += acc   (fp32 accumulation across calls, e.g. a weight gradient
// summed over row blocks)
struct EpiAccumF32 {
    struct Params {
        float* y;
        int64_t m, n;
    };
    struct Thread {};
    __device__ static __forceinline__ void tile_begin(const Params&, Thread&, const TileWork&, float*, int, int) {}
    __device__ static __forceinline__ void chunk(const Params& p, Thread&, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float*) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
        float* out = p.y + row * p.n + col;
        if (p.n % 4 == 0 && col + 32 <= p.n) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float4 v = *reinterpret_cast<const float4*>(out + 4 * q);
                v.x += acc[4 * q];
                v.y += acc[4 * q + 1];
                v.z += acc[4 * q + 2];
                v.w += acc[4 * q + 3];
                *reinterpret_cast<float4*>(out + 4 * q) = v;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < p.n) out[j] += acc[j];
        }
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// ---- FP8 operands (e4m3 codes with one scale per A row and per W row), same fusions
// y = round(acc * a_scale[row] * w_scale[col] + bias) + residual: the FP8 GEMM's own epilogue
// (matmul_add_bias.cu) followed by the residual add, rounding where that chain rounds.
template <typename T>
struct EpiScaledBiasResidual {
    struct Params {
        const float* a_scale;   // [m]
        const float* w_scale;   // [n]
        const T* bias;          // [n] or null
        const T* residual;      // [m, n]
        T* y;
        int64_t m, n;
        int vec_ok;
    };
    struct Thread { float a_scale; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int row_in_tile) {
        const int64_t n0 = static_cast<int64_t>(w.n_tile) * kBN;
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
    __device__ static __forceinline__ void chunk(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
        const T* res = p.residual + row * p.n + col;
        if (p.vec_ok && col + 32 <= p.n) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float r[8];
                unpack<T>(ld_stream(res + 8 * q), r);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int j = 8 * q + i;
                    acc[j] = Store<T>::round(fmaf(acc[j] * th.a_scale, scratch[c0 + j], scratch[kBN + c0 + j])) + r[i];
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < p.n)
                    acc[j] = Store<T>::round(fmaf(acc[j] * th.a_scale, scratch[c0 + j], scratch[kBN + c0 + j])) +
                             Store<T>::load1(res + j);
        }
        store32<T>(p.y + row * p.n + col, acc, col, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// y = rope(round(acc * a_scale[row] * w_scale[col] + bias)) on the columns below rope_cols: the FP8 GEMM's
// own epilogue followed by the rotation of EpiBiasRope, rounding where that chain rounds.
template <typename T>
struct EpiScaledBiasRope {
    static constexpr bool kPairedHalves = true;
    static constexpr int kPairStride = 64;
    struct Params {
        const float* a_scale;   // [m]
        const float* w_scale;   // [n]
        const T* bias;          // [n] or null
        const float* cos_t;     // [seq_len, 64]
        const float* sin_t;
        T* y;
        int64_t m, n, rope_cols;
        int seq_len;
        int vec_ok;
    };
    struct Thread { float a_scale; int pos; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int row_in_tile) {
        const int64_t n0 = static_cast<int64_t>(w.n_tile) * kBN;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            const bool in = col < p.n;
            scratch[lane + 32 * i] = in ? p.w_scale[col] : 0.0f;
            scratch[kBN + lane + 32 * i] = (in && p.bias != nullptr) ? Store<T>::load1(p.bias + col) : 0.0f;
        }
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        th.a_scale = row < p.m ? p.a_scale[row] : 0.0f;
        th.pos = static_cast<int>(row % p.seq_len);
    }
    __device__ static __forceinline__ void chunk2(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                  float (&lo)[32], float (&hi)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            lo[j] = Store<T>::round(fmaf(lo[j] * th.a_scale, scratch[c0 + j], scratch[kBN + c0 + j]));
            hi[j] = Store<T>::round(fmaf(hi[j] * th.a_scale, scratch[c0 + 64 + j], scratch[kBN + c0 + 64 + j]));
        }
        if (col < p.rope_cols) {
            const int64_t t = static_cast<int64_t>(th.pos) * 64 + (c0 & 63);
            const float4* cp = reinterpret_cast<const float4*>(p.cos_t + t);
            const float4* sp = reinterpret_cast<const float4*>(p.sin_t + t);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 c = __ldg(cp + q), sn = __ldg(sp + q);
                rope_rotate(lo[4 * q], hi[4 * q], c.x, sn.x, lo[4 * q], hi[4 * q]);
                rope_rotate(lo[4 * q + 1], hi[4 * q + 1], c.y, sn.y, lo[4 * q + 1], hi[4 * q + 1]);
                rope_rotate(lo[4 * q + 2], hi[4 * q + 2], c.z, sn.z, lo[4 * q + 2], hi[4 * q + 2]);
                rope_rotate(lo[4 * q + 3], hi[4 * q + 3], c.w, sn.w, lo[4 * q + 3], hi[4 * q + 3]);
            }
        }
        T* out = p.y + row * p.n + col;
        store32<T>(out, lo, col, p.n, p.vec_ok);
        store32<T>(out + 64, hi, col + 64, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// y = silu(gate) * up with gate / up = acc * a_scale[row] * w_scale[fused weight row], rounded where
// the chain (two FP8 GEMMs, then swiglu) rounds; and, for the per-token quantiser of the down
// projection's input, the largest stored magnitude per row and tile of 128 output columns
// (row_amax [f / 128, m], may be null).
template <typename T>
struct EpiScaledSwiGLU {
    static constexpr bool kPairedHalves = true;
    struct Params {
        const float* a_scale;   // [m]
        const float* w_scale;   // [2 f], in the interleaved row order of the fused weight
        T* y;
        float* amax;            // [f / 128, m] or null
        int64_t m, f;
        int vec_ok;
    };
    struct Thread { float a_scale, amax; };
    __device__ static __forceinline__ void tile_begin(const Params& p, Thread& th, const TileWork& w, float* scratch,
                                                      int lane, int row_in_tile) {
        const int64_t n0 = static_cast<int64_t>(w.n_tile) * kBN;
#pragma unroll
        for (int i = 0; i < kBN / 32; ++i) {
            const int64_t col = n0 + lane + 32 * i;
            scratch[lane + 32 * i] = col < 2 * p.f ? p.w_scale[col] : 0.0f;
        }
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        th.a_scale = row < p.m ? p.a_scale[row] : 0.0f;
        th.amax = 0.0f;
    }
    __device__ static __forceinline__ void chunk2(const Params& p, Thread& th, const TileWork& w, int row_in_tile, int c0,
                                                  float (&gate)[32], float (&up)[32], const float* scratch) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * (kBN / 2) + c0;
        if (row >= p.m || col >= p.f) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float g = Store<T>::round(gate[j] * th.a_scale * scratch[c0 + j]);
            const float u = Store<T>::round(up[j] * th.a_scale * scratch[kBN / 2 + c0 + j]);
            gate[j] = Store<T>::round(glu1<T>(g, u));
            if (col + j < p.f) th.amax = fmaxf(th.amax, fabsf(gate[j]));
        }
        store32<T>(p.y + row * p.f + col, gate, col, p.f, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params& p, Thread& th, const TileWork& w, int row_in_tile) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        if (row < p.m && p.amax != nullptr) p.amax[static_cast<int64_t>(w.n_tile) * p.m + row] = th.amax;
    }
};

// ---- epilogue: y = round(acc), nothing else (the general-layout GEMM below)
template <typename T>
struct EpiStore {
    struct Params {
        T* y;
        int64_t m, n;
        int vec_ok;
    };
    struct Thread {};
    __device__ static __forceinline__ void tile_begin(const Params&, Thread&, const TileWork&, float*, int, int) {}
    __device__ static __forceinline__ void chunk(const Params& p, Thread&, const TileWork& w, int row_in_tile, int c0,
                                                 float (&acc)[32], const float*) {
        const int64_t row = static_cast<int64_t>(w.m_tile) * kBM + row_in_tile;
        const int64_t col = static_cast<int64_t>(w.n_tile) * kBN + c0;
        if (row >= p.m || col >= p.n) return;
        store32<T>(p.y + row * p.n + col, acc, col, p.n, p.vec_ok);
    }
    __device__ static __forceinline__ void tile_end(const Params&, Thread&, const TileWork&, int) {}
};

// y[m, n] = op(a) op(b)^T with either operand stored as it is (K-major: a [m, k], b [n, k]) or
// transposed (MN-major: a [k, m], b [k, n]); see the layout note at the top of gemm_tcgen05.cuh.
template <typename T, class Epi, int kMajors>
cudaError_t run_general(const void* a, const void* b, int64_t m, int64_t k, int64_t n, const typename Epi::Params& ep,
                        cudaStream_t s) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr bool a_mn = (kMajors & kAMn) != 0, b_mn = (kMajors & kBMn) != 0;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int m_tiles = static_cast<int>(ceil_div64(m, kBM)), n_tiles = static_cast<int>(ceil_div64(n, kBN));
    const uint32_t fmt = is_bf16 ? 1u : 0u;
    const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<false, SchedGemm, Epi, kMajors>() > 0;
    CUtensorMap ta, tb;
    cudaError_t e = a_mn ? make_tmap_mn(&ta, dt, a, k, m) : make_tmap(&ta, dt, 2, a, m, k, kBM);
    if (e != cudaSuccess) return e;
    e = b_mn ? make_tmap_mn(&tb, dt, b, k, n) : make_tmap(&tb, dt, 2, b, n, k, pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    if (pair) {
        const int m_pairs = (m_tiles + 1) / 2;
        SchedGemm::Params sp{m_pairs, n_tiles, raster_group(2 * kBM, k, 2, m_pairs)};
        return launch_pair<false, SchedGemm, Epi, kMajors>(ta, tb, sp, ep, k,
                                                            ptx::instr_desc(fmt, fmt, 2 * kBM, kBN, a_mn, b_mn),
                                                            static_cast<int64_t>(m_pairs) * n_tiles, s);
    }
    SchedGemm::Params sp{m_tiles, n_tiles, raster_group(kBM, k, 2, m_tiles)};
    const int64_t tiles = static_cast<int64_t>(m_tiles) * n_tiles;
    const int ctas = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    return launch<false, SchedGemm, Epi, kBN, kMajors>(ta, tb, sp, ep, k, ptx::instr_desc(fmt, fmt, kBM, kBN, a_mn, b_mn),
                                                       ctas, s);
}

// e4m3 operands; pair kernel when the problem has at least two row tiles, else the single-CTA kernel
template <class Epi>
cudaError_t run_fused_fp8(const uint8_t* a, const uint8_t* w, int64_t m, int64_t k, int64_t n_rows_of_w,
                          const typename Epi::Params& ep, cudaStream_t s) {
    const int m_tiles = static_cast<int>(ceil_div64(m, kBM)), n_tiles = static_cast<int>(ceil_div64(n_rows_of_w, kBN));
    const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<true, SchedGemm, Epi>() > 0;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, m, k, kBM);
    if (e != cudaSuccess) return e;
    e = make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, n_rows_of_w, k, pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    const int m_units = pair ? (m_tiles + 1) / 2 : m_tiles;
    SchedGemm::Params sp{m_units, n_tiles, raster_group(pair ? 2 * kBM : kBM, k, 1, m_units)};
    const int64_t tiles = static_cast<int64_t>(m_units) * n_tiles;
    const uint32_t idesc = ptx::instr_desc(0u, 0u, pair ? 2 * kBM : kBM, kBN);
    if (pair) return launch_pair<true, SchedGemm, Epi>(ta, tb, sp, ep, k, idesc, tiles, s);
    return launch<true, SchedGemm, Epi>(ta, tb, sp, ep, k, idesc, static_cast<int>(tiles < sm_count() ? tiles : sm_count()), s);
}

template <typename T, class Epi>
cudaError_t run_general_majors(const void* a, const void* b, int64_t m, int64_t k, int64_t n, int a_is_km, int b_is_kn,
                               const typename Epi::Params& ep, cudaStream_t s) {
    if (a_is_km && b_is_kn) return run_general<T, Epi, kAMn | kBMn>(a, b, m, k, n, ep, s);
    if (b_is_kn) return run_general<T, Epi, kBMn>(a, b, m, k, n, ep, s);
    if (a_is_km) return run_general<T, Epi, kAMn>(a, b, m, k, n, ep, s);
    return run_general<T, Epi, 0>(a, b, m, k, n, ep, s);
}

inline bool tc_shape_ok(const void* a, const void* b, int64_t m, int64_t k, int64_t n) {
    return k % 8 == 0 && k >= 8 && aligned16(a) && aligned16(b) && m < (1LL << 31) && n < (1LL << 31) &&
           k < (1LL << 31);
}

template <typename T, class Epi>
cudaError_t run_fused(const void* x, const void* w, int64_t m, int64_t k, int64_t n_rows_of_w,
                      const typename Epi::Params& ep, cudaStream_t s) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int m_tiles = static_cast<int>(ceil_div64(m, kBM)), n_tiles = static_cast<int>(ceil_div64(n_rows_of_w, kBN));
    const uint32_t fmt = is_bf16 ? 1u : 0u;
    const bool pair = m_tiles >= 2 && pair_kernels_enabled() && max_pairs<false, SchedGemm, Epi>() > 0;
    CUtensorMap ta, tb;
    cudaError_t e = make_tmap(&ta, dt, 2, x, m, k, kBM);
    if (e != cudaSuccess) return e;
    e = make_tmap(&tb, dt, 2, w, n_rows_of_w, k, pair ? 128 : kBN);
    if (e != cudaSuccess) return e;
    if (pair) {
        const int m_pairs = (m_tiles + 1) / 2;
        SchedGemm::Params sp{m_pairs, n_tiles, raster_group(2 * kBM, k, 2, m_pairs)};
        return launch_pair<false, SchedGemm, Epi>(ta, tb, sp, ep, k, ptx::instr_desc(fmt, fmt, 2 * kBM, kBN),
                                                  static_cast<int64_t>(m_pairs) * n_tiles, s);
    }
    SchedGemm::Params sp{m_tiles, n_tiles, raster_group(kBM, k, 2, m_tiles)};
    const int64_t tiles = static_cast<int64_t>(m_tiles) * n_tiles;
    const int ctas = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    return launch<false, SchedGemm, Epi>(ta, tb, sp, ep, k, ptx::instr_desc(fmt, fmt, kBM, kBN), ctas, s);
}

}  // namespace tc
}  // namespace cck

extern "C" int32_t launch_matmul_swiglu_fwd(const void* x, const void* w_gate_up, void* y, int64_t m, int64_t k,
                                            int64_t f, int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || f <= 0) return cudaSuccess;
    if (f % 128 != 0 || !tc_shape_ok(x, w_gate_up, m, k, 2 * f)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = (f % 8 == 0 && aligned16(y)) ? 1 : 0;
    if (dtype == kBF16) {
        EpiSwiGLU<__nv_bfloat16>::Params ep{static_cast<__nv_bfloat16*>(y), m, f, vec_ok};
        return run_fused<__nv_bfloat16, EpiSwiGLU<__nv_bfloat16>>(x, w_gate_up, m, k, 2 * f, ep, s);
    }
    if (dtype == kF16) {
        EpiSwiGLU<__half>::Params ep{static_cast<__half*>(y), m, f, vec_ok};
        return run_fused<__half, EpiSwiGLU<__half>>(x, w_gate_up, m, k, 2 * f, ep, s);
    }
    return cudaErrorInvalidValue;
}

extern "C" int32_t launch_matmul_add_bias_rope_fwd(const void* x, const void* weight, const void* bias,
                                                   const float* cos_table, const float* sin_table, void* y, int64_t m,
                                                   int64_t k, int64_t n, int64_t rope_cols, int64_t seq_len,
                                                   int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (cos_table == nullptr || sin_table == nullptr || n % 128 != 0 || rope_cols % 128 != 0 || rope_cols < 0 ||
        rope_cols > n || seq_len <= 0 || seq_len >= (1LL << 31) || !aligned16(cos_table) || !aligned16(sin_table) ||
        !tc_shape_ok(x, weight, m, k, n))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = aligned16(y) ? 1 : 0;
    if (dtype == kBF16) {
        EpiBiasRope<__nv_bfloat16>::Params ep{static_cast<const __nv_bfloat16*>(bias), cos_table, sin_table,
                                              static_cast<__nv_bfloat16*>(y), m, n, rope_cols, static_cast<int>(seq_len), vec_ok};
        return run_fused<__nv_bfloat16, EpiBiasRope<__nv_bfloat16>>(x, weight, m, k, n, ep, s);
    }
    if (dtype == kF16) {
        EpiBiasRope<__half>::Params ep{static_cast<const __half*>(bias), cos_table, sin_table, static_cast<__half*>(y),
                                       m, n, rope_cols, static_cast<int>(seq_len), vec_ok};
        return run_fused<__half, EpiBiasRope<__half>>(x, weight, m, k, n, ep, s);
    }
    return cudaErrorInvalidValue;
}

extern "C" int32_t launch_matmul_add_bias_residual_fwd(const void* x, const void* weight, const void* bias,
                                                       const void* residual, void* y, int64_t m, int64_t k,
                                                       int64_t n, int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (residual == nullptr || !tc_shape_ok(x, weight, m, k, n)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = (n % 8 == 0 && aligned16(y) && aligned16(residual)) ? 1 : 0;
    if (dtype == kBF16) {
        if (m <= kDecMaxTokens && splitk_enabled(m))        // decode-sized batch: weight rows on the M side, K split over a cluster
            return launch_decode<__nv_bfloat16>(x, weight, static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y),
                                                m, k, n, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 1u, s,
                                                static_cast<const __nv_bfloat16*>(residual));
        EpiBiasResidual<__nv_bfloat16>::Params ep{static_cast<const __nv_bfloat16*>(bias),
                                                  static_cast<const __nv_bfloat16*>(residual),
                                                  static_cast<__nv_bfloat16*>(y), m, n, vec_ok};
        return run_fused<__nv_bfloat16, EpiBiasResidual<__nv_bfloat16>>(x, weight, m, k, n, ep, s);
    }
    if (dtype == kF16) {
        if (m <= kDecMaxTokens && splitk_enabled(m))
            return launch_decode<__half>(x, weight, static_cast<const __half*>(bias), static_cast<__half*>(y), m, k, n,
                                         CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 0u, s, static_cast<const __half*>(residual));
        EpiBiasResidual<__half>::Params ep{static_cast<const __half*>(bias), static_cast<const __half*>(residual),
                                           static_cast<__half*>(y), m, n, vec_ok};
        return run_fused<__half, EpiBiasResidual<__half>>(x, weight, m, k, n, ep, s);
    }
    return cudaErrorInvalidValue;
}

// y = x @ weight^T + bias (+ residual when not NULL), bit for bit what launch_matmul_add_bias_fwd
// (launch_matmul_add_bias_residual_fwd) stores, plus the per-(row, 256-column tile) statistics of the
// stored values the next op needs: row_sumsq / row_amax are [cck_gemm_stat_tiles(n), m] float32,
// either may be NULL.
extern "C" int64_t cck_gemm_stat_tiles(int64_t n) { return n <= 0 ? 0 : (n + cck::tc::kBN - 1) / cck::tc::kBN; }

extern "C" int32_t launch_matmul_add_bias_stats_fwd(const void* x, const void* weight, const void* bias,
                                                    const void* residual, void* y, float* row_sumsq, float* row_amax,
                                                    int64_t m, int64_t k, int64_t n, int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (!tc_shape_ok(x, weight, m, k, n)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = (n % 8 == 0 && aligned16(y) && (residual == nullptr || aligned16(residual))) ? 1 : 0;
    if (dtype == kBF16) {
        using T = __nv_bfloat16;
        EpiBiasResidualStats<T>::Params ep{static_cast<const T*>(bias), static_cast<const T*>(residual),
                                           static_cast<T*>(y), row_sumsq, row_amax, m, n, vec_ok};
        return run_fused<T, EpiBiasResidualStats<T>>(x, weight, m, k, n, ep, s);
    }
    if (dtype == kF16) {
        using T = __half;
        EpiBiasResidualStats<T>::Params ep{static_cast<const T*>(bias), static_cast<const T*>(residual),
                                           static_cast<T*>(y), row_sumsq, row_amax, m, n, vec_ok};
        return run_fused<T, EpiBiasResidualStats<T>>(x, weight, m, k, n, ep, s);
    }
    return cudaErrorInvalidValue;
}

// y_f32[m, n] += x[m, k] @ weight[n, k]^T: 16-bit operands, fp32 output accumulated in place
// across calls (no counterpart in the reference).  y must be 16-byte aligned.
extern "C" int32_t launch_matmul_accumulate_f32_fwd(const void* x, const void* weight, float* y, int64_t m, int64_t k,
                                                    int64_t n, int32_t dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (!tc_shape_ok(x, weight, m, k, n) || !aligned16(y)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EpiAccumF32::Params ep{y, m, n};
    if (dtype == kBF16) return run_fused<__nv_bfloat16, EpiAccumF32>(x, weight, m, k, n, ep, s);
    if (dtype == kF16) return run_fused<__half, EpiAccumF32>(x, weight, m, k, n, ep, s);
    return cudaErrorInvalidValue;
}

// y[m, n] = A B^T where A is stored [m, k] (a_is_km = 0) or transposed as [k, m] (a_is_km = 1)
// and B is stored [n, k] (b_is_kn = 0, the nn.Linear layout) or transposed as [k, n] (b_is_kn = 1):
// the gradient GEMMs dX = dY W (B transposed) and dW = dY^T X (both transposed) read their
// operands as stored, through MN-major tensor-core descriptors - no transposed copies.
// accumulate_f32 = 0: y is in `dtype`, overwritten; 1: y is float32 and the product is added to
// it (a weight gradient summed over row chunks).  float16 / bfloat16.  The contiguous dimension
// of every operand must be a multiple of 8 elements (K for a K-major operand, M or N for a
// transposed one), pointers 16-byte aligned; otherwise cudaErrorInvalidValue.
extern "C" int32_t launch_matmul_general_fwd(const void* a, const void* b, void* y, int64_t m, int64_t k, int64_t n,
                                             int32_t a_is_km, int32_t b_is_kn, int32_t accumulate_f32, int32_t dtype,
                                             void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (!aligned16(a) || !aligned16(b) || !aligned16(y) || m >= (1LL << 31) || n >= (1LL << 31) || k >= (1LL << 31))
        return cudaErrorInvalidValue;
    if ((a_is_km ? m : k) % 8 != 0 || (b_is_kn ? n : k) % 8 != 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype != kBF16 && dtype != kF16) return cudaErrorInvalidValue;
    if (accumulate_f32) {
        EpiAccumF32::Params ep{static_cast<float*>(y), m, n};
        return dtype == kBF16 ? run_general_majors<__nv_bfloat16, EpiAccumF32>(a, b, m, k, n, a_is_km, b_is_kn, ep, s)
                              : run_general_majors<__half, EpiAccumF32>(a, b, m, k, n, a_is_km, b_is_kn, ep, s);
    }
    const int vec_ok = n % 8 == 0 ? 1 : 0;
    if (dtype == kBF16) {
        EpiStore<__nv_bfloat16>::Params ep{static_cast<__nv_bfloat16*>(y), m, n, vec_ok};
        return run_general_majors<__nv_bfloat16, EpiStore<__nv_bfloat16>>(a, b, m, k, n, a_is_km, b_is_kn, ep, s);
    }
    EpiStore<__half>::Params ep{static_cast<__half*>(y), m, n, vec_ok};
    return run_general_majors<__half, EpiStore<__half>>(a, b, m, k, n, a_is_km, b_is_kn, ep, s);
}

// FP8 forms of the two fused projections (e4m3 codes, per-row scales of both operands; K a multiple
// of 16, 16-byte aligned codes; otherwise cudaErrorInvalidValue).  Results equal, bit for bit, the
// chain launch_matmul_add_bias_fp8_fwd -> (swiglu | residual add) of this library.
//   launch_matmul_swiglu_fp8_fwd: w_gate_up [2 f, k] interleaved as for launch_matmul_swiglu_fwd, w_scale
//       [2 f] in the same row order; row_amax [f / 128, m] (or NULL) receives the largest magnitude of
//       every row of y per 128 output columns, for launch_fp8_quant_token_from_amax_fwd.
extern "C" int32_t launch_matmul_swiglu_fp8_fwd(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_gate_up,
                                                const float* w_scale, void* y, float* row_amax, int64_t m, int64_t k,
                                                int64_t f, int32_t out_dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || f <= 0) return cudaSuccess;
    if (f % 128 != 0 || k % 16 != 0 || !aligned16(a_codes) || !aligned16(w_gate_up) || m >= (1LL << 31) ||
        f >= (1LL << 30) || k >= (1LL << 31))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = (f % 8 == 0 && aligned16(y)) ? 1 : 0;
    if (out_dtype == kBF16) {
        using T = __nv_bfloat16;
        EpiScaledSwiGLU<T>::Params ep{a_scale, w_scale, static_cast<T*>(y), row_amax, m, f, vec_ok};
        return run_fused_fp8<EpiScaledSwiGLU<T>>(a_codes, w_gate_up, m, k, 2 * f, ep, s);
    }
    if (out_dtype == kF16) {
        using T = __half;
        EpiScaledSwiGLU<T>::Params ep{a_scale, w_scale, static_cast<T*>(y), row_amax, m, f, vec_ok};
        return run_fused_fp8<EpiScaledSwiGLU<T>>(a_codes, w_gate_up, m, k, 2 * f, ep, s);
    }
    return cudaErrorInvalidValue;
}

extern "C" int32_t launch_matmul_add_bias_rope_fp8_fwd(const uint8_t* a_codes, const float* a_scale,
                                                       const uint8_t* w_codes, const float* w_scale, const void* bias,
                                                       const float* cos_table, const float* sin_table, void* y,
                                                       int64_t m, int64_t k, int64_t n, int64_t rope_cols,
                                                       int64_t seq_len, int32_t out_dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (cos_table == nullptr || sin_table == nullptr || n % 128 != 0 || rope_cols % 128 != 0 || rope_cols < 0 ||
        rope_cols > n || seq_len <= 0 || seq_len >= (1LL << 31) || !aligned16(cos_table) || !aligned16(sin_table) ||
        k % 16 != 0 || !aligned16(a_codes) || !aligned16(w_codes) || m >= (1LL << 31) || n >= (1LL << 31) ||
        k >= (1LL << 31))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = aligned16(y) ? 1 : 0;
    if (out_dtype == kBF16) {
        using T = __nv_bfloat16;
        EpiScaledBiasRope<T>::Params ep{a_scale, w_scale, static_cast<const T*>(bias), cos_table, sin_table,
                                        static_cast<T*>(y), m, n, rope_cols, static_cast<int>(seq_len), vec_ok};
        return run_fused_fp8<EpiScaledBiasRope<T>>(a_codes, w_codes, m, k, n, ep, s);
    }
    if (out_dtype == kF16) {
        using T = __half;
        EpiScaledBiasRope<T>::Params ep{a_scale, w_scale, static_cast<const T*>(bias), cos_table, sin_table,
                                        static_cast<T*>(y), m, n, rope_cols, static_cast<int>(seq_len), vec_ok};
        return run_fused_fp8<EpiScaledBiasRope<T>>(a_codes, w_codes, m, k, n, ep, s);
    }
    return cudaErrorInvalidValue;
}

extern "C" int32_t launch_matmul_add_bias_residual_fp8_fwd(const uint8_t* a_codes, const float* a_scale,
                                                           const uint8_t* w_codes, const float* w_scale,
                                                           const void* bias, const void* residual, void* y, int64_t m,
                                                           int64_t k, int64_t n, int32_t out_dtype, void* stream) {
    using namespace cck;
    using namespace cck::tc;
    if (m <= 0 || k <= 0 || n <= 0) return cudaSuccess;
    if (residual == nullptr || k % 16 != 0 || !aligned16(a_codes) || !aligned16(w_codes) || m >= (1LL << 31) ||
        n >= (1LL << 31) || k >= (1LL << 31))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec_ok = (n % 8 == 0 && aligned16(y) && aligned16(residual)) ? 1 : 0;
    if (out_dtype == kBF16) {
        using T = __nv_bfloat16;
        EpiScaledBiasResidual<T>::Params ep{a_scale, w_scale, static_cast<const T*>(bias), static_cast<const T*>(residual),
                                            static_cast<T*>(y), m, n, vec_ok};
        return run_fused_fp8<EpiScaledBiasResidual<T>>(a_codes, w_codes, m, k, n, ep, s);
    }
    if (out_dtype == kF16) {
        using T = __half;
        EpiScaledBiasResidual<T>::Params ep{a_scale, w_scale, static_cast<const T*>(bias), static_cast<const T*>(residual),
                                            static_cast<T*>(y), m, n, vec_ok};
        return run_fused_fp8<EpiScaledBiasResidual<T>>(a_codes, w_codes, m, k, n, ep, s);
    }
    return cudaErrorInvalidValue;
}
