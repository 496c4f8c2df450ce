// Host side of TMA: the driver's tensor-map encoder, looked up through the runtime so that
// the library needs no link-time dependency on libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace cck {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Device word that collects wait time-outs of kernels that wait on mbarriers
// (bit 0: tensor-core GEMM kernels, bit 1: TMA-staged FP8 block quantisation).
unsigned int* status_word();

}  // namespace tc
}  // namespace cck
