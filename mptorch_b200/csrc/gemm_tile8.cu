// Instantiations of the GEMM kernel (gemm_kernel.cuh): the reference CUDA kernels' 8-wide tiled order.
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_tile8(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    return fma ? launch_mm<ALGO_TILE8, true>(p, batch, vec, st) : launch_mm<ALGO_TILE8, false>(p, batch, vec, st);
}

}  // namespace mpt
