// Instantiations of the GEMM kernel (gemm_kernel.cuh): stochastic rounding.
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_sr(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    return fma ? launch_mm<ALGO_SR, true>(p, batch, vec, st) : launch_mm<ALGO_SR, false>(p, batch, vec, st);
}

}  // namespace mpt
