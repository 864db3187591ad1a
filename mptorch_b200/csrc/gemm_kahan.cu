// Instantiations of the GEMM kernel (gemm_kernel.cuh): Kahan-compensated accumulation.
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_kahan(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    return fma ? launch_mm<ALGO_KAHAN, true>(p, batch, vec, st) : launch_mm<ALGO_KAHAN, false>(p, batch, vec, st);
}

}  // namespace mpt
