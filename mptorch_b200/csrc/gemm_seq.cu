// Instantiations of the GEMM kernel (gemm_kernel.cuh): sequential accumulation order.
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_seq(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    return fma ? launch_mm<ALGO_SEQ, true>(p, batch, vec, st) : launch_mm<ALGO_SEQ, false>(p, batch, vec, st);
}

}  // namespace mpt
