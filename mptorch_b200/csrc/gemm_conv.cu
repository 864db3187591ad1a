// Instantiations of the GEMM kernel (gemm_kernel.cuh): convolution as an implicit GEMM, both accumulation orders.
#include "gemm_kernel.cuh"

namespace mpt {

int launch_conv_any(int algo, bool fma, const MmParams& p, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_conv<ALGO_SEQ, true>(p, st) : launch_conv<ALGO_SEQ, false>(p, st);
    return fma ? launch_conv<ALGO_TILE8, true>(p, st) : launch_conv<ALGO_TILE8, false>(p, st);
}

int launch_conv_wgrad_any(int algo, bool fma, const MmParams& p, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_conv_wgrad<ALGO_SEQ, true>(p, st) : launch_conv_wgrad<ALGO_SEQ, false>(p, st);
    return fma ? launch_conv_wgrad<ALGO_TILE8, true>(p, st) : launch_conv_wgrad<ALGO_TILE8, false>(p, st);
}

}  // namespace mpt
