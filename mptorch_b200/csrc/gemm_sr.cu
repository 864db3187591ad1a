// Instantiations of the GEMM kernel (gemm_kernel.cuh): stochastic rounding.
//
// This kernel is bound by the latency of its Philox chains (ten dependent rounds per call), not by registers' worth of
// outputs per thread: 64 x 64 tiles with 4 x 4 outputs per thread fit 128 registers, so two CTAs (16 warps) share an
// SM and cover those latencies, where the 128 x 64 tile of the other kernels needs all 255 registers for one CTA.
#define MPT_MM_TM 4
#define MPT_MM_SR_MIN_CTAS 2
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_sr(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    return fma ? launch_mm<ALGO_SR, true>(p, batch, vec, st) : launch_mm<ALGO_SR, false>(p, batch, vec, st);
}

}  // namespace mpt
