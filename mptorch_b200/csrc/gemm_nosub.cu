// Instantiations of the GEMM kernel (gemm_kernel.cuh): float formats without subnormals (the default of the
// reference's FloatingPoint), both accumulation orders, on the range-checked path with the rounding that settles what
// lands below the smallest normal value (fast_rn_nosub in cast.cuh).
#include "gemm_kernel.cuh"

namespace mpt {

int launch_mm_nosub(int algo, bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_mm_nosub_t<ALGO_SEQ, true>(p, batch, vec, st) : launch_mm_nosub_t<ALGO_SEQ, false>(p, batch, vec, st);
    return fma ? launch_mm_nosub_t<ALGO_TILE8, true>(p, batch, vec, st) : launch_mm_nosub_t<ALGO_TILE8, false>(p, batch, vec, st);
}

}  // namespace mpt
