// Instantiations of the GEMM kernel (gemm_kernel.cuh) with 16 x 64 tiles and 1 x 4 outputs per thread, for products
// with a small result and a long K: the weight gradient of a convolution with few channels, and plain products of the
// same shape (the weight gradient of a linear layer over a large batch, the unfold + GEMM form of the same convolution).
//
// The convolution's GEMM has a small result (output channels x input channels * KH * KW: 64 x 576 for a 3 x 3 layer of 64
// channels) and a very long K (images x output positions: 200,704 for batch 64 at 56 x 56), and every output is one
// sequential chain of rounded sums over K, so the only parallelism is across outputs.  128 x 64 tiles make 9 CTAs of
// that layer; 16 x 64 tiles make 36, each with an eighth of the work.  The residency bound differs from the other
// instantiation files', which also keeps this file's kernels distinct instantiations.
#define MPT_MM_TM 1
#define MPT_MM_MIN_CTAS 4
#include "gemm_kernel.cuh"

namespace mpt {

static_assert(BM == kSmallTileRows, "the host side sizes its grid checks with kSmallTileRows");

int launch_mm_small(int algo, bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_mm<ALGO_SEQ, true>(p, batch, vec, st) : launch_mm<ALGO_SEQ, false>(p, batch, vec, st);
    return fma ? launch_mm<ALGO_TILE8, true>(p, batch, vec, st) : launch_mm<ALGO_TILE8, false>(p, batch, vec, st);
}

int launch_conv_wgrad_small_any(int algo, bool fma, const MmParams& p, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_conv_wgrad<ALGO_SEQ, true>(p, st) : launch_conv_wgrad<ALGO_SEQ, false>(p, st);
    return fma ? launch_conv_wgrad<ALGO_TILE8, true>(p, st) : launch_conv_wgrad<ALGO_TILE8, false>(p, st);
}

}  // namespace mpt
