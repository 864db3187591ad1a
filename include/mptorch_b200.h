/*
 * mptorch_b200.h -- C ABI of the B200 (sm_100a) simulated-arithmetic kernels.
 *
 * Drop-in boundary: each entry point below replaces one function of the reference's
 * `quant_cuda` pybind11 module (mptorch/quant/quant_cuda/pybind_cuda.cpp); the citation
 * beside each declaration names the registration it stands in for.  Signatures carry only
 * plain pointers, sizes and format parameters: no torch types.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer to fp32 data in row-major contiguous layout unless
 *     stated otherwise; inputs are never modified; outputs are fully overwritten (no
 *     pre-zeroing needed, unlike the reference);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); all
 *     work is enqueued on it and the call returns without synchronising;
 *   - the current CUDA device must be the one that owns the pointers;
 *   - a format is (man, exp, subnormals, saturate): mantissa bits 0..23 (hidden bit not
 *     counted), exponent bits 1..8, and two flags (0/1);
 *   - no entry point allocates or frees device memory; where scratch space is needed the
 *     caller passes it as `workspace`;
 *   - return value: MPT_OK, or an error code; mpt_last_error() gives a message for the
 *     calling thread.
 */
#ifndef MPTORCH_B200_H
#define MPTORCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MPT_API __attribute__((visibility("default")))
#else
#define MPT_API
#endif

enum {
    MPT_OK = 0,
    MPT_ERR_INVALID_ARGUMENT = 1,
    MPT_ERR_CUDA = 2,
    MPT_ERR_WORKSPACE = 3
};

/* rounding modes of the elementwise quantizers */
enum { MPT_RND_NEAREST = 0, MPT_RND_STOCHASTIC = 1, MPT_RND_TRUNCATE = 2 };

/* binary8 overflow policies; values match the reference's OverflowPolicy enum
 * (quant_cuda/binary8_kernel.h:20-25, registered at pybind_cuda.cpp:784-787) */
enum { MPT_SATURATE_INFTY = 0, MPT_SATURATE_MAXFLOAT = 1, MPT_SATURATE_MAXFLOAT2 = 2 };

/* K-accumulation order of the GEMMs and association of the row reductions.
 *   MPT_ORDER_SEQ  : strictly sequential, what the reference CPU path computes
 *                    (quant_cpu/mm_kernel.h:9-20, softmax.h, layernorm.h)
 *   MPT_ORDER_CUDA : what the reference CUDA kernels compute: 8-wide K tiles with an inner
 *                    and an outer accumulator for the GEMM (quant_cuda/mm_kernel.h:34-70),
 *                    64-way strided partials folded by a shuffle tree for softmax and
 *                    layernorm (quant_cuda/softmax_kernel.h:5-21, layernorm_kernel.h:29-50) */
enum { MPT_ORDER_SEQ = 0, MPT_ORDER_CUDA = 1 };

MPT_API const char *mpt_last_error(void);
MPT_API int mpt_version(void);

/* No counterpart in the reference (host helper of the multi-GPU decomposition).  The numerically lowest and highest
 * priorities a stream of the current device can take (cudaDeviceGetStreamPriorityRange; smaller = more urgent): the
 * row-sharded GEMM runs its row panels on streams of descending priority so that a panel's tail is filled by the next. */
MPT_API int mpt_stream_priority_range(int *lowest, int *highest);

/* No counterpart in the reference (host helper of the K-panel pipeline of float_mm_streamed).  Copies `rows` rows of
 * `width_bytes` bytes between two pitched buffers, host or device on either side (one cudaMemcpy2DAsync with
 * cudaMemcpyDefault on `stream`): a column panel of a row-major host matrix into a dense device buffer. */
MPT_API int mpt_copy_columns_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                                   size_t rows, void *stream);

/* No counterpart in the reference (the layers there call .contiguous() on transposed views: functional.py:128,154).
 * out[b][c][r] = in[b][r][c] for `batch` dense row-major matrices of `rows` x `cols` floats: the dense copy of a
 * transposed operand (W^T, dY^T, X^T, K^T) the GEMM entry points need, at close to the copy bandwidth.
 * batch and rows / 64 are limited to 65535. */
MPT_API int mpt_transpose_last2(const float *in, float *out, int64_t batch, int64_t rows, int64_t cols, void *stream);

/* ---- elementwise quantizers ------------------------------------------------------------- */

/* replaces float_quantize_nearest (pybind_cuda.cpp:44 -> quant.cu:143 -> fp_kernel.cu:164) */
MPT_API int mpt_float_quantize_nearest(const float *in, float *out, int64_t n, int man, int exp,
                                       int subnormals, int saturate, void *stream);

/* NEW (no reference counterpart): truncation toward zero with the nearest path's clipping */
MPT_API int mpt_float_quantize_truncate(const float *in, float *out, int64_t n, int man, int exp,
                                        int subnormals, int saturate, void *stream);

/* replaces float_quantize_stochastic (pybind_cuda.cpp:98 -> quant.cu:126 -> fp_kernel.cu:150).
 * `rand` holds one int32 random word per element, as the reference draws with
 * randint_like(a, INT_MAX); feeding the same words gives the same bits as the reference. */
MPT_API int mpt_float_quantize_stochastic(const float *in, const int32_t *rand, float *out, int64_t n,
                                          int man, int exp, int prng_bits, int subnormals, int saturate,
                                          void *stream);

/* NEW: same rounding with the random words generated in the kernel (Philox4x32-10, key = seed,
 * counter = element index / 4), which removes the 4 B/element random-word stream. */
MPT_API int mpt_float_quantize_stochastic_philox(const float *in, float *out, int64_t n, int man, int exp,
                                                 int prng_bits, int subnormals, int saturate,
                                                 uint64_t seed, void *stream);

/* NEW, no reference counterpart: the same casts over a list of tensors in one launch per 48 tensors, for the
 * optimizer wrappers that quantize every parameter, gradient and moment tensor of a model each step (the
 * reference's optim_low.py:65-113 calls its quantizer once per tensor).  `in`, `out` and `n` are HOST arrays of
 * `count` device pointers / element counts; out[i] may equal in[i].  `rounding` is an MPT_RND_* value;
 * MPT_RND_NEAREST and MPT_RND_TRUNCATE give the bits of the single-tensor entry points, MPT_RND_STOCHASTIC uses
 * the in-kernel Philox words (key = seed with the tensor's position in the list mixed in, counter = element
 * index / 4).  Nothing is allocated. */
MPT_API int mpt_float_quantize_multi(const float *const *in, float *const *out, const int64_t *n, int count,
                                     int man, int exp, int subnormals, int saturate, int rounding,
                                     int prng_bits, uint64_t seed, void *stream);

/* replaces binary8_quantize_nearest / _stochastic / _truncate (pybind_cuda.cpp:61,107,115 ->
 * quant.cu:173-242 -> binary8_kernel.cu:278-342).  `rounding` is an MPT_RND_* value; `rand`
 * is read only for MPT_RND_STOCHASTIC. */
MPT_API int mpt_binary8_quantize(const float *in, const int32_t *rand, float *out, int64_t n, int P,
                                 int is_signed, int overflow_policy, int subnormals, int rounding,
                                 int prng_bits, void *stream);

/* replaces superfp_quantize_nearest (pybind_cuda.cpp:53 -> quant.cu:158 -> superfp_kernel.cu:70) */
MPT_API int mpt_superfp_quantize_nearest(const float *in, float *out, int64_t n, int man, int exp,
                                         int binades_l, int binades_u, int saturate, void *stream);

/* ---- per-MAC rounded GEMM ------------------------------------------------------------------ */

/* Bytes of scratch the GEMM entry points want in `workspace` (device memory, 16-byte aligned) for a
 * given batch count: 16 bytes of operand statistics per batch entry, rounded up to 256.  The GEMM
 * rewrites it on every call; it need not be initialised and can be reused by the next call on the
 * same stream.  With workspace == NULL (or too small) the GEMM still runs, on the slower exact-cast
 * path only. */
MPT_API size_t mpt_mm_workspace_bytes(int64_t batch);

/* replaces float_quantize_nearest_mm and _bmm (pybind_cuda.cpp:123,140 -> quant.cu:335,362 ->
 * fp_kernel.cu:174-245 -> mm_kernel.h:19-132) and their CPU twins (quant_cpu/mm_kernel.h:9-34).
 *   C[b] = A[b] x B[b],  A: [batch, M, K], B: [batch, K, N], C: [batch, M, N]
 * every product is rounded to (man_mul, exp_mul) and every sum to (man_add, exp_add); both use the
 * `subnormals` and `saturate` flags.  order: MPT_ORDER_SEQ or MPT_ORDER_CUDA.
 * compensated != 0 selects Kahan summation (mm_kernel.h:457-676).
 * A format with man >= 23 and exp >= 8 rounds nothing (fp32 accumulation).  With such a multiply format the
 * reference's CUDA build evaluates `sum + a * b` as one fused multiply-add; MPT_ORDER_CUDA does the same (its
 * results are those of mpt_float_mm_nearest_fma with the add format), MPT_ORDER_SEQ multiplies and adds
 * separately as the reference's CPU build does. */
MPT_API int mpt_float_mm_nearest(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                                 int man_add, int exp_add, int man_mul, int exp_mul,
                                 int subnormals, int saturate, int compensated, int order,
                                 void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference: the product of mpt_float_mm_nearest / _fma (not compensated) computed in
 * pieces along K, for callers whose operands arrive piece by piece (a host buffer copied in K panels while
 * the panels before are being multiplied).  One call handles the steps k0 .. k0 + K - 1 of the full product:
 * A: [batch, M, K] holds those columns of the full A, B: [batch, K, N] those rows of the full B, both dense.
 *   MPT_MM_PIECE_FROM_C: C holds the running sums after the steps before k0 (written by the call for the
 *                        piece before); without it the sums start from zero (the first piece).
 *   MPT_MM_PIECE_MORE:   another piece follows; K must then be a multiple of 8, the group size of the CUDA
 *                        accumulation order, and the zero padding that order walks after the last step is
 *                        left to the last piece.
 * The rounded running sums ARE the result so far, so the pieces in sequence perform exactly the operations
 * of the single call and leave the same bits in C.  fma != 0 selects the fused form (man_mul / exp_mul
 * unused). */
enum { MPT_MM_PIECE_FROM_C = 1, MPT_MM_PIECE_MORE = 2 };
MPT_API int mpt_float_mm_nearest_piece(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                                       int man_add, int exp_add, int man_mul, int exp_mul,
                                       int subnormals, int saturate, int fma, int order, int flags,
                                       void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference.  Same computation and same results as mpt_float_mm_nearest, for
 * callers that cannot allocate device memory and therefore have no workspace to pass (an application
 * whose own pool owns the whole GPU, a plugin interface that hands over only inputs and outputs, a loop
 * where cudaMalloc's implicit synchronisation is not allowed).  The operand statistics are kept in a
 * 64 KiB array built into the library (held by every GPU that loads it, until the process exits), which
 * bounds the batch count: batch > 4096 is rejected with MPT_ERR_INVALID_ARGUMENT.  The call allocates
 * and frees nothing.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture.  The address is cached per device ordinal and
 *     stays valid for the lifetime of the device's primary context: after a cudaDeviceReset (or any
 *     other teardown of that context) the library must be reloaded before this entry point is used again.
 *   - All calls share the array and each one rewrites the part it uses, so calls that may overlap on
 *     the GPU (different streams, or different host threads without ordering) race; serialise them or
 *     use mpt_float_mm_nearest with one workspace per stream. */
MPT_API int mpt_float_mm_nearest_static(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                                        int man_add, int exp_add, int man_mul, int exp_mul,
                                        int subnormals, int saturate, int compensated, int order, void *stream);

/* NEW (the reference's QConv2d materialises the unfolded input, conv.py:591-617, and multiplies it with
 * float_quantize_nearest_mm / _mm_fma): 2-D convolution as an implicit GEMM with the same product order
 * (channel, kernel row, kernel column) and the same accumulation orders, reading the NCHW input in place.
 *   x  [n_img, c_in, H, W]; y [n_img, c_out, OH, OW] with OH = (H + 2 pad_h - dil_h (KH - 1) - 1) / stride_h + 1;
 *   wt [groups][c_in / groups * KH * KW][c_out / groups]: per group the weight matrix TRANSPOSED (K rows, outputs
 *      contiguous), i.e. weight[g].reshape(c_out / groups, K).t().contiguous().
 * Zero padding only (other modes: pad the input first).  Bias is not added.  `workspace` as for mpt_float_mm_nearest
 * with batch = 1.  With fma != 0 every step is one fused multiply-add rounded to (man_add, exp_add). */
MPT_API int mpt_float_conv2d_nearest(const float *x, const float *wt, float *y, int n_img, int c_in, int H, int W,
                                     int c_out, int groups, int KH, int KW, int stride_h, int stride_w, int pad_h,
                                     int pad_w, int dil_h, int dil_w, int man_add, int exp_add, int man_mul,
                                     int exp_mul, int subnormals, int saturate, int fma, int order, void *workspace,
                                     size_t workspace_bytes, void *stream);

/* replaces, in the backward pass of QConv2d, the unfold of the saved input and the GEMM on it for the weight gradient
 * (mptorch/quant/modules/conv.py:537-640 with functional.py:150-155): grad_w[o][(channel, kh, kw)] = sum over (image,
 * oh, ow), in that order, of grad_out[image][o][oh][ow] * x[image][channel][ih][iw], every product and sum rounded as in
 * mpt_float_mm_nearest.  grad_out: [n_img, c_out, OH, OW]; x: [n_img, c_in, H, W]; grad_w: [c_out, c_in / groups * KH *
 * KW].  The unfolded input never exists.  workspace as for mpt_float_mm_nearest with batch = 1. */
MPT_API int mpt_float_conv2d_wgrad_nearest(const float *grad_out, const float *x, float *grad_w, int n_img, int c_in, int H,
                                           int W, int c_out, int groups, int KH, int KW, int stride_h, int stride_w,
                                           int pad_h, int pad_w, int dil_h, int dil_w, int man_add, int exp_add,
                                           int man_mul, int exp_mul, int subnormals, int saturate, int fma, int order,
                                           void *workspace, size_t workspace_bytes, void *stream);

/* replaces float_quantize_nearest_mm_fma and _bmm_fma (pybind_cuda.cpp:157,173 -> quant.cu ->
 * fp_kernel.cu:247-307 -> mm_kernel.h:134-246): acc = Q(fmaf(a, b, acc)). */
MPT_API int mpt_float_mm_nearest_fma(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                                     int man_fma, int exp_fma, int subnormals, int saturate, int compensated,
                                     int order, void *workspace, size_t workspace_bytes, void *stream);

/* replaces float_quantize_stochastic_mm / _bmm / _mm_fma / _bmm_fma (pybind_cuda.cpp:254-300 ->
 * fp_kernel.cu:309-415 -> mm_kernel.h:248-455).  Single accumulator over the zero-padded K range.
 * The reference draws from a per-block cuRAND state seeded by the clock and is not reproducible;
 * here the random words come from Philox4x32-10 keyed by `seed`, so results are a pure function of
 * the inputs and the seed.  Accumulation step k of the output with linear index `lin` in C uses
 * counter (k / 2, lin) and words 2 (k % 2) for the sum and 2 (k % 2) + 1 for the product; the fused
 * form (fma != 0, format (man_add, exp_add, rbits_add)) uses counter (k / 4, lin) and word k % 4.
 * workspace (mpt_mm_workspace_bytes(batch) bytes, 16-byte aligned) enables the range-checked fast
 * path as for mpt_float_mm_nearest; NULL runs the whole-domain casters.  Same bits either way. */
MPT_API int mpt_float_mm_stochastic(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                                    int man_add, int exp_add, int rbits_add,
                                    int man_mul, int exp_mul, int rbits_mul,
                                    int subnormals, int saturate, int fma, uint64_t seed,
                                    void *workspace, size_t workspace_bytes, void *stream);

/* ---- quantized row reductions ------------------------------------------------------------------
 * The tensor is viewed as [outer, channel, inner] (the reference's partition_tensor,
 * quant_cuda/quant.cu:678-726); a row is the `channel` elements at a fixed (outer, inner) position.
 * order: MPT_ORDER_CUDA = the reference CUDA kernels' 64-partials + shuffle-tree association,
 *        MPT_ORDER_SEQ  = the reference CPU loops' left-to-right association. */

/* replaces float_quantize_nearest_softmax_forward (pybind_cuda.cpp:599 -> quant.cu:854 ->
 * fp_kernel.cu:417 -> softmax_kernel.h:23-100; CPU twin quant_cpu/softmax.h:11-46) */
MPT_API int mpt_float_softmax_forward(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                      int man_exp, int exp_exp, int man_off, int exp_off, int man_acc, int exp_acc,
                                      int subnormals, int saturate, int order, void *stream);

/* replaces float_quantize_nearest_softmax_lse_forward (pybind_cuda.cpp:615 -> quant.cu:868 ->
 * softmax_kernel.h:102-171; CPU twin quant_cpu/softmax.h:50-87) */
MPT_API int mpt_float_softmax_lse_forward(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                          int man_off, int exp_off, int man_lse, int exp_lse,
                                          int subnormals, int saturate, int order, void *stream);

/* replaces float_quantize_nearest_softmax_backward (pybind_cuda.cpp:629 -> quant.cu:880 ->
 * softmax_kernel.h:173-222; CPU twin quant_cpu/softmax.h:89-114).  y: softmax output, grad: dL/dy. */
MPT_API int mpt_float_softmax_backward(const float *y, const float *grad, float *out, int64_t outer, int channel,
                                       int64_t inner, int man_add, int exp_add, int man_mul, int exp_mul,
                                       int subnormals, int saturate, int order, void *stream);

/* replaces float_quantize_layernorm_forward (pybind_cuda.cpp:434 -> quant.cu:728 -> fp_kernel.cu:452 ->
 * layernorm_kernel.h:7-100; CPU twin quant_cpu/layernorm.h:10-57).  weight, bias: [channel];
 * mean, rstd: [outer * inner] outputs. */
MPT_API int mpt_float_layernorm_forward(const float *in, const float *weight, const float *bias, float *out,
                                        float *mean, float *rstd, float eps, int64_t outer, int channel, int64_t inner,
                                        int man_acc, int exp_acc, int man_mul, int exp_mul, int man_div, int exp_div,
                                        int man_sqrt, int exp_sqrt, int subnormals, int saturate, int order,
                                        void *stream);

/* replaces float_quantize_layernorm_backward (pybind_cuda.cpp:459 -> quant.cu:748 -> fp_kernel.cu:468-488 ->
 * layernorm_kernel.h:105-237; CPU twin quant_cpu/layernorm.h:60-116).  Needs no scratch tensor: the
 * reference's [rows, channel] x-hat*dy staging buffer (a cudaMalloc per call) is recomputed instead.
 * grad_gamma, grad_beta: [channel], fully overwritten. */
MPT_API int mpt_float_layernorm_backward(const float *in, const float *grad_out, const float *weight,
                                         const float *mean, const float *rstd, float *grad_in, float *grad_gamma,
                                         float *grad_beta, int64_t outer, int channel, int64_t inner,
                                         int man_acc, int exp_acc, int man_mul, int exp_mul, int man_div, int exp_div,
                                         int subnormals, int saturate, int order, void *stream);

/* Sequential rounded column sums of a [rows, cols] matrix: out[c] = Q(...Q(Q(0 + x[0,c]) + x[1,c])...).
 * One launch for what the reference does as a Python loop of one quantize call per row
 * (mptorch/quant/functional.py:736-748, used for the bias gradient at :160-168). */
MPT_API int mpt_qsum_rows(const float *in, float *out, int64_t rows, int64_t cols, int man, int exp,
                          int subnormals, int saturate, void *stream);

/* ---- the same GEMM and reductions for the other nearest-rounding format families --------------------
 * The reference instantiates its mm / softmax / layernorm templates with the supernormal-float caster
 * (superfp_quantize_nearest_mm, _bmm, _mm_fma, _bmm_fma, pybind_cuda.cpp:815-824; superfp softmax and
 * layernorm :887-893, :914-917) and, for the reductions, with the binary8 caster (:897-903, :921-924).
 * One descriptor covers all three families. */
enum { MPT_FMT_FLOAT = 0, MPT_FMT_SUPERFP = 1, MPT_FMT_BINARY8 = 2 };
typedef struct mpt_format {
    int kind;                 /* MPT_FMT_* */
    int man, exp;             /* float, superfp */
    int subnormals;           /* float, binary8 */
    int saturate;             /* float, superfp */
    int binades_l, binades_u; /* superfp */
    int P, is_signed, overflow_policy;   /* binary8 */
} mpt_format;

/* C = A x B with the add and multiply results rounded to `add` and `mul` (fma != 0: one rounding to `add`).
 * Float formats take the same fast kernels as mpt_float_mm_nearest. */
MPT_API int mpt_mm_nearest_fmt(const float *a, const float *b, float *c, int64_t batch, int M, int N, int K,
                               const mpt_format *add, const mpt_format *mul, int fma, int order,
                               void *workspace, size_t workspace_bytes, void *stream);
MPT_API int mpt_softmax_forward_fmt(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                    const mpt_format *fexp, const mpt_format *foff, const mpt_format *facc,
                                    int order, void *stream);
MPT_API int mpt_softmax_lse_forward_fmt(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                        const mpt_format *foff, const mpt_format *flse, int order, void *stream);
MPT_API int mpt_softmax_backward_fmt(const float *y, const float *grad, float *out, int64_t outer, int channel,
                                     int64_t inner, const mpt_format *fadd, const mpt_format *fmul, int order,
                                     void *stream);
MPT_API int mpt_layernorm_forward_fmt(const float *in, const float *weight, const float *bias, float *out,
                                      float *mean, float *rstd, float eps, int64_t outer, int channel, int64_t inner,
                                      const mpt_format *facc, const mpt_format *fmul, const mpt_format *fdiv,
                                      const mpt_format *fsqrt, int order, void *stream);
MPT_API int mpt_layernorm_backward_fmt(const float *in, const float *grad_out, const float *weight,
                                       const float *mean, const float *rstd, float *grad_in, float *grad_gamma,
                                       float *grad_beta, int64_t outer, int channel, int64_t inner,
                                       const mpt_format *facc, const mpt_format *fmul, const mpt_format *fdiv,
                                       int order, void *stream);

/* ---- block-scaled quantizers (NEW: the reference has no MX / NVFP4 kernels) ----------------------
 * Blocks run along the last, contiguous dimension of a [rows, cols] matrix; `out` receives the
 * dequantized fp32 values. */
enum { MPT_ELEM_E4M3 = 0, MPT_ELEM_E2M1 = 1 };   /* OCP element formats: max 448 and 6 */

/* OCP MX: one E8M0 scale 2^(floor(log2 amax) - emax_elem) per `block` elements (32 for MXFP8 / MXFP4),
 * elements rounded to nearest even in `elem_format` with saturation.  `scales` (optional) receives the
 * E8M0 codes, [rows, ceil(cols / block)], 0xFF for a block holding NaN or infinity.  `codes` (optional)
 * receives the packed elements: [rows, cols] bytes for E4M3, [rows, ceil(cols / 2)] bytes for E2M1 with
 * element 2i in the low nibble (needs an even block size); a poisoned block writes 0x7F / 0. */
MPT_API int mpt_mx_quantize(const float *in, float *out, uint8_t *scales, uint8_t *codes, int64_t rows, int64_t cols,
                            int block, int elem_format, void *stream);

/* NVFP4: E2M1 elements in blocks of 16, one E4M3 scale per block (optional output `block_scales`,
 * [rows, ceil(cols / 16)], as fp32 values) and one fp32 scale per tensor.  global_scale > 0 is used as
 * given; otherwise it is computed as amax(tensor) / (448 * 6), which needs 4 bytes of device
 * `workspace` and one extra read of the input; the maximum is taken over the finite entries.
 * `global_scale_out` (optional, device) receives the scale that was used.  `codes` (optional): packed
 * E2M1 elements, [rows, ceil(cols / 2)] bytes, element 2i in the low nibble; `scale_codes` (optional):
 * the block scales as E4M3 bytes.  A NaN element stays NaN in `out` and is coded as 0 (E2M1 has no NaN);
 * an infinite one saturates its block scale at 448 and itself at +-6. */
MPT_API int mpt_nvfp4_quantize(const float *in, float *out, float *block_scales, uint8_t *codes, uint8_t *scale_codes,
                               int64_t rows, int64_t cols, float global_scale, void *workspace,
                               float *global_scale_out, void *stream);

/* ---- quantized optimizer steps and tensor scaling -----------------------------------------------------
 * One launch updates many tensors in place (up to 40 per launch; more are split over launches).  The
 * table is a HOST array; nothing is allocated.  Quantizers are the reference's callables of the form
 * Q(x + y * z) with Q = round to nearest in a (man, exp) format; `*_quant` = 0 means "no quantizer given"
 * (the plain fp32 update of that part).  Scalars arrive already rounded to fp32 the way the reference's
 * torch expressions round them (e.g. one_minus_dampening = (float)(1.0 - dampening)). */
enum { MPT_OPT_FIRST_STEP = 1 };   /* per-tensor flag: the momentum buffer does not exist yet (QSGD) */
typedef struct mpt_optim_tensor {
    float *param;      /* updated in place */
    float *grad;       /* QSGD with weight decay adds weight_decay * param into it, as the reference does */
    float *buf0;       /* QSGD: momentum buffer (momentum != 0)            QAdamW: exp_avg */
    float *buf1;       /* QSGD: compensation buffer (compensated)          QAdamW: exp_avg_sq */
    float *buf2;       /*                                                  QAdamW: compensation buffer (compensated) */
    float *buf3;       /*                                                  QAdamW: max_exp_avg_sq (amsgrad) */
    int64_t n;         /* elements */
    int32_t flags;     /* MPT_OPT_* */
} mpt_optim_tensor;

/* replaces the per-parameter loop of QSGD.step (mptorch/optim/sgd.py:63-150): weight decay into the gradient,
 * momentum buffer update buf = Qm(buf * momentum + d_p * (1 - dampening)) (first step: Qm(d_p)), Nesterov
 * look-ahead, and the weight update p = Qa(p - lr * d_p) or its Kahan-compensated form with the buffer in buf1. */
MPT_API int mpt_qsgd_step(const mpt_optim_tensor *tensors, int count, float lr, float momentum,
                          float one_minus_dampening, float weight_decay, int nesterov, int compensated,
                          int momentum_quant, int man_mom, int exp_mom, int acc_quant, int man_acc, int exp_acc,
                          int subnormals, int saturate, void *stream);

/* replaces the per-parameter loop of QAdamW.step (mptorch/optim/adamw.py:44-150) for tensors that share one
 * step count: moments m = Qm(m * beta1 + g * (1 - beta1)), v = Qm(v * beta2 + g^2 * (1 - beta2)), optional
 * amsgrad maximum, denom = sqrt(v) * inv_sqrt_bias_correction2 + eps, and the weight update
 * p = Qa(p - step_size * m / denom) or its Kahan-compensated form.  step_size = lr / bias_correction1 and
 * inv_sqrt_bias_correction2 = (float)(1.0 / sqrt(bias_correction2)) are computed by the caller. */
MPT_API int mpt_qadamw_step(const mpt_optim_tensor *tensors, int count, float beta1, float beta2,
                            float one_minus_beta1, float one_minus_beta2, float inv_sqrt_bias_correction2,
                            float eps, float step_size, int amsgrad, int compensated,
                            int momentum_quant, int man_mom, int exp_mom, int acc_quant, int man_acc, int exp_acc,
                            int subnormals, int saturate, void *stream);

/* replaces compute_bias + scale + the quantizer call of the layers' tensor scaling
 * (mptorch/quant/functional.py:39-53 as used at :82-90): for each of `matrices` consecutive blocks of
 * `per_matrix` elements, s = floor(log2(normal_max / amax)) - margin (log2 in double precision) and
 * out = Q(in * 2^s); `quantize` = 0 leaves the scaled values unrounded.  `scale_out` (optional, device,
 * `matrices` floats) receives s.  workspace: mpt_scale_quantize_workspace_bytes(matrices) bytes. */
MPT_API size_t mpt_scale_quantize_workspace_bytes(int64_t matrices);
MPT_API int mpt_scale_quantize(const float *in, float *out, int64_t matrices, int64_t per_matrix, double normal_max,
                               int margin, int quantize, int man, int exp, int subnormals, int saturate,
                               float *scale_out, void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MPTORCH_B200_H */
