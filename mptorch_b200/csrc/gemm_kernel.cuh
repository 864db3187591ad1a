// Per-MAC rounded GEMM for sm_100a: C = A x B where every product and every partial sum is
// rounded to a user format before it is used again.
//
// This is CUDA-core work by construction: each output's K accumulation is a serial chain of
// (multiply, round, add, round), so tensor cores cannot be used.  The kernel is bound by the
// instruction issue rate; the design goal is the smallest number of issued instructions per
// MAC that still reproduces the reference bit for bit:
//
//   * fast path, 10 instructions per MAC (FMUL, 4 for the product rounding, FADD, 4 for the sum
//     rounding), see FastRn in cast.cuh.  It is exact whenever no intermediate value can leave
//     the finite range of its format.  That is established from the magnitude statistics of A
//     and B (a tiny pre-pass writes one record per batch entry to the workspace) plus a
//     per-thread check of the running accumulators at every fold;
//   * exact path: the complete reference caster (every corner case), taken per thread and per
//     8-step group whenever the fast path's precondition cannot be shown.
//
// Tiling: 128x64 outputs per CTA, 256 threads, 8x4 outputs per thread, K in slabs of 32 staged
// through a 3-deep cp.async pipeline in shared memory.  Memory traffic is negligible next to
// the arithmetic (about 140 GB/s at 8192^3), so tiles are plain cp.async copies.
//
// Accumulation orders (both kept bit-exact):
//   MPT_ORDER_SEQ   acc = Qadd(acc + Qmul(a*b)), k = 0..K-1   (reference quant_cpu/mm_kernel.h:9-20)
//   MPT_ORDER_CUDA  K walked in groups of 8, zero padded, one extra all-zero group when 8 | K;
//                   inner accumulates a group, then outer = Qadd(outer + inner)
//                   (reference quant_cuda/mm_kernel.h:34-70; fma variant :134-186)
// Kahan-compensated and stochastic variants follow quant_cuda/mm_kernel.h:457-520 and :248-295.
//
// Files: gemm_kernel.cuh (this file: the kernel and its launch templates), gemm.cu (C entry points, operand
// statistics, problem set-up) and one file per group of instantiations (gemm_seq.cu, gemm_tile8.cu, gemm_kahan.cu,
// gemm_sr.cu, gemm_conv.cu) so that they compile side by side.
#pragma once
#include <cuda_pipeline.h>

#include <cstdlib>
#include <mutex>

#include "cast.cuh"
#include "common.cuh"

namespace mpt {


#ifndef MPT_MM_TM
#define MPT_MM_TM 8          // output rows per thread
#endif
#ifndef MPT_MM_MIN_CTAS
#define MPT_MM_MIN_CTAS 2    // resident CTAs per SM the register allocation is held to
#endif
#ifndef MPT_MM_SR_MIN_CTAS
#define MPT_MM_SR_MIN_CTAS 1 // the same for the stochastic kernel
#endif
constexpr int TM = MPT_MM_TM, TN = 4;
constexpr int BM = 16 * TM, BN = 64, BK = 32;
constexpr int THREADS = 256;
constexpr int STAGES = 3;
constexpr int AS_LD = BK + 4;   // row stride of the A tile: keeps 16-byte chunks aligned, spreads banks
constexpr int SMEM_A = BM * AS_LD, SMEM_B = BK * BN;
constexpr size_t SMEM_BYTES = (size_t)STAGES * (SMEM_A + SMEM_B) * sizeof(float);

enum Algo : int { ALGO_SEQ = 0, ALGO_TILE8 = 1, ALGO_KAHAN = 2, ALGO_SR = 3 };

// Magnitude statistics of the operands, produced by stats_kernel into the workspace.
struct MmStats {
    uint32_t max_a, max_b;       // largest |x| bit pattern (NaN and inf compare above every finite)
    uint32_t minnz_a, minnz_b;   // smallest nonzero |x| bit pattern, 0xFFFFFFFF if all zero
};

// Convolution as an implicit GEMM: row m of A is output position (image, oh, ow), column k is (channel, kh, kw) in
// that order (the order of F.unfold and of the reference's unfoldNd, conv.py:591-617), and the element is read
// straight from the NCHW input (zero outside the image), so the unfolded matrix never exists.  C is written to the
// NCHW output.
// The weight gradient of the same convolution is a GEMM too (CONV mode 2): dW[o][(channel, kh, kw)] = sum over k =
// (image, oh, ow) of dY[image][o][oh][ow] * x[image][channel][ih][iw], i.e. A = dY seen as [c_out, images * OH * OW]
// (row o, column k: a strided read of the NCHW gradient) and B = the unfolded input, gathered on the fly; K runs over
// the images and output positions in the order of the reference's unfold + transpose (conv.py:591-617).
struct ConvGeom {
    int H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    int64_t x_image_stride, y_image_stride;      // elements between consecutive images of input and output
};
enum ConvMode : int { CONV_NONE = 0, CONV_FWD = 1, CONV_WGRAD = 2 };

struct MmParams {
    ConvGeom cv;                 // used by the CONV instantiations only
    const float* a;
    const float* b;
    float* c;
    int M, N, K;
    int64_t stride_a, stride_b, stride_c;
    FpFmt fadd, fmul;            // float view of the formats (fast path, plan)
    AnyFmt gadd, gmul;           // the formats as the exact path rounds them (float, superfp or binary8)
    FastRn radd, rmul;
    int rbits_add, rbits_mul;
    uint32_t seed_lo, seed_hi;
    const MmStats* stats;        // one record per batch entry; NULL: exact path only
    float growth8;               // upper bound of (1 + 2^-(man_add+1))^8
    // whole-domain fast casters for the variants without a range-checked fast path (Kahan, stochastic): same bits as
    // the exact casters on every input at a fraction of the instructions, for the formats that support them
    FullRn wadd, wmul;
    int whole_ok;
    FullSr sadd, smul;
    int sr_ok;
    int sr_nosub = 0;            // formats without subnormals: the in-range stochastic rounding below covers them too
    // Kahan fast path: with |sum|, |comp| <= L and |a*b| <= P at the start of an 8-step group, every intermediate of
    // the group stays below kah_sc * L + kah_p * P + kah_const (coefficients worked out on the host from the add
    // format's rounding error, see kahan_bounds in gemm.cu)
    float kah_sc, kah_p, kah_const;
    float growth8_sr;            // upper bound of (1 + 2^-man_add)^8: eight stochastic roundings of a sum
    // A product computed in pieces along K (ALGO_SEQ / ALGO_TILE8 only; every piece but the last a multiple of 8 steps):
    // MM_FROM_C starts the running sums from what C holds (the sums after the pieces before) instead of zero,
    // MM_MORE says another piece follows, so the zero padding the CUDA order walks after the last step is left to it.
    int resume = 0;
    // Set when a launch of exact_mm_kernel for the same product follows on the stream: a batch entry whose operand
    // statistics rule the range-checked path out altogether (a NaN or infinity among the operands, products or
    // sums beyond the formats' ranges, denormal intermediates of 8-bit-exponent formats) is left to that kernel,
    // which is shaped for the exact casters; mm_kernel returns at once for it, exact_mm_kernel for every other entry.
    int defer_exact = 0;
    int nosub = 0;               // the formats have no subnormals and the launch is of the NOSUB instantiation
};
enum { MM_FROM_C = 1, MM_MORE = 2 };

// The format that rounds nothing (man >= 23 and exp >= 8: the reference's `noquantize`, fp_kernel.cu:23): fp32
// accumulation of low-precision products is the usual use.  The range-checked fast path covers it with the magic
// constant set to zero: FFMA(m, 0, x) = x + 0 leaves every finite x as it is, except that -0 becomes +0, which no sum
// can tell apart here (the running sums start at +0 and an IEEE sum is -0 only when both terms are).
__host__ __device__ inline bool fmt_identity(const FpFmt& f) { return f.man >= 23 && f.exp >= 8; }
__host__ __device__ inline bool mm_fast_format(const FpFmt& f) { return fast_rn_supported(f) || fmt_identity(f); }
__host__ __device__ inline FastRn mm_fast_rn(const FpFmt& f) {
    FastRn r = FastRn::make(f);
    if (fmt_identity(f)) r.k = 0.0f;
    return r;
}

// Nearest rounding to the add / multiply format on the whole input domain.  The exact caster is an out-of-line call
// (taken for formats without the fast rounding, and for the tiny or huge inputs 8-bit-exponent formats treat
// specially), so that the many rounding sites of the Kahan kernels stay small.
static __device__ __noinline__ float exact_add_cold(const MmParams* p, float x) { return cast_any(x, p->gadd); }
static __device__ __noinline__ float exact_mul_cold(const MmParams* p, float x) { return cast_any(x, p->gmul); }
__device__ __forceinline__ bool whole_fast(const FullRn& w, float x, float& out) {
    const uint32_t t = __float_as_uint(x), a = t & 0x7FFFFFFFu;
    if (w.fmt.exp == 8 && (a >= w.exact_from || a < 0x00800000u)) return false;
    const float y = w.fast(x);
    const float over = (a >= 0x7F800000u) ? x : __uint_as_float((t & 0x80000000u) | w.ovf_value);
    out = (a >= w.ovf_from) ? over : y;
    return true;
}
__device__ __forceinline__ float round_add(const MmParams& p, float x) {
    float r;
    if (p.whole_ok && whole_fast(p.wadd, x, r)) return r;
    return exact_add_cold(&p, x);
}
__device__ __forceinline__ float round_mul(const MmParams& p, float x) {
    float r;
    if (p.whole_ok && whole_fast(p.wmul, x, r)) return r;
    return exact_mul_cold(&p, x);
}
__device__ __forceinline__ float sr_add(const MmParams& p, float x, uint32_t r) {
    return p.sr_ok ? p.sadd(x, r) : cast_fp_stochastic(x, r, p.rbits_add, p.fadd);
}
__device__ __forceinline__ float sr_mul(const MmParams& p, float x, uint32_t r) {
    return p.sr_ok ? p.smul(x, r) : cast_fp_stochastic(x, r, p.rbits_mul, p.fmul);
}

static __global__ void stats_init_kernel(MmStats* s, int64_t batch) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) { s[i].max_a = 0u; s[i].max_b = 0u; s[i].minnz_a = 0xFFFFFFFFu; s[i].minnz_b = 0xFFFFFFFFu; }
}

// blockIdx.y walks the batch; `which` selects the A (0) or B (1) fields of that entry's record.
static __global__ void __launch_bounds__(256) stats_kernel(const float* __restrict__ base, int64_t n, MmStats* stats, int which) {
    const float* x = base + (int64_t)blockIdx.y * n;
    uint32_t* mx = which ? &stats[blockIdx.y].max_b : &stats[blockIdx.y].max_a;
    uint32_t* mn = which ? &stats[blockIdx.y].minnz_b : &stats[blockIdx.y].minnz_a;
    uint32_t lmax = 0u, lmin = 0xFFFFFFFFu;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    auto take = [&](float v) {
        const uint32_t a = __float_as_uint(v) & 0x7FFFFFFFu;
        lmax = max(lmax, a);
        lmin = min(lmin, a - 1u);                      // zero wraps to the largest value and so never wins
    };
    // 16-byte loads, four in flight per thread, where this entry starts on a 16-byte boundary
    const int64_t n4 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 ? n / 4 : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 4
    for (int64_t i = tid; i < n4; i += stride) {
        const float4 v = x4[i];
        take(v.x); take(v.y); take(v.z); take(v.w);
    }
    for (int64_t i = 4 * n4 + tid; i < n; i += stride) take(x[i]);
    lmin = lmin == 0xFFFFFFFFu ? lmin : lmin + 1u;     // back from (pattern - 1); all zero stays 0xFFFFFFFF
    lmax = __reduce_max_sync(0xFFFFFFFFu, lmax);
    lmin = __reduce_min_sync(0xFFFFFFFFu, lmin);
    if ((threadIdx.x & 31) == 0) {
        atomicMax(mx, lmax);
        atomicMin(mn, lmin);
    }
}

__device__ __forceinline__ void cp_async16(float* dst, const float* src, int src_bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src, int src_bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Stage one K slab: As[m][k] (row stride AS_LD) and Bs[k][n].  Elements outside the matrices are
// zero filled (cp.async with a source size of 0), which is also how K is zero padded.
struct ConvRow { int64_t base; int ih0, iw0; };     // per output position: image offset, top-left input coordinate

template <bool VEC, int CONV = CONV_NONE>
__device__ __forceinline__ void load_tiles(const MmParams& p, const float* A, const float* B, float* As, float* Bs,
                                           int m0, int n0, int k0, int tid, const ConvRow* rows = nullptr) {
    if (CONV == CONV_WGRAD) {
        const int L = p.cv.OH * p.cv.OW;
        {   // A[m][k] = dY[image(k)][m][position(k)]: the thread's slab column is fixed, its rows are (tid >> 5) + 8 u
            const int kk = tid & 31, gk = k0 + kk;
            const bool kok = gk < p.K;
            const int img = gk / L, l = gk - img * L;
            const int64_t koff = (int64_t)img * p.cv.y_image_stride + l;
#pragma unroll 4
            for (int u = 0; u < BM / 8; ++u) {
                const int row = (tid >> 5) + 8 * u, gm = m0 + row;
                const bool ok = kok && gm < p.M;
                cp_async4(As + row * AS_LD + kk, ok ? A + koff + (int64_t)gm * L : A, ok ? 4 : 0);
            }
        }
        {   // B[k][j] = x[image(k)][channel(j)][ih][iw]: the thread's column j is fixed, its slab rows are (tid >> 6) + 4 u
            const int nn = tid & 63, gj = n0 + nn;
            const int khkw = p.cv.KH * p.cv.KW;
            const int ch = gj / khkw, rem = gj - ch * khkw;
            const int kh = rem / p.cv.KW, kw = rem - kh * p.cv.KW;
            const bool jok = gj < p.N;
            const int dih = kh * p.cv.dh - p.cv.ph, diw = kw * p.cv.dw - p.cv.pw;
            const int64_t coff = (int64_t)ch * p.cv.H * p.cv.W;
#pragma unroll 4
            for (int u = 0; u < (BK * BN) / THREADS; ++u) {
                const int kr = (tid >> 6) + 4 * u, gk = k0 + kr;
                const int img = gk / L, l = gk - img * L;
                const int oh = l / p.cv.OW, ow = l - oh * p.cv.OW;
                const int ih = oh * p.cv.sh + dih, iw = ow * p.cv.sw + diw;
                const bool ok = jok && gk < p.K && (unsigned)ih < (unsigned)p.cv.H && (unsigned)iw < (unsigned)p.cv.W;
                cp_async4(Bs + kr * BN + nn, ok ? B + (int64_t)img * p.cv.x_image_stride + coff + (int64_t)ih * p.cv.W + iw : B, ok ? 4 : 0);
            }
        }
        return;
    }
    if (CONV == CONV_FWD) {
        // A: the thread's column of the slab is fixed (tid & 31), its rows are (tid >> 5) + 8 u
        const int kk = tid & 31, gk = k0 + kk;
        const int khkw = p.cv.KH * p.cv.KW;
        const int ch = gk / khkw, rem = gk - ch * khkw;
        const int kh = rem / p.cv.KW, kw = rem - kh * p.cv.KW;
        const bool kok = gk < p.K;
        const int dih = kh * p.cv.dh, diw = kw * p.cv.dw;
        const int64_t coff = (int64_t)ch * p.cv.H * p.cv.W;
#pragma unroll 4
        for (int u = 0; u < BM / 8; ++u) {
            const int row = (tid >> 5) + 8 * u;
            const ConvRow r = rows[row];
            const int ih = r.ih0 + dih, iw = r.iw0 + diw;
            const bool ok = kok && (unsigned)ih < (unsigned)p.cv.H && (unsigned)iw < (unsigned)p.cv.W;
            cp_async4(As + row * AS_LD + kk, ok ? A + r.base + coff + (int64_t)ih * p.cv.W + iw : A, ok ? 4 : 0);
        }
#pragma unroll 4
        for (int u = 0; u < (BK * BN) / THREADS; ++u) {
            const int c = tid + u * THREADS;
            const int kr = c >> 6, nn = c & 63;
            const int gk2 = k0 + kr, gn = n0 + nn;
            const bool ok = gk2 < p.K && gn < p.N;
            cp_async4(Bs + kr * BN + nn, ok ? B + (int64_t)gk2 * p.N + gn : B, ok ? 4 : 0);
        }
        return;
    }
    if (VEC) {
#pragma unroll
        constexpr int kAChunks = BM * BK / 4;               // 16-byte pieces of the A tile; fewer than threads for 16-row tiles
        for (int u = 0; u < (kAChunks + THREADS - 1) / THREADS; ++u) {
            const int c = tid + u * THREADS;
            if (kAChunks % THREADS != 0 && c >= kAChunks) break;
            const int row = c >> 3, kc = (c & 7) << 2;
            const int gm = m0 + row, gk = k0 + kc;
            int bytes = (gm < p.M) ? (p.K - gk) * 4 : 0;
            bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
            const float* src = bytes ? A + (int64_t)gm * p.K + gk : A;
            cp_async16(As + row * AS_LD + kc, src, bytes);
        }
#pragma unroll
        for (int u = 0; u < (BK * BN / 4) / THREADS; ++u) {
            const int c = tid + u * THREADS;
            const int kr = c >> 4, nc = (c & 15) << 2;
            const int gk = k0 + kr, gn = n0 + nc;
            int bytes = (gk < p.K) ? (p.N - gn) * 4 : 0;
            bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
            const float* src = bytes ? B + (int64_t)gk * p.N + gn : B;
            cp_async16(Bs + kr * BN + nc, src, bytes);
        }
    } else {
#pragma unroll 4
        for (int u = 0; u < (BM * BK) / THREADS; ++u) {
            const int c = tid + u * THREADS;
            const int row = c >> 5, kk = c & 31;
            const int gm = m0 + row, gk = k0 + kk;
            const bool ok = gm < p.M && gk < p.K;
            cp_async4(As + row * AS_LD + kk, ok ? A + (int64_t)gm * p.K + gk : A, ok ? 4 : 0);
        }
#pragma unroll 4
        for (int u = 0; u < (BK * BN) / THREADS; ++u) {
            const int c = tid + u * THREADS;
            const int kr = c >> 6, nn = c & 63;
            const int gk = k0 + kr, gn = n0 + nn;
            const bool ok = gk < p.K && gn < p.N;
            cp_async4(Bs + kr * BN + nn, ok ? B + (int64_t)gk * p.N + gn : B, ok ? 4 : 0);
        }
    }
}

// One accumulation step on the exact path.
template <bool FMA>
__device__ __forceinline__ float mac_exact(float acc, float a, float b, const AnyFmt& fadd, const AnyFmt& fmul) {
    if (FMA) return cast_any(fma_rn(a, b, acc), fadd);
    return cast_any(add_rn(acc, cast_any(mul_rn(a, b), fmul)), fadd);
}
// Formats without subnormals, inner sums of the CUDA order: the sum rounding only flags a result that needs the
// settling rule; the caller redoes the group of eight steps (which started from zero) on the exact casters.
template <bool FMA>
__device__ __forceinline__ float mac_fast_flag(float acc, float a, float b, const FastRn& radd, const FastRn& rmul, uint32_t& rare) {
    if (FMA) return fast_rn_nosub_flag(radd, fma_rn(a, b, acc), rare);
    return fast_rn_nosub_flag(radd, add_rn(acc, fast_rn_nosub(rmul, mul_rn(a, b))), rare);
}
template <bool FMA, bool NOSUB = false>
__device__ __forceinline__ float mac_fast(float acc, float a, float b, const FastRn& radd, const FastRn& rmul) {
    if (NOSUB) {
        // products land below the smallest normal value all the time (branch-free settling); sums of rounded products
        // almost never do (settling behind a branch)
        if (FMA) return fast_rn_nosub(radd, fma_rn(a, b, acc));
        return fast_rn_nosub_rare(radd, add_rn(acc, fast_rn_nosub(rmul, mul_rn(a, b))));
    }
    if (FMA) return radd(fma_rn(a, b, acc));
    return radd(add_rn(acc, rmul(mul_rn(a, b))));
}

// Two accumulation steps at once on sm_100's packed fp32x2 instructions (FMUL2 / FADD2 / FFMA2): the six
// FP-pipe instructions of a MAC are shared by two neighbouring outputs, so a MAC costs 3 packed FP
// instructions + 4 ALU instructions (the exponent extraction stays per element) = 7 issue slots
// instead of 10.  Each half of a packed instruction rounds exactly like its scalar form.
//
// GUARD = false drops the clamp of the exponent at the format's smallest normal binade (one IMNMX per
// element).  That is exact for the SUM rounding whenever the multiply format's smallest subnormal is
// not finer than the add format's: every product and every partial sum is then a multiple of the add
// format's smallest subnormal, so a sum that lands in the add format's subnormal range has no bits
// below that quantum and rounding it at its own exponent leaves it unchanged, exactly like the
// clamped rounding (a zero sum gives m = 0 and comes out as +0).
template <bool GUARD>
__device__ __forceinline__ float2 fast_rn2(const FastRn& r, float2 x) {
    int e0 = __float_as_int(x.x) & 0x7F800000, e1 = __float_as_int(x.y) & 0x7F800000;
    if (GUARD) { e0 = max(e0, r.min_e_bits); e1 = max(e1, r.min_e_bits); }
    const float2 m = make_float2(__int_as_float(e0), __int_as_float(e1));
    const float2 y = __ffma2_rn(m, make_float2(r.k, r.k), x);
    return __ffma2_rn(m, make_float2(-r.k, -r.k), y);
}
template <bool FMA, bool ADDG>
__device__ __forceinline__ float2 mac_fast2(float2 acc, float2 a2, float2 b2, const FastRn& radd, const FastRn& rmul) {
    if (FMA) return fast_rn2<true>(radd, __ffma2_rn(a2, b2, acc));
    return fast_rn2<ADDG>(radd, __fadd2_rn(acc, fast_rn2<true>(rmul, __fmul2_rn(a2, b2))));
}

// One accumulation step of the exact path for four outputs that share the A element, as a function call: the exact
// casters are long (three format kinds, subnormal and overflow branches), and a copy inlined at each of the 64
// roundings of a thread's step would not fit the instruction cache.  The kind is tested once per call.
template <bool FMA>
static __device__ __noinline__ float4 mac_exact4(float4 acc, float a, float4 b, const MmParams* pp) {
    const AnyFmt& fa = pp->gadd;
    const AnyFmt& fm = pp->gmul;
    if (pp->whole_ok) {
        // formats the FP-pipe rounding covers: its whole-domain form (same bits as the exact caster on every input)
        const MmParams& p = *pp;
        if (FMA) {
            acc.x = round_add(p, fma_rn(a, b.x, acc.x)); acc.y = round_add(p, fma_rn(a, b.y, acc.y));
            acc.z = round_add(p, fma_rn(a, b.z, acc.z)); acc.w = round_add(p, fma_rn(a, b.w, acc.w));
        } else {
            acc.x = round_add(p, add_rn(acc.x, round_mul(p, mul_rn(a, b.x)))); acc.y = round_add(p, add_rn(acc.y, round_mul(p, mul_rn(a, b.y))));
            acc.z = round_add(p, add_rn(acc.z, round_mul(p, mul_rn(a, b.z)))); acc.w = round_add(p, add_rn(acc.w, round_mul(p, mul_rn(a, b.w))));
        }
        return acc;
    }
    if (fa.kind == FMT_FLOAT && (FMA || fm.kind == FMT_FLOAT)) {
        const FpFmt ga = fa.fp, gm = fm.fp;
        if (FMA) {
            acc.x = cast_fp_nearest(fma_rn(a, b.x, acc.x), ga); acc.y = cast_fp_nearest(fma_rn(a, b.y, acc.y), ga);
            acc.z = cast_fp_nearest(fma_rn(a, b.z, acc.z), ga); acc.w = cast_fp_nearest(fma_rn(a, b.w, acc.w), ga);
        } else {
            acc.x = cast_fp_nearest(add_rn(acc.x, cast_fp_nearest(mul_rn(a, b.x), gm)), ga);
            acc.y = cast_fp_nearest(add_rn(acc.y, cast_fp_nearest(mul_rn(a, b.y), gm)), ga);
            acc.z = cast_fp_nearest(add_rn(acc.z, cast_fp_nearest(mul_rn(a, b.z), gm)), ga);
            acc.w = cast_fp_nearest(add_rn(acc.w, cast_fp_nearest(mul_rn(a, b.w), gm)), ga);
        }
        return acc;
    }
    acc.x = mac_exact<FMA>(acc.x, a, b.x, fa, fm); acc.y = mac_exact<FMA>(acc.y, a, b.y, fa, fm);
    acc.z = mac_exact<FMA>(acc.z, a, b.z, fa, fm); acc.w = mac_exact<FMA>(acc.w, a, b.w, fa, fm);
    return acc;
}

// `nk` (1..8) accumulation steps starting at slab row kbase, for the thread's 8x4 outputs.
// REDO (formats without subnormals, sums that start from zero): returns true when a sum rounding met a value that needs
// the settling rule; the caller then zeroes the accumulators and runs the group on the exact path.
template <bool FMA, bool FAST, bool PACKED, bool ADDG, bool NOSUB = false, bool REDO = false>
__device__ __forceinline__ bool group_steps(float (&acc)[TM][TN], const float* As, const float* Bs, int kbase, int nk,
                                            int ty, int tx, const MmParams& p) {
    uint32_t rare = 0u;
    if (FAST && nk == 8) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float4 av[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i)
                av[i] = *reinterpret_cast<const float4*>(As + (ty + 16 * i) * AS_LD + kbase + 4 * h);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 bv = *reinterpret_cast<const float4*>(Bs + (kbase + 4 * h + j) * BN + tx * 4);
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float a = j == 0 ? av[i].x : j == 1 ? av[i].y : j == 2 ? av[i].z : av[i].w;
                    if (PACKED) {
                        const float2 a2 = make_float2(a, a);
                        const float2 lo = mac_fast2<FMA, ADDG>(make_float2(acc[i][0], acc[i][1]), a2, make_float2(bv.x, bv.y), p.radd, p.rmul);
                        const float2 hi = mac_fast2<FMA, ADDG>(make_float2(acc[i][2], acc[i][3]), a2, make_float2(bv.z, bv.w), p.radd, p.rmul);
                        acc[i][0] = lo.x; acc[i][1] = lo.y; acc[i][2] = hi.x; acc[i][3] = hi.y;
                    } else if (NOSUB && REDO) {
                        acc[i][0] = mac_fast_flag<FMA>(acc[i][0], a, bv.x, p.radd, p.rmul, rare);
                        acc[i][1] = mac_fast_flag<FMA>(acc[i][1], a, bv.y, p.radd, p.rmul, rare);
                        acc[i][2] = mac_fast_flag<FMA>(acc[i][2], a, bv.z, p.radd, p.rmul, rare);
                        acc[i][3] = mac_fast_flag<FMA>(acc[i][3], a, bv.w, p.radd, p.rmul, rare);
                    } else {
                        acc[i][0] = mac_fast<FMA, NOSUB>(acc[i][0], a, bv.x, p.radd, p.rmul);
                        acc[i][1] = mac_fast<FMA, NOSUB>(acc[i][1], a, bv.y, p.radd, p.rmul);
                        acc[i][2] = mac_fast<FMA, NOSUB>(acc[i][2], a, bv.z, p.radd, p.rmul);
                        acc[i][3] = mac_fast<FMA, NOSUB>(acc[i][3], a, bv.w, p.radd, p.rmul);
                    }
                }
            }
        }
        return rare != 0u;
    }
#pragma unroll 1
    for (int k = 0; k < nk; ++k) {
        const float4 bv = *reinterpret_cast<const float4*>(Bs + (kbase + k) * BN + tx * 4);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const float a = As[(ty + 16 * i) * AS_LD + kbase + k];
            if (FAST) {
                acc[i][0] = mac_fast<FMA, NOSUB>(acc[i][0], a, bv.x, p.radd, p.rmul);
                acc[i][1] = mac_fast<FMA, NOSUB>(acc[i][1], a, bv.y, p.radd, p.rmul);
                acc[i][2] = mac_fast<FMA, NOSUB>(acc[i][2], a, bv.z, p.radd, p.rmul);
                acc[i][3] = mac_fast<FMA, NOSUB>(acc[i][3], a, bv.w, p.radd, p.rmul);
            } else {
                const float4 r = mac_exact4<FMA>(make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]), a, bv, &p);
                acc[i][0] = r.x; acc[i][1] = r.y; acc[i][2] = r.z; acc[i][3] = r.w;
            }
        }
    }
    return false;
}

// ---- Kahan-compensated accumulation (reference quant_cuda/mm_kernel.h:487-497, fma variant :600-608) --------------
//     update = Qmul(a*b);  y = Qadd(update - comp);  t = Qadd(sum + y);  comp = Qadd(Qadd(t - sum) - y);  sum = t
// One step on the exact casters.
template <bool FMA>
__device__ __forceinline__ void kahan_exact(float& sum, float& comp, float a, float b, const MmParams& p) {
    const float y = FMA ? round_add(p, fma_rn(a, b, -comp)) : round_add(p, add_rn(round_mul(p, mul_rn(a, b)), -comp));
    const float t = round_add(p, add_rn(sum, y));
    comp = round_add(p, add_rn(round_add(p, add_rn(t, -sum)), -y));
    sum = t;
}
// Two neighbouring outputs at once on the packed fp32x2 instructions, five 4-instruction roundings per step.  The state
// carried through a group is the NEGATED compensation term nc = -comp, so that every subtraction is an FADD2 or an FFMA2
// with the constant -1 (t - sum = fma(sum, -1, t), one rounding, like the subtraction itself) and no separate negations
// are issued; rounding to nearest is symmetric, so Q(y - c1) = -Q(c1 - y).
template <bool FMA, bool ADDG>
__device__ __forceinline__ void kahan_fast2(float2& sum, float2& nc, float2 a2, float2 b2, const FastRn& radd, const FastRn& rmul) {
    const float2 m1 = make_float2(-1.0f, -1.0f);
    const float2 y = FMA ? fast_rn2<true>(radd, __ffma2_rn(a2, b2, nc))
                         : fast_rn2<ADDG>(radd, __fadd2_rn(fast_rn2<true>(rmul, __fmul2_rn(a2, b2)), nc));
    const float2 t = fast_rn2<ADDG || FMA>(radd, __fadd2_rn(sum, y));
    const float2 c1 = fast_rn2<ADDG || FMA>(radd, __ffma2_rn(sum, m1, t));
    nc = fast_rn2<ADDG || FMA>(radd, __ffma2_rn(c1, m1, y));
    sum = t;
}
// Eight accumulation steps starting at slab row kbase; acc = running sums, aux = compensation terms.
template <bool FMA, bool ADDG>
__device__ __forceinline__ void kahan_group_fast(float (&acc)[TM][TN], float (&aux)[TM][TN], const float* As, const float* Bs,
                                                 int kbase, int ty, int tx, const MmParams& p) {
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) aux[i][j] = add_rn(0.0f, -aux[i][j]);      // nc = -comp (+0 for a zero term)
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
        float4 av[TM];
#pragma unroll
        for (int i = 0; i < TM; ++i) av[i] = *reinterpret_cast<const float4*>(As + (ty + 16 * i) * AS_LD + kbase + 4 * h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 bv = *reinterpret_cast<const float4*>(Bs + (kbase + 4 * h + j) * BN + tx * 4);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const float a = j == 0 ? av[i].x : j == 1 ? av[i].y : j == 2 ? av[i].z : av[i].w;
                const float2 a2 = make_float2(a, a);
                float2 s0 = make_float2(acc[i][0], acc[i][1]), c0 = make_float2(aux[i][0], aux[i][1]);
                float2 s1 = make_float2(acc[i][2], acc[i][3]), c1 = make_float2(aux[i][2], aux[i][3]);
                kahan_fast2<FMA, ADDG>(s0, c0, a2, make_float2(bv.x, bv.y), p.radd, p.rmul);
                kahan_fast2<FMA, ADDG>(s1, c1, a2, make_float2(bv.z, bv.w), p.radd, p.rmul);
                acc[i][0] = s0.x; acc[i][1] = s0.y; acc[i][2] = s1.x; acc[i][3] = s1.y;
                aux[i][0] = c0.x; aux[i][1] = c0.y; aux[i][2] = c1.x; aux[i][3] = c1.y;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) aux[i][j] = add_rn(0.0f, -aux[i][j]);
}

// ---- stochastic rounding -------------------------------------------------------------------------------------------
// Random words of accumulation step k of output `lin` (its linear index in C): Philox4x32-10 with the seed as key and
// the counter (k / 2, lin) for the two-rounding MAC (words 0,1 serve the even step's sum and product, words 2,3 the odd
// step's), (k / 4, lin) for the fused MAC (word k % 4), so that every generated word is used.
// Stochastic rounding of a finite value that cannot reach the format's overflow threshold (the caller has shown so):
// FullSr without its NaN branch and overflow select.
template <bool NOSUB>
__device__ __forceinline__ float sr_inrange(const FullSr& f, float x, uint32_t rnd) {
    if (NOSUB) {
        // Without subnormals the reference rounds every value at its own exponent and then settles what landed below
        // 2^min_exp (bit_helper.cu:110-123): the smallest normal value with the input's sign if the rounded magnitude
        // exceeds 2^(min_exp - 1), +0 otherwise.  Integer arithmetic throughout, so every finite input is covered.
        const uint32_t t = __float_as_uint(x);
        const uint32_t q = (t + (rnd & f.rmask)) & f.keep;
        const uint32_t a = q & 0x7FFFFFFFu;
        const uint32_t settled = a > f.min_norm - 0x00800000u ? ((t & 0x80000000u) | f.min_norm) : 0u;
        return __uint_as_float(a < f.min_norm ? settled : q);
    }
    // values below the smallest normal are lifted into its binade, rounded there and brought back; for all others the
    // lift is zero and both additions leave the value as it is (a zero input counts as small, so -0 never meets + 0)
    const float lift = fabsf(x) < __uint_as_float(f.min_norm) ? copysignf(__uint_as_float(f.min_norm), x) : 0.0f;
    const uint32_t v = __float_as_uint(add_rn(x, lift));
    const uint32_t q = (v + (rnd & f.rmask)) & f.keep;
    return add_rn(__uint_as_float(q), -lift);
}
// One accumulation step; FAST: the caller has shown that nothing can leave the formats' ranges.
template <bool FMA, bool FAST, bool NOSUB = false>
__device__ __forceinline__ float sr_mac(float acc, float a, float b, uint32_t radd_word, uint32_t rmul_word, const MmParams& p) {
    if (FAST) {
        if (FMA) return sr_inrange<NOSUB>(p.sadd, fma_rn(a, b, acc), radd_word);
        return sr_inrange<NOSUB>(p.sadd, add_rn(acc, sr_inrange<NOSUB>(p.smul, mul_rn(a, b), rmul_word)), radd_word);
    }
    if (FMA) return sr_add(p, fma_rn(a, b, acc), radd_word);
    return sr_add(p, add_rn(acc, sr_mul(p, mul_rn(a, b), rmul_word)), radd_word);
}
// Eight steps (kglob .. kglob + 7, kglob a multiple of 8) for the thread's outputs on the fast path, one Philox call per
// output and PER steps.  The loop over the Philox calls stays rolled (the body, unrolled over the 32 outputs, is large).
template <bool FMA, bool NOSUB>
__device__ __forceinline__ void sr_group_fast(float (&acc)[TM][TN], const float* As, const float* Bs, int kbase, uint32_t kglob,
                                              int ty, int tx, int m0, int n0, int64_t batch, const MmParams& p) {
    constexpr int PER = FMA ? 4 : 2;          // accumulation steps served by one Philox call
    const uint64_t lin0 = (uint64_t)batch * p.M * p.N + (uint64_t)(m0 + ty) * p.N + (n0 + tx * 4);
#pragma unroll 1
    for (int c = 0; c < 8 / PER; ++c) {
        const int k0 = kbase + c * PER;
        float bv[PER][4];
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const float4 b4 = *reinterpret_cast<const float4*>(Bs + (k0 + u) * BN + tx * 4);
            bv[u][0] = b4.x; bv[u][1] = b4.y; bv[u][2] = b4.z; bv[u][3] = b4.w;
        }
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            float av[PER];
            if (FMA) {
                const float4 a4 = *reinterpret_cast<const float4*>(As + (ty + 16 * i) * AS_LD + k0);
                av[0] = a4.x; av[1] = a4.y; av[PER - 2] = a4.z; av[PER - 1] = a4.w;
            } else {
                const float2 a2 = *reinterpret_cast<const float2*>(As + (ty + 16 * i) * AS_LD + k0);
                av[0] = a2.x; av[1] = a2.y;
            }
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const uint64_t lin = lin0 + (uint64_t)(16 * i) * p.N + j;
                Philox ph(kglob / PER + c, (uint32_t)lin, (uint32_t)(lin >> 32), 0u);
                ph.run(p.seed_lo, p.seed_hi);
                float v = acc[i][j];
#pragma unroll
                for (int u = 0; u < PER; ++u)
                    v = FMA ? sr_mac<true, true, NOSUB>(v, av[u], bv[u][j], ph.c[u], 0u, p)
                            : sr_mac<false, true, NOSUB>(v, av[u], bv[u][j], ph.c[2 * u], ph.c[2 * u + 1], p);
                acc[i][j] = v;
            }
        }
    }
}
// The same eight steps on the whole-domain casters: an out-of-line function over a copy of the accumulators in local
// memory, with every loop rolled, so that this rarely taken path costs the fast one neither registers nor code size.
template <bool FMA>
static __device__ __noinline__ void sr_group_exact(float* accv, const float* As, const float* Bs, int kbase, uint32_t kglob,
                                                   int ty, int tx, int m0, int n0, int64_t batch, const MmParams* pp) {
    const MmParams& p = *pp;
    constexpr int PER = FMA ? 4 : 2;
#pragma unroll 1
    for (int o = 0; o < TM * TN; ++o) {
        const int i = o / TN, j = o % TN;
        const uint64_t lin = (uint64_t)batch * p.M * p.N + (uint64_t)(m0 + ty + 16 * i) * p.N + (n0 + tx * 4 + j);
        float v = accv[o];
#pragma unroll 1
        for (int c = 0; c < 8 / PER; ++c) {
            Philox ph(kglob / PER + c, (uint32_t)lin, (uint32_t)(lin >> 32), 0u);
            ph.run(p.seed_lo, p.seed_hi);
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int k = kbase + c * PER + u;
                const float a = As[(ty + 16 * i) * AS_LD + k], b = Bs[k * BN + tx * 4 + j];
                v = FMA ? sr_mac<true, false>(v, a, b, ph.c[u], 0u, p) : sr_mac<false, false>(v, a, b, ph.c[2 * u], ph.c[2 * u + 1], p);
            }
        }
        accv[o] = v;
    }
}

__device__ __forceinline__ float absmax_of(const float (&v)[TM][TN]) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) m = fmaxf(m, fabsf(v[i][j]));   // NaN entries are skipped by fmaxf
    return m;
}

// What the fast path may assume for this launch, from the operand statistics.
//   ok        : products can take the fast rounding (finite, no overflow in the multiply format,
//               no fp32-denormal intermediates where the reference treats those specially)
//   acc_limit : an accumulator with |acc| below this stays on the fast path for 8 more steps
//               (ALGO_SEQ), or an outer sum below this takes the fast fold (ALGO_TILE8)
struct FastPlan { bool ok; float acc_limit; };

// Formats without subnormals qualify when the launch is of the NOSUB instantiation (the host decides; the kernel's
// roundings then settle what lands below the smallest normal value the way the reference does).
__host__ __device__ inline bool mm_fast_format_nosub(const FpFmt& f) { return !f.sub && f.man <= 21 && f.exp >= 2; }

template <int ALGO, bool FMA>
__device__ __forceinline__ FastPlan make_plan(const MmParams& p, int64_t batch) {
    FastPlan plan{false, 0.0f};
    if (p.stats == nullptr) return plan;
    const MmStats s = p.stats[batch];
    if (s.max_a >= 0x7F800000u || s.max_b >= 0x7F800000u) return plan;
    // |a| < 2^(ea+1), |b| < 2^(eb+1)  =>  |a*b| < 2^pe
    const int pe = (int)(s.max_a >> 23) + (int)(s.max_b >> 23) - 254 + 2;
    if (ALGO == ALGO_SR) {
        // stochastic rounding moves a value by less than one quantum: a product below 2^pe stays at or below 2^pe, a sum
        // grows by at most (1 + 2^-man) per step; nothing may reach the upper edge of the top binade (the exponent clip)
        if (!p.sr_ok && !p.sr_nosub) return plan;
        const int top_add = p.fadd.max_store - 127, top_mul = p.fmul.max_store - 127;
        if (!FMA && pe > top_mul) return plan;
        const float lim = ldexpf(1.0f, top_add) / p.growth8_sr - ldexpf(8.0f, pe);
        if (!(lim > 0.0f)) return plan;
        plan.ok = true;
        plan.acc_limit = lim;
        return plan;
    }
    const bool nosub = p.nosub != 0;
    if (nosub ? (!mm_fast_format_nosub(p.fadd) || (!FMA && !mm_fast_format_nosub(p.fmul)))
              : (!mm_fast_format(p.fadd) || (!FMA && !mm_fast_format(p.fmul)))) return plan;
    if (nosub && ALGO == ALGO_KAHAN) return plan;
    // the compensated sum's bounds are worked out for formats that round; it keeps the exact path for the identity
    if (ALGO == ALGO_KAHAN && (fmt_identity(p.fadd) || (!FMA && fmt_identity(p.fmul)))) return plan;
    const int lim_add = fast_rn_exp_limit(p.fadd);
    if (!FMA && pe - 1 > fast_rn_exp_limit(p.fmul)) return plan;
    // (without subnormals every value is rounded at its own exponent, which the FP-pipe rounding does for normal
    // fp32 numbers only: the same proof that no nonzero intermediate is an fp32 denormal is needed)
    if (nosub || p.fadd.exp == 8 || (!FMA && p.fmul.exp == 8)) {
        // the reference rounds fp32-denormal inputs of 8-bit-exponent formats one bit coarser;
        // stay exact unless every nonzero intermediate is provably far above 2^-126
        if (s.minnz_a < 0x00800000u || s.minnz_b < 0x00800000u) return plan;
        if (s.minnz_a != 0xFFFFFFFFu && s.minnz_b != 0xFFFFFFFFu) {
            // a rounded product is a multiple of 2^(lo - 23), an exact (fused) one of 2^(lo - 46); sums, differences
            // and roundings of such multiples are multiples again, so nothing nonzero can fall below that grid
            const int lo = (int)(s.minnz_a >> 23) + (int)(s.minnz_b >> 23) - 254;
            if (lo - (FMA ? 46 : 23) < -120) return plan;
        }
    }
    // eight steps from |acc| = x reach at most (x + 8 * 2^pe) * growth8
    const float step8 = ldexpf(8.0f, pe) * p.growth8;
    const float top = ldexpf(1.0f, lim_add + 1);
    if (ALGO == ALGO_KAHAN) {
        const float lim = (top - p.kah_p * ldexpf(1.0f, pe) - p.kah_const) / p.kah_sc;
        if (!(lim > 0.0f)) return plan;
        plan.ok = true;
        plan.acc_limit = lim;
    } else if (ALGO == ALGO_TILE8) {
        // inner sums start from zero: |inner| <= step8; the fold needs |outer| + |inner| < top
        if (!(step8 <= ldexpf(1.0f, lim_add))) return plan;
        plan.ok = true;
        plan.acc_limit = ldexpf(1.0f, lim_add);
    } else {
        const float lim = top / p.growth8 - ldexpf(8.0f, pe);
        if (!(lim > 0.0f)) return plan;
        plan.ok = true;
        plan.acc_limit = lim;
    }
    return plan;
}

template <int ALGO, bool FMA, bool VEC, bool PACKED, bool ADDG, int CONV = CONV_NONE, int MINB = MPT_MM_MIN_CTAS, bool NOSUB = false>
__global__ void __launch_bounds__(THREADS, MINB) mm_kernel(const __grid_constant__ MmParams p) {
    extern __shared__ __align__(16) float smem[];
    float* As = smem;
    float* Bs = smem + STAGES * SMEM_A;
    ConvRow* crow = reinterpret_cast<ConvRow*>(smem + STAGES * (SMEM_A + SMEM_B));      // CONV: BM entries

    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    // CTAs are launched x-fastest; walking the output in bands of kGroupM row tiles (all column tiles of a band before
    // the next band) keeps the A rows and B columns that concurrently resident CTAs share inside L2, so the operands
    // are read from HBM a few times instead of once per row of tiles.
    int tile_m, tile_n;
    {
        constexpr int kGroupM = 8;
        // 64-bit: gridDim.x * gridDim.y can pass 2^31 for a very wide N
        const uint64_t pid = (uint64_t)blockIdx.y * gridDim.x + blockIdx.x;
        const uint64_t per_band = (uint64_t)kGroupM * gridDim.x;
        const int band = (int)(pid / per_band);
        const uint64_t in_band = pid - (uint64_t)band * per_band;
        const int first_m = band * kGroupM;
        const int rows_here = min((int)gridDim.y - first_m, kGroupM);
        tile_n = (int)(in_band / (unsigned)rows_here);
        tile_m = first_m + (int)(in_band - (uint64_t)tile_n * rows_here);
    }
    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int64_t batch = blockIdx.z;
    const float* A = p.a + batch * p.stride_a;
    const float* B = p.b + batch * p.stride_b;
    float* C = p.c + batch * p.stride_c;

    // number of accumulation steps walked: exactly K for the sequential order, the zero-padded
    // range K + 8 - K % 8 for every order that follows the reference CUDA kernels
    const int ksteps = (ALGO == ALGO_SEQ || (p.resume & MM_MORE)) ? p.K : p.K + 8 - p.K % 8;
    const int ntiles = (ksteps + BK - 1) / BK;

    const FastPlan plan = make_plan<ALGO, FMA>(p, batch);
    if (CONV == CONV_NONE && p.defer_exact && !plan.ok) return;

    if (CONV == CONV_FWD) {
        if (tid < BM) {
            const int gm = m0 + tid;
            ConvRow r;
            if (gm < p.M) {
                const int L = p.cv.OH * p.cv.OW;
                const int img = gm / L, l = gm - img * L;
                const int oh = l / p.cv.OW, ow = l - oh * p.cv.OW;
                r.base = (int64_t)img * p.cv.x_image_stride;
                r.ih0 = oh * p.cv.sh - p.cv.ph;
                r.iw0 = ow * p.cv.sw - p.cv.pw;
            } else {
                r.base = 0; r.ih0 = -(1 << 30); r.iw0 = -(1 << 30);      // fails every bounds check: zero rows
            }
            crow[tid] = r;
        }
        __syncthreads();
    }

    float acc[TM][TN];    // running sum (inner sum for ALGO_TILE8)
    float aux[TM][TN];    // outer sum (ALGO_TILE8) or compensation term (ALGO_KAHAN)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) { acc[i][j] = 0.0f; aux[i][j] = 0.0f; }
    if (CONV == CONV_NONE && (ALGO == ALGO_SEQ || ALGO == ALGO_TILE8) && (p.resume & MM_FROM_C)) {
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int gm = m0 + ty + 16 * i;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int gn = n0 + tx * 4 + j;
                const float v = (gm < p.M && gn < p.N) ? C[(int64_t)gm * p.N + gn] : 0.0f;
                if (ALGO == ALGO_TILE8) aux[i][j] = v; else acc[i][j] = v;
            }
        }
    }

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < ntiles) load_tiles<VEC, CONV>(p, A, B, As + s * SMEM_A, Bs + s * SMEM_B, m0, n0, s * BK, tid, crow);
        cp_async_commit();
    }

    for (int t = 0; t < ntiles; ++t) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nt = t + STAGES - 1;
            if (nt < ntiles) load_tiles<VEC, CONV>(p, A, B, As + (nt % STAGES) * SMEM_A, Bs + (nt % STAGES) * SMEM_B, m0, n0, nt * BK, tid, crow);
            cp_async_commit();
        }
        const float* as = As + (t % STAGES) * SMEM_A;
        const float* bs = Bs + (t % STAGES) * SMEM_B;
        const int kleft = ksteps - t * BK;
        const int nk_tile = kleft < BK ? kleft : BK;

        if (ALGO == ALGO_SEQ || ALGO == ALGO_TILE8) {
            for (int g = 0; g * 8 < nk_tile; ++g) {
                const int nk = (nk_tile - g * 8) < 8 ? (nk_tile - g * 8) : 8;
                if (ALGO == ALGO_TILE8) {
                    if (plan.ok) {
                        // without subnormals: a flagged group starts over from its zeros on the exact casters
                        if (group_steps<FMA, true, PACKED, ADDG, NOSUB, NOSUB>(acc, as, bs, g * 8, nk, ty, tx, p)) {
#pragma unroll
                            for (int i = 0; i < TM; ++i)
#pragma unroll
                                for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
                            group_steps<FMA, false, false, true>(acc, as, bs, g * 8, nk, ty, tx, p);
                        }
                    } else group_steps<FMA, false, false, true>(acc, as, bs, g * 8, nk, ty, tx, p);
                    // fold the group into the outer sum
                    if (plan.ok && absmax_of(aux) < plan.acc_limit) {
#pragma unroll
                        for (int i = 0; i < TM; ++i) {
                            if (PACKED) {
                                const float2 lo = fast_rn2<ADDG>(p.radd, __fadd2_rn(make_float2(aux[i][0], aux[i][1]), make_float2(acc[i][0], acc[i][1])));
                                const float2 hi = fast_rn2<ADDG>(p.radd, __fadd2_rn(make_float2(aux[i][2], aux[i][3]), make_float2(acc[i][2], acc[i][3])));
                                aux[i][0] = lo.x; aux[i][1] = lo.y; aux[i][2] = hi.x; aux[i][3] = hi.y;
                            } else {
#pragma unroll
                                for (int j = 0; j < TN; ++j)
                                    aux[i][j] = NOSUB ? fast_rn_nosub_rare(p.radd, add_rn(aux[i][j], acc[i][j])) : p.radd(add_rn(aux[i][j], acc[i][j]));
                            }
#pragma unroll
                            for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < TM; ++i)
#pragma unroll
                            for (int j = 0; j < TN; ++j) { aux[i][j] = cast_any(add_rn(aux[i][j], acc[i][j]), p.gadd); acc[i][j] = 0.0f; }
                    }
                } else {
                    if (plan.ok && absmax_of(acc) < plan.acc_limit) group_steps<FMA, true, PACKED, ADDG, NOSUB>(acc, as, bs, g * 8, nk, ty, tx, p);
                    else group_steps<FMA, false, false, true>(acc, as, bs, g * 8, nk, ty, tx, p);
                }
            }
        } else if (ALGO == ALGO_KAHAN) {
            // the reference pads K to a multiple of 8 (and walks the padding), so a tile is whole groups of 8 steps
            for (int g = 0; g * 8 < nk_tile; ++g) {
                if (PACKED && plan.ok && absmax_of(acc) < plan.acc_limit && absmax_of(aux) < plan.acc_limit) {
                    kahan_group_fast<FMA, ADDG>(acc, aux, as, bs, g * 8, ty, tx, p);
                } else {
#pragma unroll 1
                    for (int k = g * 8; k < g * 8 + 8; ++k) {
                        const float4 bv4 = *reinterpret_cast<const float4*>(bs + k * BN + tx * 4);
                        const float bvv[4] = {bv4.x, bv4.y, bv4.z, bv4.w};
#pragma unroll
                        for (int i = 0; i < TM; ++i) {
                            const float a = as[(ty + 16 * i) * AS_LD + k];
#pragma unroll
                            for (int j = 0; j < TN; ++j) kahan_exact<FMA>(acc[i][j], aux[i][j], a, bvv[j], p);
                        }
                    }
                }
            }
        } else {   // ALGO_SR
            for (int g = 0; g * 8 < nk_tile; ++g) {
                const uint32_t kglob = (uint32_t)(t * BK + g * 8);
                if (plan.ok && absmax_of(acc) < plan.acc_limit) sr_group_fast<FMA, NOSUB>(acc, as, bs, g * 8, kglob, ty, tx, m0, n0, batch, p);
                else {
                    float tmp[TM * TN];
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) tmp[i * TN + j] = acc[i][j];
                    sr_group_exact<FMA>(tmp, as, bs, g * 8, kglob, ty, tx, m0, n0, batch, &p);
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) acc[i][j] = tmp[i * TN + j];
                }
            }
        }
    }
    cp_async_wait<0>();

    // epilogue
    if (CONV == CONV_FWD) {     // C[m][n] goes to y[image][n][oh][ow]: consecutive m are consecutive addresses
        const int L = p.cv.OH * p.cv.OW;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int gm = m0 + ty + 16 * i;
            if (gm >= p.M) continue;
            const int img = gm / L, l = gm - img * L;
            const float* r = (ALGO == ALGO_TILE8) ? aux[i] : acc[i];
            float* dst = C + (int64_t)img * p.cv.y_image_stride + l;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int gn = n0 + tx * 4 + j;
                if (gn < p.N) dst[(int64_t)gn * L] = r[j];
            }
        }
        return;
    }
    const bool vec_store = VEC && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty + 16 * i;
        if (gm >= p.M) continue;
        const float* r = (ALGO == ALGO_TILE8) ? aux[i] : acc[i];
        const int gn = n0 + tx * 4;
        float* dst = C + (int64_t)gm * p.N + gn;
        if (vec_store && gn + 3 < p.N) *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
        else {
#pragma unroll
            for (int j = 0; j < TN; ++j)
                if (gn + j < p.N) dst[j] = r[j];
        }
    }
}

// The packed fp32x2 fast path is the default; MPT_MM_SCALAR=1 in the environment selects the scalar
// fast path (same bits; kept for A/B measurements).
inline bool use_packed() {
    static const bool packed = [] { const char* e = getenv("MPT_MM_SCALAR"); return !(e && e[0] == '1'); }();
    return packed;
}

// TILE_ROWS names the tile height of the including translation unit, so that units built with different heights
// instantiate different functions.
template <int ALGO, bool FMA, int TILE_ROWS = BM>
int launch_mm(const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    static_assert(TILE_ROWS == BM, "one tile height per translation unit");
    dim3 grid((unsigned)(((int64_t)p.N + BN - 1) / BN), (unsigned)(((int64_t)p.M + BM - 1) / BM), (unsigned)batch);
    if (grid.y > 65535u) { set_error("float_mm: M=%d has more than 65535 row tiles of %d", p.M, BM); return MPT_ERR_INVALID_ARGUMENT; }
    // The stochastic kernel has one form (scalar, both clamps); its translation unit picks tile height and residency.
    constexpr bool kHasFast = ALGO != ALGO_SR;
    constexpr int kMinB = ALGO == ALGO_SR ? MPT_MM_SR_MIN_CTAS : MPT_MM_MIN_CTAS;
    const bool packed = kHasFast && use_packed();
    // the sum rounding needs its subnormal clamp only if products can carry bits below the add format's
    // smallest subnormal (always the case for a fused multiply-add, whose sum is not a sum of rounded values)
    const bool add_guard = FMA || !packed || (p.fmul.min_exp - p.fmul.man) < (p.fadd.min_exp - p.fadd.man);
    constexpr bool kCanDrop = kHasFast && !FMA;
    auto kern = vec ? (packed ? (add_guard ? mm_kernel<ALGO, FMA, true, kHasFast, true, CONV_NONE, kMinB> : mm_kernel<ALGO, FMA, true, kHasFast, !kCanDrop, CONV_NONE, kMinB>)
                              : mm_kernel<ALGO, FMA, true, false, true, CONV_NONE, kMinB>)
                    : (packed ? (add_guard ? mm_kernel<ALGO, FMA, false, kHasFast, true, CONV_NONE, kMinB> : mm_kernel<ALGO, FMA, false, kHasFast, !kCanDrop, CONV_NONE, kMinB>)
                              : mm_kernel<ALGO, FMA, false, false, true, CONV_NONE, kMinB>);
    if (ALGO == ALGO_SR && p.sr_nosub)      // formats without subnormals: the instantiation with their in-range rounding
        kern = vec ? mm_kernel<ALGO, FMA, true, false, true, CONV_NONE, kMinB, true> : mm_kernel<ALGO, FMA, false, false, true, CONV_NONE, kMinB, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) { set_error("float_mm: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(p);
    return check_launch("float_mm");
}

// Formats without subnormals: the scalar range-checked path with the settling rounding (fast_rn_nosub).
template <int ALGO, bool FMA, int TILE_ROWS = BM>
int launch_mm_nosub_t(const MmParams& p, int64_t batch, bool vec, cudaStream_t st) {
    static_assert(TILE_ROWS == BM, "one tile height per translation unit");
    dim3 grid((unsigned)(((int64_t)p.N + BN - 1) / BN), (unsigned)(((int64_t)p.M + BM - 1) / BM), (unsigned)batch);
    if (grid.y > 65535u) { set_error("float_mm: M=%d has more than 65535 row tiles of %d", p.M, BM); return MPT_ERR_INVALID_ARGUMENT; }
    auto kern = vec ? mm_kernel<ALGO, FMA, true, false, true, CONV_NONE, MPT_MM_MIN_CTAS, true>
                    : mm_kernel<ALGO, FMA, false, false, true, CONV_NONE, MPT_MM_MIN_CTAS, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) { set_error("float_mm: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(p);
    return check_launch("float_mm");
}

// Convolution launch: scalar operand copies (the gather has no 16-byte runs), packed fast path.
template <int ALGO, bool FMA>
int launch_conv(const MmParams& p, cudaStream_t st) {
    dim3 grid((unsigned)(((int64_t)p.N + BN - 1) / BN), (unsigned)(((int64_t)p.M + BM - 1) / BM), 1);
    const bool add_guard = FMA || (p.fmul.min_exp - p.fmul.man) < (p.fadd.min_exp - p.fadd.man);
    auto kern = add_guard ? mm_kernel<ALGO, FMA, false, true, true, CONV_FWD> : mm_kernel<ALGO, FMA, false, true, FMA, CONV_FWD>;
    if (p.nosub) kern = mm_kernel<ALGO, FMA, false, false, true, CONV_FWD, MPT_MM_MIN_CTAS, true>;      // formats without subnormals
    const size_t smem = SMEM_BYTES + BM * sizeof(ConvRow);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("float_conv2d: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    kern<<<grid, THREADS, smem, st>>>(p);
    return check_launch("float_conv2d");
}

// Weight-gradient launch: both operands are gathered with scalar copies; the result is an ordinary row-major matrix.
// TILE_ROWS names the tile height of the including translation unit, so that units built with different heights
// instantiate different functions.
template <int ALGO, bool FMA, int TILE_ROWS = BM>
int launch_conv_wgrad(const MmParams& p, cudaStream_t st) {
    static_assert(TILE_ROWS == BM, "one tile height per translation unit");
    dim3 grid((unsigned)(((int64_t)p.N + BN - 1) / BN), (unsigned)(((int64_t)p.M + BM - 1) / BM), 1);
    const bool add_guard = FMA || (p.fmul.min_exp - p.fmul.man) < (p.fadd.min_exp - p.fadd.man);
    auto kern = add_guard ? mm_kernel<ALGO, FMA, false, true, true, CONV_WGRAD> : mm_kernel<ALGO, FMA, false, true, FMA, CONV_WGRAD>;
    if (p.nosub) kern = mm_kernel<ALGO, FMA, false, false, true, CONV_WGRAD, MPT_MM_MIN_CTAS, true>;    // formats without subnormals
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) { set_error("float_conv2d_wgrad: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(p);
    return check_launch("float_conv2d_wgrad");
}

// Defined in the instantiation files.
int launch_mm_seq(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);
int launch_mm_tile8(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);
int launch_mm_kahan(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);
int launch_mm_sr(bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);
int launch_conv_any(int algo, bool fma, const MmParams& p, cudaStream_t st);
int launch_conv_wgrad_any(int algo, bool fma, const MmParams& p, cudaStream_t st);
int launch_conv_wgrad_small_any(int algo, bool fma, const MmParams& p, cudaStream_t st);
int launch_mm_small(int algo, bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);   // ALGO_SEQ / ALGO_TILE8
int launch_mm_exact(int algo, bool fma, const MmParams& p, int64_t batch, cudaStream_t st);             // all but ALGO_SR
int launch_mm_nosub(int algo, bool fma, const MmParams& p, int64_t batch, bool vec, cudaStream_t st);  // ALGO_SEQ / ALGO_TILE8
constexpr int kSmallTileRows = 16;      // tile height of the instantiation behind launch_conv_wgrad_small_any

}  // namespace mpt
