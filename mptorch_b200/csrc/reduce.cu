// Quantized row reductions: softmax (division and log-sum-exp forms, backward) and layer
// normalisation (forward, backward), every intermediate rounded to its user format.
//
// A tensor is viewed as [outer, channel, inner]; a "row" is the `channel` elements at a fixed
// (outer, inner) position, `inner` elements apart.
//
// Two associations of the row sums are provided, both bit-exact with their reference:
//   MPT_ORDER_CUDA  the reference CUDA kernels' order (quant_cuda/softmax_kernel.h:23-222,
//                   layernorm_kernel.h:7-237): 64 strided partial sums (element k belongs to
//                   partial k mod 64, accumulated in increasing k), two 32-wide shuffle trees with
//                   offsets 16, 8, 4, 2, 1, then tree0 (op) tree1.  Here ONE WARP owns a row and
//                   every lane carries two of the 64 partials (lane l: partials l and l + 32), so a
//                   row needs no shared memory and no block barrier, rows of 4 KB stay in L1/L2
//                   between the passes, and a CTA of 8 warps works on 8 rows at once.
//   MPT_ORDER_SEQ   the reference CPU loops (quant_cpu/softmax.h, layernorm.h): one running value
//                   per row, left to right; one thread per row.
// expf/logf/sqrtf/division are the same CUDA math functions the reference CUDA build calls; this
// file is compiled with nvcc's default floating-point flags for that reason, and every multiply,
// add and subtract of the algorithm itself is written with an explicit rounding intrinsic.
#include "cast.cuh"
#include "common.cuh"

namespace mpt {
namespace {

constexpr int kWarpsPerBlock = 8;

struct RowGeom {
    int64_t rows;      // outer * inner
    int channel;
    int64_t inner;
};

__device__ __forceinline__ int64_t row_base(const RowGeom& g, int64_t row) {
    return (row / g.inner) * (int64_t)g.channel * g.inner + row % g.inner;
}

// Fold the 64 partials held as (p0, p1) per lane; every lane receives the result.
template <class Op>
__device__ __forceinline__ float tree64(float p0, float p1, Op op) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float o0 = __shfl_down_sync(0xFFFFFFFFu, p0, off);
        const float o1 = __shfl_down_sync(0xFFFFFFFFu, p1, off);
        p0 = op(p0, o0);
        p1 = op(p1, o1);
    }
    const float r = op(p0, p1);
    return __shfl_sync(0xFFFFFFFFu, r, 0);
}

struct QAdd {
    FpFmt f;
    __device__ __forceinline__ float operator()(float a, float b) const { return cast_fp_nearest(__fadd_rn(a, b), f); }
};
struct FMax {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};
struct QLse {
    FpFmt f;
    __device__ __forceinline__ float operator()(float a, float b) const {
        return cast_fp_nearest(logf(__fadd_rn(expf(a), expf(b))), f);
    }
};

// ----------------------------------------------------------------------------------------- softmax
template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                         RowGeom g, FpFmt fexp, FpFmt foff, FpFmt facc) {
    const QAdd qadd{facc};
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        const float* x = in + row_base(g, row);
        float* y = out + row_base(g, row);
        const int C = g.channel;
        const int64_t st = g.inner;
        float m0 = -INFINITY, m1 = -INFINITY;
        for (int k = lane; k < C; k += 64) {
            m0 = fmaxf(m0, x[k * st]);
            if (k + 32 < C) m1 = fmaxf(m1, x[(k + 32) * st]);
        }
        const float mx = tree64(m0, m1, FMax{});
        float s0 = 0.f, s1 = 0.f;
        for (int k = lane; k < C; k += 64) {
            const float e0 = cast_fp_nearest(expf(cast_fp_nearest(__fsub_rn(x[k * st], mx), foff)), fexp);
            y[k * st] = e0;
            s0 = qadd(s0, e0);
            if (k + 32 < C) {
                const float e1 = cast_fp_nearest(expf(cast_fp_nearest(__fsub_rn(x[(k + 32) * st], mx), foff)), fexp);
                y[(k + 32) * st] = e1;
                s1 = qadd(s1, e1);
            }
        }
        const float sum = tree64(s0, s1, qadd);
        for (int k = lane; k < C; k += 32) y[k * st] = __fdiv_rn(y[k * st], sum);
    } else {
        const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (row >= g.rows) return;
        const float* x = in + row_base(g, row);
        float* y = out + row_base(g, row);
        const int C = g.channel;
        const int64_t st = g.inner;
        float mx = x[0];
        for (int k = 1; k < C; ++k) mx = fmaxf(mx, x[k * st]);
        float sum = 0.f;
        for (int k = 0; k < C; ++k) {
            const float e = cast_fp_nearest(expf(cast_fp_nearest(__fsub_rn(x[k * st], mx), foff)), fexp);
            y[k * st] = e;
            sum = qadd(sum, e);
        }
        for (int k = 0; k < C; ++k) y[k * st] = __fdiv_rn(y[k * st], sum);
    }
}

template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_lse_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                             RowGeom g, FpFmt foff, FpFmt flse) {
    const QLse qlse{flse};
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        const float* x = in + row_base(g, row);
        float* y = out + row_base(g, row);
        const int C = g.channel;
        const int64_t st = g.inner;
        float m0 = -INFINITY, m1 = -INFINITY;
        for (int k = lane; k < C; k += 64) {
            m0 = fmaxf(m0, x[k * st]);
            if (k + 32 < C) m1 = fmaxf(m1, x[(k + 32) * st]);
        }
        const float mx = tree64(m0, m1, FMax{});
        float l0 = -INFINITY, l1 = -INFINITY;
        for (int k = lane; k < C; k += 64) {
            const float v0 = cast_fp_nearest(__fsub_rn(x[k * st], mx), foff);
            y[k * st] = v0;
            l0 = qlse(l0, v0);
            if (k + 32 < C) {
                const float v1 = cast_fp_nearest(__fsub_rn(x[(k + 32) * st], mx), foff);
                y[(k + 32) * st] = v1;
                l1 = qlse(l1, v1);
            }
        }
        const float lgs = tree64(l0, l1, qlse);
        for (int k = lane; k < C; k += 32) y[k * st] = expf(cast_fp_nearest(__fsub_rn(y[k * st], lgs), foff));
    } else {
        const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (row >= g.rows) return;
        const float* x = in + row_base(g, row);
        float* y = out + row_base(g, row);
        const int C = g.channel;
        const int64_t st = g.inner;
        float mx = x[0];
        for (int k = 1; k < C; ++k) mx = fmaxf(mx, x[k * st]);
        float lgs = cast_fp_nearest(__fsub_rn(x[0], mx), foff);   // the CPU loop seeds with the first element
        y[0] = lgs;
        for (int k = 1; k < C; ++k) {
            const float v = cast_fp_nearest(__fsub_rn(x[k * st], mx), foff);
            y[k * st] = v;
            lgs = qlse(lgs, v);
        }
        for (int k = 0; k < C; ++k) y[k * st] = expf(cast_fp_nearest(__fsub_rn(y[k * st], lgs), foff));
    }
}

template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_bwd_kernel(const float* __restrict__ yv, const float* __restrict__ gv,
                                                                         float* __restrict__ out, RowGeom g, FpFmt fadd, FpFmt fmul) {
    const QAdd qadd{fadd};
    const int C = g.channel;
    const int64_t st = g.inner;
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        const int64_t base = row_base(g, row);
        const float *y = yv + base, *gr = gv + base;
        float* o = out + base;
        float s0 = 0.f, s1 = 0.f;
        for (int k = lane; k < C; k += 64) {
            s0 = qadd(s0, cast_fp_nearest(__fmul_rn(y[k * st], gr[k * st]), fmul));
            if (k + 32 < C) s1 = qadd(s1, cast_fp_nearest(__fmul_rn(y[(k + 32) * st], gr[(k + 32) * st]), fmul));
        }
        const float s = tree64(s0, s1, qadd);
        for (int k = lane; k < C; k += 32) o[k * st] = __fmul_rn(cast_fp_nearest(__fsub_rn(gr[k * st], s), fadd), y[k * st]);
    } else {
        const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (row >= g.rows) return;
        const int64_t base = row_base(g, row);
        const float *y = yv + base, *gr = gv + base;
        float* o = out + base;
        float s = 0.f;
        for (int k = 0; k < C; ++k) s = qadd(s, cast_fp_nearest(__fmul_rn(y[k * st], gr[k * st]), fmul));
        for (int k = 0; k < C; ++k) o[k * st] = __fmul_rn(cast_fp_nearest(__fsub_rn(gr[k * st], s), fadd), y[k * st]);
    }
}

// ----------------------------------------------------------------------------------------- layernorm
struct LnFmt { FpFmt acc, mul, div, sqrt; };

template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_fwd_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                                           const float* __restrict__ bias, float* __restrict__ out,
                                                                           float* __restrict__ mean, float* __restrict__ rstd,
                                                                           float eps, RowGeom g, LnFmt f) {
    const QAdd qacc{f.acc};
    const int C = g.channel;
    const int64_t st = g.inner;
    const float fC = (float)C;
    int64_t row;
    int lane = 0, step = 1;
    if (TREE) {
        lane = threadIdx.x & 31; step = 32;
        row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    } else {
        row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    }
    if (row >= g.rows) return;
    const float* x = in + row_base(g, row);
    float* y = out + row_base(g, row);
    float m, var;
    if (TREE) {
        float s0 = 0.f, s1 = 0.f;
        for (int k = lane; k < C; k += 64) {
            s0 = qacc(s0, x[k * st]);
            if (k + 32 < C) s1 = qacc(s1, x[(k + 32) * st]);
        }
        m = __fdiv_rn(tree64(s0, s1, qacc), fC);               // the CUDA kernel leaves the mean unrounded
        s0 = 0.f; s1 = 0.f;
        for (int k = lane; k < C; k += 64) {
            const float d0 = cast_fp_nearest(__fsub_rn(x[k * st], m), f.acc);
            s0 = qacc(s0, cast_fp_nearest(__fmul_rn(d0, d0), f.mul));
            if (k + 32 < C) {
                const float d1 = cast_fp_nearest(__fsub_rn(x[(k + 32) * st], m), f.acc);
                s1 = qacc(s1, cast_fp_nearest(__fmul_rn(d1, d1), f.mul));
            }
        }
        var = __fdiv_rn(tree64(s0, s1, qacc), fC);
    } else {
        float s = 0.f;
        for (int k = 0; k < C; ++k) s = qacc(s, x[k * st]);
        m = cast_fp_nearest(__fdiv_rn(s, fC), f.div);          // the CPU loop rounds mean and variance
        s = 0.f;
        for (int k = 0; k < C; ++k) {
            const float d = cast_fp_nearest(__fsub_rn(x[k * st], m), f.acc);
            s = qacc(s, cast_fp_nearest(__fmul_rn(d, d), f.mul));
        }
        var = cast_fp_nearest(__fdiv_rn(s, fC), f.div);
    }
    const float sd = cast_fp_nearest(__fsqrt_rn(cast_fp_nearest(__fadd_rn(var, eps), f.acc)), f.sqrt);
    for (int k = lane; k < C; k += step) {
        const float norm = cast_fp_nearest(__fdiv_rn(cast_fp_nearest(__fsub_rn(x[k * st], m), f.acc), sd), f.div);
        y[k * st] = __fadd_rn(cast_fp_nearest(__fmul_rn(w[k], norm), f.mul), bias[k]);
    }
    if (lane == 0) {
        mean[row] = m;
        rstd[row] = cast_fp_nearest(__fdiv_rn(1.0f, sd), f.div);
    }
}

// Input gradient, one row per warp (or per thread in sequential order).
template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_bwd_dx_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                              const float* __restrict__ w, const float* __restrict__ mean,
                                                                              const float* __restrict__ rstd, float* __restrict__ gin,
                                                                              RowGeom g, LnFmt f) {
    const QAdd qacc{f.acc};
    const int C = g.channel;
    const int64_t st = g.inner;
    const float fC = (float)C;
    int64_t row;
    int lane = 0, step = 1;
    if (TREE) {
        lane = threadIdx.x & 31; step = 32;
        row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    } else {
        row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    }
    if (row >= g.rows) return;
    const int64_t base = row_base(g, row);
    const float *x = in + base, *gr = gout + base;
    float* o = gin + base;
    const float m = mean[row], r = rstd[row];
    auto terms = [&](int k, float& ng, float& dot) {
        const float xhat = cast_fp_nearest(__fmul_rn(cast_fp_nearest(__fsub_rn(x[k * st], m), f.acc), r), f.mul);
        ng = cast_fp_nearest(__fmul_rn(w[k], gr[k * st]), f.mul);
        dot = cast_fp_nearest(__fmul_rn(xhat, ng), f.mul);
    };
    float gs, gsx;
    if (TREE) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f, ng, dot;
        for (int k = lane; k < C; k += 64) {
            terms(k, ng, dot);
            a0 = qacc(a0, ng); b0 = qacc(b0, dot);
            if (k + 32 < C) {
                terms(k + 32, ng, dot);
                a1 = qacc(a1, ng); b1 = qacc(b1, dot);
            }
        }
        gs = tree64(a0, a1, qacc);
        gsx = tree64(b0, b1, qacc);
    } else {
        gs = 0.f; gsx = 0.f;
        float ng, dot;
        for (int k = 0; k < C; ++k) {
            terms(k, ng, dot);
            gs = qacc(gs, ng); gsx = qacc(gsx, dot);
        }
    }
    gs = cast_fp_nearest(__fdiv_rn(gs, fC), f.div);
    gsx = cast_fp_nearest(__fdiv_rn(gsx, fC), f.div);
    for (int k = lane; k < C; k += step) {
        const float xhat = cast_fp_nearest(__fmul_rn(cast_fp_nearest(__fsub_rn(x[k * st], m), f.acc), r), f.mul);
        const float ng = cast_fp_nearest(__fmul_rn(w[k], gr[k * st]), f.mul);
        const float wg = cast_fp_nearest(__fmul_rn(xhat, gsx), f.mul);
        float gi = cast_fp_nearest(__fsub_rn(ng, gs), f.acc);
        gi = cast_fp_nearest(__fsub_rn(gi, wg), f.acc);
        o[k * st] = cast_fp_nearest(__fmul_rn(gi, r), f.mul);
    }
}

// Weight and bias gradients: per channel, a sequential rounded sum over rows 0..R-1 (the order of
// both references).  One thread per channel; consecutive threads read consecutive channels, so each
// row is read coalesced.  x-hat * dy is recomputed from the inputs rather than staged through a
// scratch tensor as the reference does (layernorm_kernel.h:189, fp_kernel.cu:481-487): same values,
// one tensor less written and read.
__global__ void __launch_bounds__(128) layernorm_bwd_params_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                   float* __restrict__ ggamma, float* __restrict__ gbeta, RowGeom g, LnFmt f) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= g.channel) return;
    const QAdd qacc{f.acc};
    const int64_t st = g.inner;
    float gg = 0.f, gb = 0.f;
    constexpr int U = 8;
    int64_t row = 0;
    for (; row + U <= g.rows; row += U) {
        float xv[U], gv[U], mv[U], rv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t idx = row_base(g, row + u) + k * st;
            xv[u] = in[idx]; gv[u] = gout[idx]; mv[u] = mean[row + u]; rv[u] = rstd[row + u];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float xhat = cast_fp_nearest(__fmul_rn(cast_fp_nearest(__fsub_rn(xv[u], mv[u]), f.acc), rv[u]), f.mul);
            gg = qacc(gg, cast_fp_nearest(__fmul_rn(xhat, gv[u]), f.mul));
            gb = qacc(gb, gv[u]);
        }
    }
    for (; row < g.rows; ++row) {
        const int64_t idx = row_base(g, row) + k * st;
        const float xhat = cast_fp_nearest(__fmul_rn(cast_fp_nearest(__fsub_rn(in[idx], mean[row]), f.acc), rstd[row]), f.mul);
        gg = qacc(gg, cast_fp_nearest(__fmul_rn(xhat, gout[idx]), f.mul));
        gb = qacc(gb, gout[idx]);
    }
    ggamma[k] = gg;
    gbeta[k] = gb;
}

// Sequential rounded column sums of a [rows, cols] matrix: out[c] = fold_r Q(acc + x[r, c]), acc0 = 0.
__global__ void __launch_bounds__(128) qsum_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows, int64_t cols, FpFmt f) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const QAdd q{f};
    float acc = 0.f;
    constexpr int U = 8;
    int64_t r = 0;
    for (; r + U <= rows; r += U) {
        float v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = in[(r + u) * cols + c];
#pragma unroll
        for (int u = 0; u < U; ++u) acc = q(acc, v[u]);
    }
    for (; r < rows; ++r) acc = q(acc, in[r * cols + c]);
    out[c] = acc;
}

int check_geom(const char* who, int64_t outer, int channel, int64_t inner) {
    MPT_REQUIRE(outer >= 0 && channel >= 0 && inner >= 0, "%s: negative extent", who);
    return MPT_OK;
}

unsigned row_blocks(int64_t rows, bool tree) {
    const int64_t per = tree ? kWarpsPerBlock : kWarpsPerBlock * 32;
    return (unsigned)((rows + per - 1) / per);
}

}  // namespace
}  // namespace mpt

using namespace mpt;

extern "C" {

int mpt_float_softmax_forward(const float* in, float* out, int64_t outer, int channel, int64_t inner, int man_exp,
                              int exp_exp, int man_off, int exp_off, int man_acc, int exp_acc, int subnormals,
                              int saturate, int order, void* stream) {
    int rc = check_geom("softmax_forward", outer, channel, inner);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_exp, exp_exp) && valid_format(man_off, exp_off) && valid_format(man_acc, exp_acc),
                "softmax_forward: unsupported format");
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "softmax_forward: null pointer");
    const FpFmt fe = make_fmt(man_exp, exp_exp, subnormals, saturate), fo = make_fmt(man_off, exp_off, subnormals, saturate),
                fa = make_fmt(man_acc, exp_acc, subnormals, saturate);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree) softmax_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fe, fo, fa);
    else softmax_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fe, fo, fa);
    return check_launch("softmax_forward");
}

int mpt_float_softmax_lse_forward(const float* in, float* out, int64_t outer, int channel, int64_t inner, int man_off,
                                  int exp_off, int man_lse, int exp_lse, int subnormals, int saturate, int order,
                                  void* stream) {
    int rc = check_geom("softmax_lse_forward", outer, channel, inner);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_off, exp_off) && valid_format(man_lse, exp_lse), "softmax_lse_forward: unsupported format");
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "softmax_lse_forward: null pointer");
    const FpFmt fo = make_fmt(man_off, exp_off, subnormals, saturate), fl = make_fmt(man_lse, exp_lse, subnormals, saturate);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree) softmax_lse_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fo, fl);
    else softmax_lse_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fo, fl);
    return check_launch("softmax_lse_forward");
}

int mpt_float_softmax_backward(const float* y, const float* grad, float* out, int64_t outer, int channel, int64_t inner,
                               int man_add, int exp_add, int man_mul, int exp_mul, int subnormals, int saturate,
                               int order, void* stream) {
    int rc = check_geom("softmax_backward", outer, channel, inner);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_add, exp_add) && valid_format(man_mul, exp_mul), "softmax_backward: unsupported format");
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(y && grad && out, "softmax_backward: null pointer");
    const FpFmt fa = make_fmt(man_add, exp_add, subnormals, saturate), fm = make_fmt(man_mul, exp_mul, subnormals, saturate);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree) softmax_bwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(y, grad, out, g, fa, fm);
    else softmax_bwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(y, grad, out, g, fa, fm);
    return check_launch("softmax_backward");
}

int mpt_float_layernorm_forward(const float* in, const float* weight, const float* bias, float* out, float* mean,
                                float* rstd, float eps, int64_t outer, int channel, int64_t inner, int man_acc,
                                int exp_acc, int man_mul, int exp_mul, int man_div, int exp_div, int man_sqrt,
                                int exp_sqrt, int subnormals, int saturate, int order, void* stream) {
    int rc = check_geom("layernorm_forward", outer, channel, inner);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_acc, exp_acc) && valid_format(man_mul, exp_mul) && valid_format(man_div, exp_div) &&
                    valid_format(man_sqrt, exp_sqrt), "layernorm_forward: unsupported format");
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0) return MPT_OK;
    MPT_REQUIRE(channel > 0, "layernorm_forward: empty normalised shape");
    MPT_REQUIRE(in && weight && bias && out && mean && rstd, "layernorm_forward: null pointer");
    const LnFmt f{make_fmt(man_acc, exp_acc, subnormals, saturate), make_fmt(man_mul, exp_mul, subnormals, saturate),
                  make_fmt(man_div, exp_div, subnormals, saturate), make_fmt(man_sqrt, exp_sqrt, subnormals, saturate)};
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree) layernorm_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, weight, bias, out, mean, rstd, eps, g, f);
    else layernorm_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, weight, bias, out, mean, rstd, eps, g, f);
    return check_launch("layernorm_forward");
}

int mpt_float_layernorm_backward(const float* in, const float* grad_out, const float* weight, const float* mean,
                                 const float* rstd, float* grad_in, float* grad_gamma, float* grad_beta, int64_t outer,
                                 int channel, int64_t inner, int man_acc, int exp_acc, int man_mul, int exp_mul,
                                 int man_div, int exp_div, int subnormals, int saturate, int order, void* stream) {
    int rc = check_geom("layernorm_backward", outer, channel, inner);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_acc, exp_acc) && valid_format(man_mul, exp_mul) && valid_format(man_div, exp_div),
                "layernorm_backward: unsupported format");
    const RowGeom g{outer * inner, channel, inner};
    if (channel == 0) return MPT_OK;
    MPT_REQUIRE(grad_gamma && grad_beta, "layernorm_backward: null pointer");
    const FpFmt fm = make_fmt(man_mul, exp_mul, subnormals, saturate);
    const LnFmt f{make_fmt(man_acc, exp_acc, subnormals, saturate), fm, make_fmt(man_div, exp_div, subnormals, saturate), fm};
    if (g.rows > 0) {
        MPT_REQUIRE(in && grad_out && weight && mean && rstd && grad_in, "layernorm_backward: null pointer");
        const bool tree = order != MPT_ORDER_SEQ;
        if (tree) layernorm_bwd_dx_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        else layernorm_bwd_dx_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        rc = check_launch("layernorm_backward (input gradient)");
        if (rc) return rc;
    }
    layernorm_bwd_params_kernel<<<(channel + 127) / 128, 128, 0, as_stream(stream)>>>(in, grad_out, mean, rstd, grad_gamma, grad_beta, g, f);
    return check_launch("layernorm_backward (parameter gradients)");
}

int mpt_qsum_rows(const float* in, float* out, int64_t rows, int64_t cols, int man, int exp, int subnormals, int saturate,
                  void* stream) {
    MPT_REQUIRE(rows >= 0 && cols >= 0, "qsum_rows: negative extent");
    MPT_REQUIRE(valid_format(man, exp), "qsum_rows: unsupported format");
    if (cols == 0) return MPT_OK;
    MPT_REQUIRE(out && (rows == 0 || in), "qsum_rows: null pointer");
    qsum_rows_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, as_stream(stream)>>>(in, out, rows, cols, make_fmt(man, exp, subnormals, saturate));
    return check_launch("qsum_rows");
}

}
