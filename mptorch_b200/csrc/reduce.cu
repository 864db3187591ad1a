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
#include "reduce.cuh"

namespace mpt {
namespace {

// ----------------------------------------------------------------------------------------- softmax
template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                         RowGeom g, Caster fexp, Caster foff, Caster facc) {
    const QAdd qadd{facc};
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        softmax_fwd_row_tree(in + row_base(g, row), out + row_base(g, row), g.channel, g.inner, lane, fexp, foff, facc);
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
                                                                             RowGeom g, Caster foff, Caster flse) {
    const QLse qlse{flse};
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        softmax_lse_row_tree(in + row_base(g, row), out + row_base(g, row), g.channel, g.inner, lane, foff, flse);
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
                                                                         float* __restrict__ out, RowGeom g, Caster fadd, Caster fmul) {
    const QAdd qadd{fadd};
    const int C = g.channel;
    const int64_t st = g.inner;
    if (TREE) {
        const int lane = threadIdx.x & 31;
        const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
        if (row >= g.rows) return;
        const int64_t base = row_base(g, row);
        softmax_bwd_row_tree(yv + base, gv + base, out + base, C, st, lane, fadd, fmul);
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
template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_fwd_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                                           const float* __restrict__ bias, float* __restrict__ out,
                                                                           float* __restrict__ mean, float* __restrict__ rstd,
                                                                           float eps, RowGeom g, LnFmt f) {
    int64_t row;
    int lane = 0, step = 1;
    if (TREE) {
        lane = threadIdx.x & 31; step = 32;
        row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    } else {
        row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    }
    if (row >= g.rows) return;
    layernorm_fwd_row<TREE>(in + row_base(g, row), w, bias, out + row_base(g, row), mean, rstd, row, eps, g.channel, g.inner, lane, step, f);
}

// Input gradient, one row per warp (or per thread in sequential order).
template <bool TREE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_bwd_dx_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                              const float* __restrict__ w, const float* __restrict__ mean,
                                                                              const float* __restrict__ rstd, float* __restrict__ gin,
                                                                              RowGeom g, LnFmt f) {
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
    layernorm_bwd_row<TREE>(in + base, gout + base, w, mean[row], rstd[row], gin + base, g.channel, g.inner, lane, step, f);
}

// Column sums in row order: out[c] = fold over rows r = 0..R-1 of Q(acc + v[r, c]), the association of both
// references for the layernorm weight/bias gradients (layernorm_kernel.h:206-237, layernorm.h:100-103) and of
// the qsum loop (functional.py:736-748).  The chain per column is serial by definition, so the kernel splits
// the work by role: a CTA owns 32 columns; eight producer warps stream row tiles (64 rows x 32 columns,
// coalesced 128-byte row segments), do the per-element arithmetic that does not depend on the running sum
// (for layernorm: x-hat * dy, recomputed from the inputs instead of staged through the reference's scratch
// tensor, fp_kernel.cu:481-487) and park the addends in shared memory; one consumer warp per chain (lane =
// column) walks the parked tile in row order through the rounded adds, 32 rows per range check so that the
// dependent adds run back to back.  Tiles are double buffered: the consumers work on tile t while the producers
// fetch tile t + 1, with one barrier per tile.
// A chain's speed is set by the latency of its dependent adds, not by how many columns share a CTA, so the tile
// is narrow: 8 columns per CTA puts four times as many SMs to work on the per-element arithmetic of the producers
// (a 32-byte sector per row and tensor).  A producer warp covers 4 rows x 8 columns per load.
constexpr int kColTile = 8;         // columns per CTA
constexpr int kRowTile = 64;        // rows per tile
constexpr int kProducerWarps = 2;   // 32 rows of a tile each
constexpr int kColsumThreads(int mode) { return (kProducerWarps + (mode == 0 ? 2 : 1)) * 32; }

// MODE 0: layernorm parameter gradients (two chains: x-hat*dy -> out0, dy -> out1).  MODE 1: plain column sum of `in`.
template <int MODE>
__global__ void __launch_bounds__(kColsumThreads(MODE)) colsum_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                float* __restrict__ out0, float* __restrict__ out1, RowGeom g,
                                                                Caster facc, Caster fmul, SeqAdder seq) {
    __shared__ float sA[2][kRowTile][kColTile];
    __shared__ float sB[MODE == 0 ? 2 : 1][MODE == 0 ? kRowTile : 1][kColTile];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cl = lane & (kColTile - 1), rs = lane / kColTile;      // column within the tile, row within a 4-row group
    const int col = blockIdx.x * kColTile + cl;
    const bool col_ok = col < g.channel;
    const int64_t st = g.inner;
    const int64_t ntiles = (g.rows + kRowTile - 1) / kRowTile;

    // Producer warp w: rows 32 w .. 32 w + 31 of a tile, eight loads of 4 rows x 8 columns.  The loads of tile t + 2
    // are issued before the arithmetic of tile t + 1, so a tile's memory latency hides behind the previous tile's work.
    static_assert(kRowTile == 32 * kProducerWarps && kColTile == 8, "eight loads of 4 rows x 8 columns per producer warp");
    struct Tile { float xv[8], gv[8], mv[8], rv[8]; };
    auto load = [&](int64_t t, Tile& T) {
        const int64_t r0 = t * kRowTile + warp * 32 + rs;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int64_t row = r0 + 4 * u;
            const bool ok = col_ok && row < g.rows;
            const int64_t idx = ok ? row_base(g, row) + col * st : 0;
            T.xv[u] = ok ? in[idx] : 0.f;
            if (MODE == 0) { T.gv[u] = ok ? gout[idx] : 0.f; T.mv[u] = ok ? mean[row] : 0.f; T.rv[u] = ok ? rstd[row] : 0.f; }
        }
    };
    auto finish = [&](int64_t t, const Tile& T) {
        const int buf = (int)(t & 1);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int lr = warp * 32 + 4 * u + rs;
            if (MODE == 0) {
                const float xhat = fmul(__fmul_rn(facc(__fsub_rn(T.xv[u], T.mv[u])), T.rv[u]));
                sA[buf][lr][cl] = fmul(__fmul_rn(xhat, T.gv[u]));
                sB[buf][lr][cl] = T.gv[u];
            } else {
                sA[buf][lr][cl] = T.xv[u];
            }
        }
    };

    float acc = 0.f;
    const int chain = warp - kProducerWarps;          // consumer warps: 0 sums sA into out0, 1 sums sB into out1
    Tile cur, nxt;
    if (warp < kProducerWarps && ntiles > 0) {
        load(0, cur);
        if (ntiles > 1) load(1, nxt);
        finish(0, cur);
    }
    __syncthreads();
    for (int64_t t = 0; t < ntiles; ++t) {
        if (warp < kProducerWarps) {
            if (t + 1 < ntiles) {
                cur = nxt;
                if (t + 2 < ntiles) load(t + 2, nxt);
                finish(t + 1, cur);
            }
        } else {
            const int buf = (int)(t & 1);
            const float (*src)[kColTile] = (MODE == 0 && chain == 1) ? sB[buf] : sA[buf];
            const int64_t left = g.rows - t * kRowTile;
            const int nrows = left < kRowTile ? (int)left : kRowTile;
            int r = 0;
            for (; r + 32 <= nrows; r += 32) {
                float v[32];
#pragma unroll
                for (int u = 0; u < 32; ++u) v[u] = src[r + u][cl];
                acc = seq.add(acc, v);
            }
            for (; r + 8 <= nrows; r += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = src[r + u][cl];
                acc = seq.add(acc, v);
            }
            for (; r < nrows; ++r) {
                const float v[1] = {src[r][cl]};
                acc = seq.add(acc, v);
            }
        }
        __syncthreads();
    }
    if (warp >= kProducerWarps && lane < kColTile && col_ok) (chain == 0 ? out0 : out1)[col] = acc;
}

int check_geom(const char* who, int64_t outer, int channel, int64_t inner) {
    MPT_REQUIRE(outer >= 0 && channel >= 0 && inner >= 0, "%s: negative extent", who);
    return MPT_OK;
}

}  // namespace
}  // namespace mpt

using namespace mpt;

namespace {

mpt_format float_desc(int man, int exp, int sub, int sat) {
    mpt_format f{};
    f.kind = MPT_FMT_FLOAT; f.man = man; f.exp = exp; f.subnormals = sub; f.saturate = sat;
    return f;
}

}  // namespace

extern "C" {

int mpt_softmax_forward_fmt(const float* in, float* out, int64_t outer, int channel, int64_t inner, const mpt_format* fexp,
                            const mpt_format* foff, const mpt_format* facc, int order, void* stream) {
    int rc = check_geom("softmax_forward", outer, channel, inner);
    if (rc) return rc;
    AnyFmt e, o, a;
    if (!convert_format("softmax_forward", fexp, &e) || !convert_format("softmax_forward", foff, &o) ||
        !convert_format("softmax_forward", facc, &a)) return MPT_ERR_INVALID_ARGUMENT;
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "softmax_forward: null pointer");
    const Caster fe = Caster::make(e), fo = Caster::make(o), fa = Caster::make(a);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree && rows_shape_ok(g, 2048) && fe.use_fast && fo.use_fast && fa.use_fast) {
        // trusted: exp(.) <= 1 must be inside the exp format's fast range
        // and x - max in (-128, 0] inside the offset format's
        const int trusted = rows_mode({&fe, &fo, &fa}, fast_rn_exp_limit(fe.any.fp) >= 0 && fast_rn_exp_limit(fo.any.fp) >= 6);
        RowLimits lim{};
        lim.top[1] = top_of(fo); lim.top[2] = top_of(fa);
        launch_softmax_fwd_rows(in, out, g, fe, fo, fa, trusted, lim, stream);
        return check_launch("softmax_forward");
    }
    if (tree) softmax_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fe, fo, fa);
    else softmax_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fe, fo, fa);
    return check_launch("softmax_forward");
}

int mpt_softmax_lse_forward_fmt(const float* in, float* out, int64_t outer, int channel, int64_t inner, const mpt_format* foff,
                                const mpt_format* flse, int order, void* stream) {
    int rc = check_geom("softmax_lse_forward", outer, channel, inner);
    if (rc) return rc;
    AnyFmt o, l;
    if (!convert_format("softmax_lse_forward", foff, &o) || !convert_format("softmax_lse_forward", flse, &l)) return MPT_ERR_INVALID_ARGUMENT;
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "softmax_lse_forward: null pointer");
    const Caster fo = Caster::make(o), fl = Caster::make(l);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree && rows_shape_ok(g, 1024) && fo.use_fast && fl.use_fast) {
        // checked modes: x - max clamped to [-128, 0] and the running log-sum in [-128, log C] must lie inside the fast
        // range of their formats (below 256)
        const int mode = rows_mode({&fo, &fl}, fast_rn_exp_limit(fo.any.fp) >= 7 && fast_rn_exp_limit(fl.any.fp) >= 7);
        launch_softmax_lse_rows(in, out, g, fo, fl, mode, stream);
        return check_launch("softmax_lse_forward");
    }
    if (tree) softmax_lse_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fo, fl);
    else softmax_lse_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, out, g, fo, fl);
    return check_launch("softmax_lse_forward");
}

int mpt_softmax_backward_fmt(const float* y, const float* grad, float* out, int64_t outer, int channel, int64_t inner,
                             const mpt_format* fadd, const mpt_format* fmul, int order, void* stream) {
    int rc = check_geom("softmax_backward", outer, channel, inner);
    if (rc) return rc;
    AnyFmt a, m;
    if (!convert_format("softmax_backward", fadd, &a) || !convert_format("softmax_backward", fmul, &m)) return MPT_ERR_INVALID_ARGUMENT;
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0 || channel == 0) return MPT_OK;
    MPT_REQUIRE(y && grad && out, "softmax_backward: null pointer");
    const Caster fa = Caster::make(a), fm = Caster::make(m);
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree && rows_shape_ok(g, 1024) && fa.use_fast && fm.use_fast) {
        const int trusted = rows_mode({&fa, &fm}, true);
        RowLimits lim{};
        lim.top[0] = top_of(fa); lim.top[1] = top_of(fm);
        lim.growth = (float)(pow(step_growth(fa), channel / 64 + 6) * 1.001);
        const double sg = step_growth(fa) > step_growth(fm) ? step_growth(fa) : step_growth(fm);
        lim.slack = (float)(sg * sg * 1.001);
        launch_softmax_bwd_rows(y, grad, out, g, fa, fm, trusted, lim, stream);
        return check_launch("softmax_backward");
    }
    if (tree) softmax_bwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(y, grad, out, g, fa, fm);
    else softmax_bwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(y, grad, out, g, fa, fm);
    return check_launch("softmax_backward");
}

int mpt_layernorm_forward_fmt(const float* in, const float* weight, const float* bias, float* out, float* mean, float* rstd,
                              float eps, int64_t outer, int channel, int64_t inner, const mpt_format* facc,
                              const mpt_format* fmul, const mpt_format* fdiv, const mpt_format* fsqrt, int order, void* stream) {
    int rc = check_geom("layernorm_forward", outer, channel, inner);
    if (rc) return rc;
    AnyFmt a, m, d, q;
    if (!convert_format("layernorm_forward", facc, &a) || !convert_format("layernorm_forward", fmul, &m) ||
        !convert_format("layernorm_forward", fdiv, &d) || !convert_format("layernorm_forward", fsqrt, &q)) return MPT_ERR_INVALID_ARGUMENT;
    const RowGeom g{outer * inner, channel, inner};
    if (g.rows == 0) return MPT_OK;
    MPT_REQUIRE(channel > 0, "layernorm_forward: empty normalised shape");
    MPT_REQUIRE(in && weight && bias && out && mean && rstd, "layernorm_forward: null pointer");
    const LnFmt f{Caster::make(a), Caster::make(m), Caster::make(d), Caster::make(q), SeqAdder::make(a)};
    const bool tree = order != MPT_ORDER_SEQ;
    if (tree && rows_shape_ok(g, 2048) && f.acc.use_fast && f.mul.use_fast && f.div.use_fast) {
        const int trusted = rows_mode({&f.acc, &f.mul, &f.div}, true);
        const RowLimits lim = ln_limits(f, channel);
        launch_layernorm_fwd_rows(in, weight, bias, out, mean, rstd, eps, g, f, trusted, lim, stream);
        return check_launch("layernorm_forward");
    }
    if (tree) layernorm_fwd_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, weight, bias, out, mean, rstd, eps, g, f);
    else layernorm_fwd_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, weight, bias, out, mean, rstd, eps, g, f);
    return check_launch("layernorm_forward");
}

int mpt_layernorm_backward_fmt(const float* in, const float* grad_out, const float* weight, const float* mean, const float* rstd,
                               float* grad_in, float* grad_gamma, float* grad_beta, int64_t outer, int channel, int64_t inner,
                               const mpt_format* facc, const mpt_format* fmul, const mpt_format* fdiv, int order, void* stream) {
    int rc = check_geom("layernorm_backward", outer, channel, inner);
    if (rc) return rc;
    AnyFmt a, m, d;
    if (!convert_format("layernorm_backward", facc, &a) || !convert_format("layernorm_backward", fmul, &m) ||
        !convert_format("layernorm_backward", fdiv, &d)) return MPT_ERR_INVALID_ARGUMENT;
    const RowGeom g{outer * inner, channel, inner};
    if (channel == 0) return MPT_OK;
    MPT_REQUIRE(grad_gamma && grad_beta, "layernorm_backward: null pointer");
    const Caster cm = Caster::make(m);
    const LnFmt f{Caster::make(a), cm, Caster::make(d), cm, SeqAdder::make(a)};
    if (g.rows > 0) {
        MPT_REQUIRE(in && grad_out && weight && mean && rstd && grad_in, "layernorm_backward: null pointer");
        const bool tree = order != MPT_ORDER_SEQ;
        if (tree && rows_shape_ok(g, 1024) && f.acc.use_fast && f.mul.use_fast) {
            const int trusted = rows_mode({&f.acc, &f.mul}, true);
            const RowLimits lim = ln_limits(f, channel);
            launch_layernorm_bwd_rows(in, grad_out, weight, mean, rstd, grad_in, g, f, trusted, lim, stream);
        } else
        if (tree) layernorm_bwd_dx_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        else layernorm_bwd_dx_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        rc = check_launch("layernorm_backward (input gradient)");
        if (rc) return rc;
    }
    colsum_kernel<0><<<(channel + kColTile - 1) / kColTile, kColsumThreads(0), 0, as_stream(stream)>>>(in, grad_out, mean, rstd, grad_gamma, grad_beta, g,
                                                                                               f.acc, f.mul, f.seq);
    return check_launch("layernorm_backward (parameter gradients)");
}

int mpt_float_softmax_forward(const float* in, float* out, int64_t outer, int channel, int64_t inner, int man_exp,
                              int exp_exp, int man_off, int exp_off, int man_acc, int exp_acc, int subnormals,
                              int saturate, int order, void* stream) {
    const mpt_format e = float_desc(man_exp, exp_exp, subnormals, saturate), o = float_desc(man_off, exp_off, subnormals, saturate),
                     a = float_desc(man_acc, exp_acc, subnormals, saturate);
    return mpt_softmax_forward_fmt(in, out, outer, channel, inner, &e, &o, &a, order, stream);
}

int mpt_float_softmax_lse_forward(const float* in, float* out, int64_t outer, int channel, int64_t inner, int man_off,
                                  int exp_off, int man_lse, int exp_lse, int subnormals, int saturate, int order,
                                  void* stream) {
    const mpt_format o = float_desc(man_off, exp_off, subnormals, saturate), l = float_desc(man_lse, exp_lse, subnormals, saturate);
    return mpt_softmax_lse_forward_fmt(in, out, outer, channel, inner, &o, &l, order, stream);
}

int mpt_float_softmax_backward(const float* y, const float* grad, float* out, int64_t outer, int channel, int64_t inner,
                               int man_add, int exp_add, int man_mul, int exp_mul, int subnormals, int saturate,
                               int order, void* stream) {
    const mpt_format a = float_desc(man_add, exp_add, subnormals, saturate), m = float_desc(man_mul, exp_mul, subnormals, saturate);
    return mpt_softmax_backward_fmt(y, grad, out, outer, channel, inner, &a, &m, order, stream);
}

int mpt_float_layernorm_forward(const float* in, const float* weight, const float* bias, float* out, float* mean,
                                float* rstd, float eps, int64_t outer, int channel, int64_t inner, int man_acc,
                                int exp_acc, int man_mul, int exp_mul, int man_div, int exp_div, int man_sqrt,
                                int exp_sqrt, int subnormals, int saturate, int order, void* stream) {
    const mpt_format a = float_desc(man_acc, exp_acc, subnormals, saturate), m = float_desc(man_mul, exp_mul, subnormals, saturate),
                     d = float_desc(man_div, exp_div, subnormals, saturate), q = float_desc(man_sqrt, exp_sqrt, subnormals, saturate);
    return mpt_layernorm_forward_fmt(in, weight, bias, out, mean, rstd, eps, outer, channel, inner, &a, &m, &d, &q, order, stream);
}

int mpt_float_layernorm_backward(const float* in, const float* grad_out, const float* weight, const float* mean,
                                 const float* rstd, float* grad_in, float* grad_gamma, float* grad_beta, int64_t outer,
                                 int channel, int64_t inner, int man_acc, int exp_acc, int man_mul, int exp_mul,
                                 int man_div, int exp_div, int subnormals, int saturate, int order, void* stream) {
    const mpt_format a = float_desc(man_acc, exp_acc, subnormals, saturate), m = float_desc(man_mul, exp_mul, subnormals, saturate),
                     d = float_desc(man_div, exp_div, subnormals, saturate);
    return mpt_layernorm_backward_fmt(in, grad_out, weight, mean, rstd, grad_in, grad_gamma, grad_beta, outer, channel, inner, &a, &m, &d,
                                      order, stream);
}

int mpt_qsum_rows(const float* in, float* out, int64_t rows, int64_t cols, int man, int exp, int subnormals, int saturate,
                  void* stream) {
    MPT_REQUIRE(rows >= 0 && cols >= 0, "qsum_rows: negative extent");
    MPT_REQUIRE(valid_format(man, exp), "qsum_rows: unsupported format");
    if (cols == 0) return MPT_OK;
    MPT_REQUIRE(out && (rows == 0 || in), "qsum_rows: null pointer");
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    MPT_REQUIRE(cols <= 0x7FFFFFFF, "qsum_rows: too many columns");
    const RowGeom g{rows, (int)cols, 1};      // a [rows, cols] matrix: outer = rows, channel = cols, inner = 1
    colsum_kernel<1><<<(unsigned)((cols + kColTile - 1) / kColTile), kColsumThreads(1), 0, as_stream(stream)>>>(in, nullptr, nullptr, nullptr, out, nullptr, g,
                                                                                                        Caster::make(f), Caster::make(f), SeqAdder::make(f));
    return check_launch("qsum_rows");
}

}
