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
// the qsum loop (functional.py:736-748).  The chain per column is serial by definition: its time is (rows) x
// (latency of one dependent rounded add, five back-to-back instructions), so everything that does not depend on the
// running sum is taken off the warps that walk the chains.  A CTA owns 32 columns (lane = column).  Six producer
// warps stream row groups (8 rows x 32 columns, coalesced 128-byte row segments), do the per-element arithmetic
// (for layernorm: x-hat * dy, recomputed from the inputs instead of staged through the reference's scratch tensor,
// fp_kernel.cu:481-487), park the addends in shared memory and record, per group and column, the largest addend and
// whether a tiny one occurred: what the consumer needs to decide, with one compare per group, whether the group may
// take the FP-pipe rounding.  One consumer warp per chain (two for layernorm: x-hat * dy and dy) carries its 32 columns
// and executes, per row, one shared-memory load and the five dependent instructions (measured: about 56 cycles per row,
// which is the floor of this formulation; two chains interleaved in one warp take 75).
// Tiles of 128 rows are double buffered with one barrier per tile.
constexpr int kChainCols = 32;        // columns per CTA
constexpr int kChainGroup = 8;        // rows per range check
constexpr int kChainTile = 128;       // rows per tile
constexpr int kChainProducers = 6;
constexpr int chain_threads(int mode) { return (kChainProducers + (mode == 0 ? 2 : 1)) * 32; }
constexpr int kChainGroups = kChainTile / kChainGroup;
constexpr size_t chain_smem_bytes(int mode) {
    return (size_t)(mode == 0 ? 2 : 1) * 2 * (kChainTile + kChainGroups) * kChainCols * sizeof(float);
}

// |v| of a group folded into one float: the maximum, negated when some addend is nonzero and below 2^-101 (formats with
// an 8-bit exponent round such values in their own way, see FullRn).
__device__ __forceinline__ void group_note(float v, float& vmax, bool& tiny) {
    vmax = fmaxf(vmax, fabsf(v));
    tiny |= (__float_as_uint(v) & 0x7FFFFFFFu) - 1u < 0x0CFFFFFFu;
}

// MODE 0: layernorm parameter gradients (two chains: x-hat*dy -> out0, dy -> out1).  MODE 1: plain column sum of `in`.
// LINE: both formats of the per-element arithmetic round on the FP pipe and have fewer than 8 exponent bits, so the
// producers use the branch-free rounding and the eight elements of a group interleave.
template <int MODE, bool LINE>
__global__ void __launch_bounds__(chain_threads(MODE)) colsum_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                               const float* __restrict__ mean, const float* __restrict__ rstd,
                                                               float* __restrict__ out0, float* __restrict__ out1, RowGeom g,
                                                               Caster facc, Caster fmul, SeqAdder seq) {
    extern __shared__ __align__(16) float chain_smem[];
    // layout: addends A [2][tile][32], group notes A [2][groups][32], then the same for B (MODE 0)
    float* sA = chain_smem;
    float* nA = sA + 2 * kChainTile * kChainCols;
    float* sB = nA + 2 * kChainGroups * kChainCols;
    float* nB = sB + 2 * kChainTile * kChainCols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * kChainCols + lane;
    const bool col_ok = col < g.channel;
    const int64_t st = g.inner;
    const int64_t ntiles = (g.rows + kChainTile - 1) / kChainTile;

    // Producer warp w fills groups w, w + 7, ... of a tile.  All loads of a group are issued before its arithmetic.
    auto produce = [&](int64_t t) {
        const int buf = (int)(t & 1);
        for (int gi = warp; gi < kChainGroups; gi += kChainProducers) {
            const int64_t r0 = t * kChainTile + gi * kChainGroup;
            if (r0 >= g.rows) break;
            float xv[kChainGroup], gv[kChainGroup], mv[kChainGroup], rv[kChainGroup];
#pragma unroll
            for (int u = 0; u < kChainGroup; ++u) {
                const int64_t row = r0 + u;
                const bool rok = row < g.rows, ok = rok && col_ok;
                const int64_t idx = ok ? row_base(g, row) + col * st : 0;
                xv[u] = ok ? in[idx] : 0.f;
                if (MODE == 0) { gv[u] = ok ? gout[idx] : 0.f; mv[u] = rok ? mean[row] : 0.f; rv[u] = rok ? rstd[row] : 0.f; }
            }
            float ma = 0.f, mb = 0.f;
            bool ta = false, tb = false;
#pragma unroll
            for (int u = 0; u < kChainGroup; ++u) {
                const int lr = gi * kChainGroup + u;
                float a = xv[u];
                if (MODE == 0) {
                    if (LINE) {
                        const float xhat = fmul.fast.line(__fmul_rn(facc.fast.line(__fsub_rn(xv[u], mv[u])), rv[u]));
                        a = fmul.fast.line(__fmul_rn(xhat, gv[u]));
                    } else {
                        const float xhat = fmul(__fmul_rn(facc(__fsub_rn(xv[u], mv[u])), rv[u]));
                        a = fmul(__fmul_rn(xhat, gv[u]));
                    }
                    sB[(buf * kChainTile + lr) * kChainCols + lane] = gv[u];
                    group_note(gv[u], mb, tb);
                }
                sA[(buf * kChainTile + lr) * kChainCols + lane] = a;
                group_note(a, ma, ta);
            }
            nA[(buf * kChainGroups + gi) * kChainCols + lane] = ta ? -ma : ma;
            if (MODE == 0) nB[(buf * kChainGroups + gi) * kChainCols + lane] = tb ? -mb : mb;
        }
    };

    // consumer warp `chain` (0: addends A into out0, 1: addends B into out1)
    const int chain = warp - kChainProducers;
    float acc = 0.f;
    if (warp < kChainProducers && ntiles > 0) produce(0);
    __syncthreads();
    for (int64_t t = 0; t < ntiles; ++t) {
        if (warp < kChainProducers) {
            if (t + 1 < ntiles) produce(t + 1);
        } else {
            const int buf = (int)(t & 1);
            const int64_t left = g.rows - t * kChainTile;
            const int nrows = left < kChainTile ? (int)left : kChainTile;
            const float* a = (chain == 0 ? sA : sB) + (size_t)buf * kChainTile * kChainCols + lane;
            const float* notes = (chain == 0 ? nA : nB) + (size_t)buf * kChainGroups * kChainCols + lane;
            int gi = 0;
            for (; (gi + 1) * kChainGroup <= nrows; ++gi) {
                float va[kChainGroup];
#pragma unroll
                for (int u = 0; u < kChainGroup; ++u) va[u] = a[(gi * kChainGroup + u) * kChainCols];
                acc = seq.add_noted(acc, va, notes[gi * kChainCols]);
            }
            for (int r = gi * kChainGroup; r < nrows; ++r) {
                const float v[1] = {a[r * kChainCols]};
                acc = seq.add(acc, v);
            }
        }
        __syncthreads();
    }
    if (warp >= kChainProducers && col_ok) (chain == 0 ? out0 : out1)[col] = acc;
}

template <int MODE>
int launch_colsum(const float* in, const float* gout, const float* mean, const float* rstd, float* out0, float* out1, const RowGeom& g,
                  const Caster& facc, const Caster& fmul, const SeqAdder& seq, cudaStream_t st, const char* who) {
    const size_t smem = chain_smem_bytes(MODE);
    const bool line = MODE == 0 && facc.use_fast && fmul.use_fast && facc.any.fp.exp < 8 && fmul.any.fp.exp < 8;
    auto kern = line ? colsum_kernel<MODE, true> : colsum_kernel<MODE, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("%s: cudaFuncSetAttribute: %s", who, cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    kern<<<(unsigned)((g.channel + kChainCols - 1) / kChainCols), chain_threads(MODE), smem, st>>>(in, gout, mean, rstd, out0, out1, g, facc, fmul, seq);
    return check_launch(who);
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
    // trusted: exp(.) <= 1 must be inside the exp format's fast range
    // and x - max in (-128, 0] inside the offset format's
    const int trusted = (tree && rows_shape_ok(g, 2048))
                            ? rows_path({&fe, &fo, &fa}, fast_rn_exp_limit(fe.any.fp) >= 0 && fast_rn_exp_limit(fo.any.fp) >= 6) : -1;
    if (trusted >= 0) {
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
    const int trusted = (tree && rows_shape_ok(g, 1024)) ? rows_path({&fa, &fm}, true) : -1;
    if (trusted >= 0) {
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
    const int trusted = (tree && rows_shape_ok(g, 2048)) ? rows_path({&f.acc, &f.mul, &f.div}, true) : -1;
    if (trusted >= 0) {
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
        const int trusted = (tree && rows_shape_ok(g, 1024)) ? rows_path({&f.acc, &f.mul}, true) : -1;
        if (trusted >= 0) {
            const RowLimits lim = ln_limits(f, channel);
            launch_layernorm_bwd_rows(in, grad_out, weight, mean, rstd, grad_in, g, f, trusted, lim, stream);
        } else
        if (tree) layernorm_bwd_dx_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        else layernorm_bwd_dx_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        rc = check_launch("layernorm_backward (input gradient)");
        if (rc) return rc;
    }
    return launch_colsum<0>(in, grad_out, mean, rstd, grad_gamma, grad_beta, g, f.acc, f.mul, f.seq, as_stream(stream),
                            "layernorm_backward (parameter gradients)");
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
    return launch_colsum<1>(in, nullptr, nullptr, nullptr, out, nullptr, g, Caster::make(f), Caster::make(f), SeqAdder::make(f),
                            as_stream(stream), "qsum_rows");
}

}
