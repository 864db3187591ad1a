// Shared by reduce.cu (general kernels, C entry points) and the rows_*.cu files (register-resident row kernels):
// row geometry, the 64-partial shuffle tree, the rounding functors, the whole-domain per-row code of softmax and
// layer normalisation, and the host-side selection of the register-resident kernels.
#pragma once
#include <cmath>
#include <initializer_list>

#include "cast.cuh"
#include "common.cuh"

namespace mpt {


constexpr int kWarpsPerBlock = 8;

struct RowGeom {
    int64_t rows;      // outer * inner
    int channel;
    int64_t inner;
};

__device__ __forceinline__ int64_t row_base(const RowGeom& g, int64_t row) {
    if (g.inner == 1) return row * (int64_t)g.channel;       // contiguous rows: no 64-bit division
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

// Nearest rounding to one format.  Formats the FP-pipe rounding supports (subnormals on, man <= 21) take
// FullRn, which equals the exact caster on every input at about a third of the instructions; the rest
// take the exact caster.  The choice is uniform across the launch.
struct Caster {
    FullRn fast;
    AnyFmt any;
    int use_fast;
    int nosub_fast;        // a float format without subnormals that the settling FP-pipe rounding (fast_rn_nosub) covers
    uint32_t neg_zero;     // what -0 rounds to: -0 in 8-bit-exponent formats, +0 in the others (as the reference does)
    __host__ static Caster make(const AnyFmt& a) {
        Caster c;
        c.any = a;
        c.neg_zero = (a.kind == FMT_FLOAT && a.fp.exp == 8) ? 0x80000000u : 0u;
        c.fast = FullRn::make(a.fp);
        c.use_fast = (a.kind == FMT_FLOAT && fast_rn_supported(a.fp)) ? 1 : 0;
        c.nosub_fast = (a.kind == FMT_FLOAT && !a.fp.sub && a.fp.man <= 21 && a.fp.exp >= 2) ? 1 : 0;
        return c;
    }
    __host__ static Caster make(const FpFmt& f) { return make(any_float(f)); }
    __device__ __forceinline__ float operator()(float x) const { return use_fast ? fast(x) : cast_any(x, any); }
};
__device__ __forceinline__ float cast_fp_nearest(float x, const Caster& c) { return c(x); }

struct QAdd {
    Caster f;
    __device__ __forceinline__ float operator()(float a, float b) const { return f(__fadd_rn(a, b)); }
};

// U sequential rounded additions acc = Q(acc + v[u]).  When the running sum provably stays inside the
// range where the 4-instruction FP-pipe rounding is exact, the chain uses it (a dependent step is then
// about 20 cycles instead of about 150), otherwise the exact caster.  The bound: acc is a value of the format,
// so rounding acc + v moves the sum by at most |v| (acc itself is a candidate), and every intermediate stays
// below |acc| + 2 * sum |v|.
struct SeqAdder {
    Caster q;
    FastRn r;
    float top;        // 2^(limit exponent + 1): every intermediate |sum| must stay below
    int chain_ok;     // format supports the fast chain
    int exp8;         // 8-bit exponent: tiny values need the exact caster (see FullRn)
    __host__ static SeqAdder make(const AnyFmt& a) {
        SeqAdder s = make(a.fp);
        s.q = Caster::make(a);
        if (a.kind != FMT_FLOAT) s.chain_ok = 0;
        return s;
    }
    __host__ static SeqAdder make(const FpFmt& f) {
        SeqAdder s;
        s.q = Caster::make(f);
        s.r = FastRn::make(f);
        s.top = ldexpf(1.0f, fast_rn_exp_limit(f) + 1);
        s.chain_ok = fast_rn_supported(f) ? 1 : 0;
        s.exp8 = f.exp == 8;
        return s;
    }
    template <int U>
    __device__ __forceinline__ float add(float acc, const float (&v)[U]) const {
        float vmax = 0.f;
        bool tiny = false;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            vmax = fmaxf(vmax, fabsf(v[u]));
            tiny |= (__float_as_uint(v[u]) & 0x7FFFFFFFu) - 1u < 0x0CFFFFFFu;     // 0 < |v| < 2^-101
        }
        tiny |= (__float_as_uint(acc) & 0x7FFFFFFFu) - 1u < 0x0CFFFFFFu;
        const bool fast = chain_ok && (fabsf(acc) + (float)(2 * U) * vmax) * 1.0001f < top && !(exp8 && tiny);
        if (fast) {
#pragma unroll
            for (int u = 0; u < U; ++u) acc = r(__fadd_rn(acc, v[u]));
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) acc = q(__fadd_rn(acc, v[u]));
        }
        return acc;
    }
    // The same with the group's largest |v| and its "tiny value present" flag precomputed (`note`: the maximum, negated
    // when the flag is set), so that the warp walking the chain spends one compare per group on the decision.
    __device__ __forceinline__ bool noted_fast(float acc, float note, int U) const {
        const bool tiny = note < 0.f || (__float_as_uint(acc) & 0x7FFFFFFFu) - 1u < 0x0CFFFFFFu;
        return chain_ok && (fabsf(acc) + (float)(2 * U) * fabsf(note)) * 1.0001f < top && !(exp8 && tiny);
    }
    template <int U>
    __device__ __forceinline__ float add_noted(float acc, const float (&v)[U], float note) const {
        if (noted_fast(acc, note, U)) {
#pragma unroll
            for (int u = 0; u < U; ++u) acc = r(__fadd_rn(acc, v[u]));
        } else {
#pragma unroll 1
            for (int u = 0; u < U; ++u) acc = q(__fadd_rn(acc, v[u]));
        }
        return acc;
    }
};
struct FMax {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};
struct QLse {
    Caster f;
    __device__ __forceinline__ float operator()(float a, float b) const { return f(logf(__fadd_rn(expf(a), expf(b)))); }
};

// Log-sum-exp form of the softmax forward, one row in the CUDA association, whole input domain.
__device__ __forceinline__ void softmax_lse_row_tree(const float* x, float* y, int C, int64_t st, int lane, const Caster& foff,
                                                     const Caster& flse) {
    const QLse qlse{flse};
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
}

// One row in the CUDA association, whole input domain; called by all 32 lanes of the warp that owns the row.
__device__ __forceinline__ void softmax_fwd_row_tree(const float* x, float* y, int C, int64_t st, int lane, const Caster& fexp,
                                                     const Caster& foff, const Caster& facc) {
    const QAdd qadd{facc};
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
}

__device__ __forceinline__ void softmax_bwd_row_tree(const float* y, const float* gr, float* o, int C, int64_t st, int lane,
                                                     const Caster& fadd, const Caster& fmul) {
    const QAdd qadd{fadd};
    float s0 = 0.f, s1 = 0.f;
    for (int k = lane; k < C; k += 64) {
        s0 = qadd(s0, cast_fp_nearest(__fmul_rn(y[k * st], gr[k * st]), fmul));
        if (k + 32 < C) s1 = qadd(s1, cast_fp_nearest(__fmul_rn(y[(k + 32) * st], gr[(k + 32) * st]), fmul));
    }
    const float s = tree64(s0, s1, qadd);
    for (int k = lane; k < C; k += 32) o[k * st] = __fmul_rn(cast_fp_nearest(__fsub_rn(gr[k * st], s), fadd), y[k * st]);
}

struct LnFmt { Caster acc, mul, div, sqrt; SeqAdder seq; };

// One row (whole input domain): all 32 lanes of the owning warp in the CUDA association (lane, step = 32), or a single
// thread in the sequential one (lane = 0, step = 1).
template <bool TREE>
__device__ __forceinline__ void layernorm_fwd_row(const float* x, const float* w, const float* bias, float* y, float* mean, float* rstd,
                                                  int64_t row, float eps, int C, int64_t st, int lane, int step, const LnFmt& f) {
    const QAdd qacc{f.acc};
    const float fC = (float)C;
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

// Input gradient of one row; lanes as in layernorm_fwd_row.
template <bool TREE>
__device__ __forceinline__ void layernorm_bwd_row(const float* x, const float* gr, const float* w, float m, float r, float* o, int C,
                                                  int64_t st, int lane, int step, const LnFmt& f) {
    const QAdd qacc{f.acc};
    const float fC = (float)C;
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

// ------------------------------------------------------------------- register-resident row kernels
// Contiguous rows (inner == 1) of 32 * JMAX elements (JMAX even, a fixed list of instantiations), in the CUDA
// association, with every format one the FP-pipe rounding supports.  One warp owns a row and keeps it in
// registers: lane l holds elements l + 32 j, so element j of a lane belongs to partial l (j even) or
// l + 32 (j odd) exactly as in the kernels above, every element is read from memory once, and the unrolled
// loops carry no index arithmetic.
//
// The checked modes (MODE 1 and 2, `TRUSTED` in the kernels) replace every rounding by the bare 4-instruction FP-pipe form and the
// per-element IEEE division by a multiply and two FMAs with the row's correctly rounded reciprocal
// (Markstein's correction step, which returns the correctly rounded quotient).  Both are exact only while
// every intermediate is finite and inside the range of its format, so the warp bounds all of them from the
// maxima of its inputs (tracked with one FMNMX per element) BEFORE anything is stored; a row that fails the
// bound, or contains NaN or infinity, is handed to the whole-domain code path above (`*_row_tree`).
// The host picks the mode from the formats.
// MODE 0: whole-domain rounding, no range checks.  MODE 1: bare FP-pipe rounding (every format has fewer than 8
// exponent bits).  MODE 2: bare FP-pipe rounding for any mix of formats; 8-bit-exponent formats keep -0 (patched in
// with a select) and round fp32-denormal inputs in their own way, so every rounding also records, branch-free,
// whether it saw a nonzero denormal, and a row that did is handed to the whole-domain fallback like a row that
// fails its range check.
// MODE 3: formats without subnormals.  The FP-pipe rounding runs without its exponent clamp and what lands below the
// smallest normal value is settled as the reference does (fast_rn_nosub); like MODE 2 it is exact for zero and normal
// fp32 inputs only, so every rounding records a nonzero denormal input and the row falls back.
template <int MODE>
__device__ __forceinline__ float rr(const Caster& c, float x, bool& odd) {
    if (MODE == 0) return c.fast(x);
    if (MODE == 3) {
        const uint32_t t = __float_as_uint(x);
        odd |= (t + t - 1u < 0x00FFFFFFu);
        return fast_rn_nosub(c.fast.fast, x);
    }
    if (MODE == 2) {
        // t + t drops the sign bit, so one three-input add and one compare find a nonzero fp32 denormal.  A zero result
        // can only come from a zero input here (8-bit-exponent formats have subnormals below every fp32 normal, and
        // denormal inputs leave this path), so OR-ing the input's sign in, where the format keeps it, restores -0.
        const uint32_t t = __float_as_uint(x);
        odd |= (t + t - 1u < 0x00FFFFFFu);
        const float r = c.fast.fast(x);
        return __uint_as_float(__float_as_uint(r) | (t & c.neg_zero));
    }
    return c.fast.fast(x);
}

// Two roundings at once for the checked modes: the exponent extraction and clamp stay per value, the two FMAs of the
// FP-pipe rounding become one packed fp32x2 instruction each.  Same operations per value as rr<MODE>.
template <int MODE>
__device__ __forceinline__ float2 rr2(const Caster& c, float2 x, bool& odd) {
    if (MODE == 0) return make_float2(c.fast(x.x), c.fast(x.y));
    if (MODE == 3) return make_float2(rr<3>(c, x.x, odd), rr<3>(c, x.y, odd));
    const FastRn& r = c.fast.fast;
    const uint32_t t0 = __float_as_uint(x.x), t1 = __float_as_uint(x.y);
    const int e0 = (int)(t0 & 0x7F800000u), e1 = (int)(t1 & 0x7F800000u);
    const float2 m = make_float2(__int_as_float(e0 > r.min_e_bits ? e0 : r.min_e_bits), __int_as_float(e1 > r.min_e_bits ? e1 : r.min_e_bits));
    const float2 y = __ffma2_rn(m, make_float2(r.k, r.k), x);
    float2 z = __ffma2_rn(m, make_float2(-r.k, -r.k), y);
    if (MODE == 2) {
        odd |= (t0 + t0 - 1u < 0x00FFFFFFu) | (t1 + t1 - 1u < 0x00FFFFFFu);
        z.x = __uint_as_float(__float_as_uint(z.x) | (t0 & c.neg_zero));
        z.y = __uint_as_float(__float_as_uint(z.y) | (t1 & c.neg_zero));
    }
    return z;
}

// a / b for two dividends, given r = RN(1 / b) (see row_div).
template <int MODE>
__device__ __forceinline__ float2 row_div2(float2 a, float b, float r, bool& odd) {
    if (MODE >= 2) {
        const uint32_t t0 = __float_as_uint(a.x), t1 = __float_as_uint(a.y);
        odd |= (t0 + t0 - 1u < 0x2BFFFFFEu) | (t1 + t1 - 1u < 0x2BFFFFFEu);
    }
    const float2 r2 = make_float2(r, r);
    const float2 q = __fmul2_rn(a, r2);
    const float2 rem = __ffma2_rn(make_float2(-b, -b), q, a);
    return __ffma2_rn(rem, r2, q);
}

template <int MODE>
struct RAdd {
    const Caster& c;
    bool& odd;
    __device__ __forceinline__ float operator()(float a, float b) const { return rr<MODE>(c, __fadd_rn(a, b), odd); }
};

// a / b given r = RN(1 / b), for the checked modes.  MODE 2 records dividends too small for the remainder to stay a
// normal number (0 < |a| < 2^-83); MODE 1 cannot meet one (its dividends are rounded to formats whose smallest
// subnormal is larger).
template <int MODE>
__device__ __forceinline__ float row_div(float a, float b, float r, bool& odd) {
    if (MODE >= 2) { const uint32_t t = __float_as_uint(a); odd |= (t + t - 1u < 0x2BFFFFFEu); }
    return div_with_rcp(a, b, r);
}

// Warp-wide maximum of non-negative values in one instruction (their bit patterns order like unsigned integers; a
// NaN pattern orders above infinity and so survives, which is what the range checks want).
__device__ __forceinline__ float warp_max_nonneg(float v) {
    return __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(v)));
}
// Upper bound of the warp-wide sum of non-negative per-lane sums.
__device__ __forceinline__ float warp_sum_bound(float v) { return 32.0f * warp_max_nonneg(v); }

// Range limits of the trusted path, prepared by the host.
struct RowLimits {
    float top[4];     // per format slot: every |value| fed to that rounding must stay below this
    float growth;     // bound of (1 + 2^-(man_acc + 1))^(depth of the row sum), with slack
    float slack;      // bound of the relative growth of two successive roundings, with slack
};

// The whole-domain fallbacks are out-of-line calls; formats travel by pointer into the kernel's parameter space
// (the kernels declare them __grid_constant__), so the hot path sets up no copies for a call it rarely makes.
static __device__ __noinline__ void softmax_fwd_row_cold(const float* x, float* y, int C, int lane, const Caster* fexp, const Caster* foff,
                                                 const Caster* facc) {
    softmax_fwd_row_tree(x, y, C, 1, lane, *fexp, *foff, *facc);
}
static __device__ __noinline__ void softmax_lse_row_cold(const float* x, float* y, int C, int lane, const Caster* foff, const Caster* flse) {
    softmax_lse_row_tree(x, y, C, 1, lane, *foff, *flse);
}
static __device__ __noinline__ void softmax_bwd_row_cold(const float* y, const float* gr, float* o, int C, int lane, const Caster* fadd,
                                                 const Caster* fmul) {
    softmax_bwd_row_tree(y, gr, o, C, 1, lane, *fadd, *fmul);
}
static __device__ __noinline__ void layernorm_fwd_row_cold(const float* x, const float* w, const float* bias, float* y, float* mean, float* rstd,
                                                   int64_t row, float eps, int C, int lane, const LnFmt* f) {
    layernorm_fwd_row<true>(x, w, bias, y, mean, rstd, row, eps, C, 1, lane, 32, *f);
}
static __device__ __noinline__ void layernorm_bwd_row_cold(const float* x, const float* gr, const float* w, float m, float r, float* o, int C,
                                                   int lane, const LnFmt* f) {
    layernorm_bwd_row<true>(x, gr, w, m, r, o, C, 1, lane, 32, *f);
}

inline unsigned row_blocks(int64_t rows, bool tree) {
    const int64_t per = tree ? kWarpsPerBlock : kWarpsPerBlock * 32;
    return (unsigned)((rows + per - 1) / per);
}

// ---- host side of the register-resident row kernels
// Row lengths with an instantiation: 32 * {2, 4, 8, 12, 16, 24, 32, 48, 64}.
inline bool rows_shape_ok(const RowGeom& g, int max_channel) {
    if (g.inner != 1 || g.channel % 64 != 0 || g.channel > max_channel) return false;
    switch (g.channel / 32) {
        case 2: case 4: case 8: case 12: case 16: case 24: case 32: case 48: case 64: return true;
        default: return false;
    }
}
inline float top_of(const Caster& c) { return ldexpf(1.0f, fast_rn_exp_limit(c.any.fp) + 1); }
inline double step_growth(const Caster& c) { return 1.0 + ldexp(1.0, -(c.any.fp.man + 1)); }
inline bool small_exp(const Caster& c) { return c.use_fast && c.any.fp.exp < 8; }
// Mode of the register-resident kernels for a set of formats the FP-pipe rounding supports.
inline int rows_mode(std::initializer_list<const Caster*> cs, bool ranges_ok) {
    if (!ranges_ok) return 0;
    for (const Caster* c : cs)
        if (!small_exp(*c)) return 2;
    return 1;
}
// The same for any set of formats: -1 when the register-resident kernels do not apply (a format without either
// FP-pipe rounding, a mixture of formats with and without subnormals, or formats without subnormals whose static
// range conditions fail: they have no whole-domain form of the fast rounding to fall back on inside those kernels).
inline int rows_path(std::initializer_list<const Caster*> cs, bool ranges_ok) {
    bool all_sub = true, all_nosub = true;
    for (const Caster* c : cs) { all_sub = all_sub && c->use_fast; all_nosub = all_nosub && c->nosub_fast; }
    if (all_sub) return rows_mode(cs, ranges_ok);
    return (all_nosub && ranges_ok) ? 3 : -1;
}

inline RowLimits ln_limits(const LnFmt& f, int channel) {
    RowLimits lim{};
    lim.top[0] = top_of(f.acc); lim.top[1] = top_of(f.mul); lim.top[2] = top_of(f.div);
    lim.growth = (float)(pow(step_growth(f.acc), channel / 64 + 6) * 1.001);
    double sg = step_growth(f.acc);
    if (step_growth(f.mul) > sg) sg = step_growth(f.mul);
    if (step_growth(f.div) > sg) sg = step_growth(f.div);
    lim.slack = (float)(sg * sg * 1.001);
    return lim;
}

#define MPT_ROWS_CASE(KERNEL, J, ...)                                                                                       \
    case J:                                                                                                                 \
        if (mode_ == 1) KERNEL<J, 1><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                                 \
        else if (mode_ == 2) KERNEL<J, 2><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                            \
        else if (mode_ == 3) KERNEL<J, 3><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                            \
        else KERNEL<J, 0><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                                            \
        break;
#define MPT_ROWS_DISPATCH(KERNEL, TRUSTED, ...)                                                                             \
    do {                                                                                                                    \
        const int mode_ = (TRUSTED);                                                                                         \
        const unsigned grid_ = row_blocks(g.rows, true);                                                                    \
        const unsigned thr_ = kWarpsPerBlock * 32;                                                                          \
        cudaStream_t st_ = as_stream(stream);                                                                               \
        switch (g.channel / 32) {                                                                                           \
            MPT_ROWS_CASE(KERNEL, 2, __VA_ARGS__)                                                                           \
            MPT_ROWS_CASE(KERNEL, 4, __VA_ARGS__)                                                                           \
            MPT_ROWS_CASE(KERNEL, 8, __VA_ARGS__)                                                                           \
            MPT_ROWS_CASE(KERNEL, 12, __VA_ARGS__)                                                                          \
            MPT_ROWS_CASE(KERNEL, 16, __VA_ARGS__)                                                                          \
            MPT_ROWS_CASE(KERNEL, 24, __VA_ARGS__)                                                                          \
            MPT_ROWS_CASE(KERNEL, 32, __VA_ARGS__)                                                                          \
            default: break;                                                                                                 \
        }                                                                                                                   \
    } while (0)
// the single-array kernels also cover rows of 1536 and 2048
#define MPT_ROWS_DISPATCH_WIDE(KERNEL, TRUSTED, ...)                                                                        \
    do {                                                                                                                    \
        if (g.channel / 32 <= 32) { MPT_ROWS_DISPATCH(KERNEL, TRUSTED, __VA_ARGS__); break; }                               \
        const int mode_ = (TRUSTED);                                                                                         \
        const unsigned grid_ = row_blocks(g.rows, true);                                                                    \
        const unsigned thr_ = kWarpsPerBlock * 32;                                                                          \
        cudaStream_t st_ = as_stream(stream);                                                                               \
        switch (g.channel / 32) {                                                                                           \
            MPT_ROWS_CASE(KERNEL, 48, __VA_ARGS__)                                                                          \
            MPT_ROWS_CASE(KERNEL, 64, __VA_ARGS__)                                                                          \
            default: break;                                                                                                 \
        }                                                                                                                   \
    } while (0)

// Launchers of the register-resident kernels (rows_*.cu); the caller has checked rows_shape_ok and the formats.
void launch_softmax_fwd_rows(const float* in, float* out, const RowGeom& g, const Caster& fe, const Caster& fo, const Caster& fa,
                             int mode, const RowLimits& lim, void* stream);
void launch_softmax_lse_rows(const float* in, float* out, const RowGeom& g, const Caster& fo, const Caster& fl, int mode, void* stream);
void launch_softmax_bwd_rows(const float* y, const float* grad, float* out, const RowGeom& g, const Caster& fa, const Caster& fm,
                             int mode, const RowLimits& lim, void* stream);
void launch_layernorm_fwd_rows(const float* in, const float* weight, const float* bias, float* out, float* mean, float* rstd, float eps,
                               const RowGeom& g, const LnFmt& f, int mode, const RowLimits& lim, void* stream);
void launch_layernorm_bwd_rows(const float* in, const float* grad_out, const float* weight, const float* mean, const float* rstd,
                               float* grad_in, const RowGeom& g, const LnFmt& f, int mode, const RowLimits& lim, void* stream);

}  // namespace mpt
