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

// Nearest rounding to one format.  Formats the FP-pipe rounding supports (subnormals on, man <= 21) take
// FullRn, which equals the exact caster on every input at about a third of the instructions; the rest
// take the exact caster.  The choice is uniform across the launch.
struct Caster {
    FullRn fast;
    AnyFmt any;
    int use_fast;
    __host__ static Caster make(const AnyFmt& a) {
        Caster c;
        c.any = a;
        c.fast = FullRn::make(a.fp);
        c.use_fast = (a.kind == FMT_FLOAT && fast_rn_supported(a.fp)) ? 1 : 0;
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

// Eight sequential rounded additions acc = Q(acc + v[u]).  When the running sum provably stays inside the
// range where the 4-instruction FP-pipe rounding is exact, the chain uses it (a dependent step is then
// about 20 cycles instead of about 150), otherwise the exact caster.
struct SeqAdder {
    Caster q;
    FastRn r;
    float top;        // 2^(limit exponent + 1): every intermediate |sum| must stay below
    float growth8;    // bound of (1 + 2^-(man+1))^8
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
        double g = 1.0;
        for (int i = 0; i < 8; ++i) g *= 1.0 + ldexp(1.0, -(f.man + 1));
        s.growth8 = (float)(g * 1.0001);
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
        const bool fast = chain_ok && (fabsf(acc) + (float)U * vmax) * growth8 < top && !(exp8 && tiny);
        if (fast) {
#pragma unroll
            for (int u = 0; u < U; ++u) acc = r(__fadd_rn(acc, v[u]));
        } else {
#pragma unroll
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

// ----------------------------------------------------------------------------------------- softmax
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

// ------------------------------------------------------------------- register-resident row kernels
// Contiguous rows (inner == 1) whose length is a multiple of 64 and at most 32 * JMAX, in the CUDA
// association, with every format one the FP-pipe rounding supports.  One warp owns a row and keeps it in
// registers: lane l holds elements l + 32 j, so element j of a lane belongs to partial l (j even) or
// l + 32 (j odd) exactly as in the kernels above, every element is read from memory once, and the unrolled
// loops carry no index arithmetic.
//
// TRUSTED = true additionally replaces every rounding by the bare 4-instruction FP-pipe form and the
// per-element IEEE division by a multiply and two FMAs with the row's correctly rounded reciprocal
// (Markstein's correction step, which returns the correctly rounded quotient).  Both are exact only while
// every intermediate is finite and inside the range of its format, so the warp bounds all of them from the
// maxima of its inputs (tracked with one FMNMX per element) BEFORE anything is stored; a row that fails the
// bound, or contains NaN or infinity, is handed to the whole-domain code path above (`*_row_tree`).
// TRUSTED needs formats with fewer than 8 exponent bits (the reference rounds fp32-denormal inputs of
// 8-bit-exponent formats differently, which only the whole-domain rounding reproduces); the host picks it.
template <bool TRUSTED>
__device__ __forceinline__ float rr(const Caster& c, float x) { return TRUSTED ? c.fast.fast(x) : c.fast(x); }

template <bool TRUSTED>
struct RAdd {
    const Caster& c;
    __device__ __forceinline__ float operator()(float a, float b) const { return rr<TRUSTED>(c, __fadd_rn(a, b)); }
};
struct FMin {
    __device__ __forceinline__ float operator()(float a, float b) const { return fminf(a, b); }
};

// Range limits of the trusted path, prepared by the host.
struct RowLimits {
    float top[4];     // per format slot: every |value| fed to that rounding must stay below this
    float growth;     // bound of (1 + 2^-(man_acc + 1))^(depth of the row sum), with slack
    float slack;      // bound of the relative growth of two successive roundings, with slack
};

// The whole-domain fallbacks are out-of-line calls; formats travel by pointer into the kernel's parameter space
// (the kernels declare them __grid_constant__), so the hot path sets up no copies for a call it rarely makes.
__device__ __noinline__ void softmax_fwd_row_cold(const float* x, float* y, int C, int lane, const Caster* fexp, const Caster* foff,
                                                 const Caster* facc);
__device__ __noinline__ void softmax_bwd_row_cold(const float* y, const float* gr, float* o, int C, int lane, const Caster* fadd,
                                                 const Caster* fmul);
__device__ __noinline__ void layernorm_fwd_row_cold(const float* x, const float* w, const float* bias, float* y, float* mean, float* rstd,
                                                   int64_t row, float eps, int C, int lane, const LnFmt* f);
__device__ __noinline__ void layernorm_bwd_row_cold(const float* x, const float* gr, const float* w, float m, float r, float* o, int C,
                                                   int lane, const LnFmt* f);

template <int JMAX, bool TRUSTED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_fwd_rows_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                              int64_t rows, int C, const __grid_constant__ Caster fexp,
                                                                              const __grid_constant__ Caster foff,
                                                                              const __grid_constant__ Caster facc, RowLimits lim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    float* y = out + row * C;
    const int nj = C >> 5;
    float v[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        if (j < nj) v[j] = x[lane + 32 * j];
    float m0 = -INFINITY, m1 = -INFINITY, n0 = INFINITY, n1 = INFINITY;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2)
        if (j < nj) {
            m0 = fmaxf(m0, v[j]); m1 = fmaxf(m1, v[j + 1]);
            if (TRUSTED) { n0 = fminf(n0, v[j]); n1 = fminf(n1, v[j + 1]); }
        }
    const float mx = tree64(m0, m1, FMax{});
    bool ok = true;
    if (TRUSTED) ok = __fsub_rn(mx, tree64(n0, n1, FMin{})) < lim.top[1];     // false for NaN and infinite extremes
    if (ok) {
        const RAdd<TRUSTED> qadd{facc};
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < JMAX; j += 2)
            if (j < nj) {
                const float e0 = rr<TRUSTED>(fexp, expf(rr<TRUSTED>(foff, __fsub_rn(v[j], mx))));
                const float e1 = rr<TRUSTED>(fexp, expf(rr<TRUSTED>(foff, __fsub_rn(v[j + 1], mx))));
                v[j] = e0; v[j + 1] = e1;
                s0 = qadd(s0, e0); s1 = qadd(s1, e1);
            }
        const float sum = tree64(s0, s1, qadd);
        if (TRUSTED) {
            // the addends are non-negative, so the total bounds every partial sum; a NaN element ends up here as well
            ok = sum >= 1.0f && sum < lim.top[2] && sum <= 0x1p20f;
            if (ok) {
                const float r = __frcp_rn(sum);
#pragma unroll
                for (int j = 0; j < JMAX; ++j)
                    if (j < nj) y[lane + 32 * j] = div_with_rcp(v[j], sum, r);
                return;
            }
        } else {
#pragma unroll
            for (int j = 0; j < JMAX; ++j)
                if (j < nj) y[lane + 32 * j] = __fdiv_rn(v[j], sum);
            return;
        }
    }
    softmax_fwd_row_cold(x, y, C, lane, &fexp, &foff, &facc);
}

template <int JMAX, bool TRUSTED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_bwd_rows_kernel(const float* __restrict__ yv, const float* __restrict__ gv,
                                                                              float* __restrict__ out, int64_t rows, int C,
                                                                              const __grid_constant__ Caster fadd,
                                                                              const __grid_constant__ Caster fmul, RowLimits lim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* y = yv + row * C;
    const float* gr = gv + row * C;
    float* o = out + row * C;
    const int nj = C >> 5;
    float a[JMAX], b[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        if (j < nj) { a[j] = y[lane + 32 * j]; b[j] = gr[lane + 32 * j]; }
    const RAdd<TRUSTED> qadd{fadd};
    float s0 = 0.f, s1 = 0.f, pm = 0.f, gm = 0.f;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2)
        if (j < nj) {
            const float p0 = __fmul_rn(a[j], b[j]), p1 = __fmul_rn(a[j + 1], b[j + 1]);
            if (TRUSTED) {
                pm = fmaxf(pm, fmaxf(fabsf(p0), fabsf(p1)));
                gm = fmaxf(gm, fmaxf(fabsf(b[j]), fabsf(b[j + 1])));
            }
            s0 = qadd(s0, rr<TRUSTED>(fmul, p0));
            s1 = qadd(s1, rr<TRUSTED>(fmul, p1));
        }
    const float s = tree64(s0, s1, qadd);
    bool ok = true;
    if (TRUSTED) {
        pm = tree64(pm, pm, FMax{}); gm = tree64(gm, gm, FMax{});
        // fmaxf skips NaN, so the inputs' finiteness is established through the sums below: a NaN or infinite input
        // makes s NaN or infinite (inf * 0 and inf - inf included)
        const float sb = (float)C * pm * lim.slack * lim.growth;                 // bound of every partial sum
        ok = pm < lim.top[1] && sb < lim.top[0] && (gm + sb) * lim.slack < lim.top[0] && fabsf(s) <= sb;
    }
    if (ok) {
#pragma unroll
        for (int j = 0; j < JMAX; ++j)
            if (j < nj) o[lane + 32 * j] = __fmul_rn(rr<TRUSTED>(fadd, __fsub_rn(b[j], s)), a[j]);
        return;
    }
    softmax_bwd_row_cold(y, gr, o, C, lane, &fadd, &fmul);
}

template <int JMAX, bool TRUSTED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_fwd_rows_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                                                const float* __restrict__ bias, float* __restrict__ out,
                                                                                float* __restrict__ mean, float* __restrict__ rstd, float eps,
                                                                                int64_t rows, int C, const __grid_constant__ LnFmt f,
                                                                                RowLimits lim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    float* y = out + row * C;
    const int nj = C >> 5;
    const float fC = (float)C;
    const RAdd<TRUSTED> qacc{f.acc};
    float v[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        if (j < nj) v[j] = x[lane + 32 * j];
    float s0 = 0.f, s1 = 0.f, xm = 0.f;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2)
        if (j < nj) {
            if (TRUSTED) xm = fmaxf(xm, fmaxf(fabsf(v[j]), fabsf(v[j + 1])));
            s0 = qacc(s0, v[j]); s1 = qacc(s1, v[j + 1]);
        }
    const float sum = tree64(s0, s1, qacc);
    const float m = __fdiv_rn(sum, fC);
    bool ok = true;
    float dm = 0.f;
    if (TRUSTED) {
        xm = tree64(xm, xm, FMax{});
        const float sb = fC * xm * lim.growth;                   // bound of every partial sum of the row
        dm = (xm + sb / fC) * lim.slack;                         // bound of |Q(x - mean)|
        ok = sb < lim.top[0] && fabsf(sum) <= sb && dm < lim.top[0] && dm * dm * lim.slack < lim.top[1] &&
             fC * dm * dm * lim.slack * lim.growth < lim.top[0];
    }
    if (ok) {
        s0 = 0.f; s1 = 0.f;
#pragma unroll
        for (int j = 0; j < JMAX; j += 2)
            if (j < nj) {
                const float d0 = rr<TRUSTED>(f.acc, __fsub_rn(v[j], m)), d1 = rr<TRUSTED>(f.acc, __fsub_rn(v[j + 1], m));
                v[j] = d0; v[j + 1] = d1;
                s0 = qacc(s0, rr<TRUSTED>(f.mul, __fmul_rn(d0, d0)));
                s1 = qacc(s1, rr<TRUSTED>(f.mul, __fmul_rn(d1, d1)));
            }
        const float var = __fdiv_rn(tree64(s0, s1, qacc), fC);
        // per-row scalars take the whole-domain rounding
        const float sd = cast_fp_nearest(__fsqrt_rn(cast_fp_nearest(__fadd_rn(var, eps), f.acc)), f.sqrt);
        float rs = 0.f;
        if (TRUSTED) {
            ok = sd >= 0x1p-20f && sd <= 0x1p20f;
            rs = __frcp_rn(sd);
            ok = ok && dm * rs * 1.001f < lim.top[2];
        }
        if (ok) {
            float pm = 0.f;
#pragma unroll
            for (int j = 0; j < JMAX; ++j)
                if (j < nj) {
                    const float q = TRUSTED ? div_with_rcp(v[j], sd, rs) : __fdiv_rn(v[j], sd);
                    const float p = __fmul_rn(w[lane + 32 * j], rr<TRUSTED>(f.div, q));
                    if (TRUSTED) pm = fmaxf(pm, fabsf(p));
                    v[j] = __fadd_rn(rr<TRUSTED>(f.mul, p), bias[lane + 32 * j]);
                }
            if (TRUSTED) {
                pm = tree64(pm, pm, FMax{});
                // fmaxf skips a NaN product (a NaN weight); the trusted rounding turns it into NaN as the exact one does
                ok = pm < lim.top[1];
            }
            if (ok) {
#pragma unroll
                for (int j = 0; j < JMAX; ++j)
                    if (j < nj) y[lane + 32 * j] = v[j];
                if (lane == 0) {
                    mean[row] = m;
                    rstd[row] = cast_fp_nearest(__fdiv_rn(1.0f, sd), f.div);
                }
                return;
            }
        }
    }
    layernorm_fwd_row_cold(x, w, bias, y, mean, rstd, row, eps, C, lane, &f);
}

template <int JMAX, bool TRUSTED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_bwd_rows_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                                const float* __restrict__ w, const float* __restrict__ mean,
                                                                                const float* __restrict__ rstd, float* __restrict__ gin,
                                                                                int64_t rows, int C, const __grid_constant__ LnFmt f,
                                                                                RowLimits lim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    const float* gr = gout + row * C;
    float* o = gin + row * C;
    const int nj = C >> 5;
    const float fC = (float)C;
    const float m = mean[row], r = rstd[row];
    const RAdd<TRUSTED> qacc{f.acc};
    float xh[JMAX], ng[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        if (j < nj) { xh[j] = x[lane + 32 * j]; ng[j] = __fmul_rn(w[lane + 32 * j], gr[lane + 32 * j]); }
    float xm = 0.f, gm = 0.f;
    if (TRUSTED) {
#pragma unroll
        for (int j = 0; j < JMAX; ++j)
            if (j < nj) { xm = fmaxf(xm, fabsf(xh[j])); gm = fmaxf(gm, fabsf(ng[j])); }
        xm = tree64(xm, xm, FMax{}); gm = tree64(gm, gm, FMax{});
    }
    bool ok = true;
    float hb = 0.f, sa = 0.f, sb = 0.f;
    if (TRUSTED) {
        const float dm = (xm + fabsf(m)) * lim.slack;            // bound of |Q(x - mean)|
        hb = dm * fabsf(r) * lim.slack;                          // bound of |x-hat|
        sa = fC * gm * lim.slack * lim.growth;                   // bound of the partial sums of w * dy
        sb = fC * hb * gm * lim.slack * lim.slack * lim.growth;  // bound of the partial sums of x-hat * w * dy
        ok = dm < lim.top[0] && hb < lim.top[1] && gm < lim.top[1] && hb * gm * lim.slack < lim.top[1] && sa < lim.top[0] &&
             sb < lim.top[0];
    }
    if (ok) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int j = 0; j < JMAX; j += 2)
            if (j < nj) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float h = rr<TRUSTED>(f.mul, __fmul_rn(rr<TRUSTED>(f.acc, __fsub_rn(xh[j + u], m)), r));
                    const float n = rr<TRUSTED>(f.mul, ng[j + u]);
                    xh[j + u] = h; ng[j + u] = n;
                    const float dot = rr<TRUSTED>(f.mul, __fmul_rn(h, n));
                    if (u == 0) { a0 = qacc(a0, n); b0 = qacc(b0, dot); }
                    else { a1 = qacc(a1, n); b1 = qacc(b1, dot); }
                }
            }
        const float ta = tree64(a0, a1, qacc), tb = tree64(b0, b1, qacc);
        // per-row scalars take the whole-domain rounding
        const float gs = cast_fp_nearest(__fdiv_rn(ta, fC), f.div);
        const float gsx = cast_fp_nearest(__fdiv_rn(tb, fC), f.div);
        if (TRUSTED) {
            // NaN or infinite inputs surface in the sums (fmaxf skipped them in the maxima)
            const float g1 = (gm * lim.slack + fabsf(gs)) * lim.slack;
            const float g2 = (g1 + hb * fabsf(gsx) * lim.slack) * lim.slack;
            ok = fabsf(ta) <= sa && fabsf(tb) <= sb && hb * fabsf(gsx) < lim.top[1] && g1 < lim.top[0] && g2 < lim.top[0] &&
                 g2 * fabsf(r) < lim.top[1];
        }
        if (ok) {
#pragma unroll
            for (int j = 0; j < JMAX; ++j)
                if (j < nj) {
                    const float wg = rr<TRUSTED>(f.mul, __fmul_rn(xh[j], gsx));
                    float gi = rr<TRUSTED>(f.acc, __fsub_rn(ng[j], gs));
                    gi = rr<TRUSTED>(f.acc, __fsub_rn(gi, wg));
                    o[lane + 32 * j] = rr<TRUSTED>(f.mul, __fmul_rn(gi, r));
                }
            return;
        }
    }
    layernorm_bwd_row_cold(x, gr, w, m, r, o, C, lane, &f);
}

__device__ __noinline__ void softmax_fwd_row_cold(const float* x, float* y, int C, int lane, const Caster* fexp, const Caster* foff,
                                                 const Caster* facc) {
    softmax_fwd_row_tree(x, y, C, 1, lane, *fexp, *foff, *facc);
}
__device__ __noinline__ void softmax_bwd_row_cold(const float* y, const float* gr, float* o, int C, int lane, const Caster* fadd,
                                                 const Caster* fmul) {
    softmax_bwd_row_tree(y, gr, o, C, 1, lane, *fadd, *fmul);
}
__device__ __noinline__ void layernorm_fwd_row_cold(const float* x, const float* w, const float* bias, float* y, float* mean, float* rstd,
                                                   int64_t row, float eps, int C, int lane, const LnFmt* f) {
    layernorm_fwd_row<true>(x, w, bias, y, mean, rstd, row, eps, C, 1, lane, 32, *f);
}
__device__ __noinline__ void layernorm_bwd_row_cold(const float* x, const float* gr, const float* w, float m, float r, float* o, int C,
                                                   int lane, const LnFmt* f) {
    layernorm_bwd_row<true>(x, gr, w, m, r, o, C, 1, lane, 32, *f);
}

// Column sums in row order: out[c] = fold over rows r = 0..R-1 of Q(acc + v[r, c]), the association of both
// references for the layernorm weight/bias gradients (layernorm_kernel.h:206-237, layernorm.h:100-103) and of
// the qsum loop (functional.py:736-748).  The chain per column is serial by definition, so the kernel splits
// the work by role: a CTA owns 32 columns; eight producer warps stream row tiles (64 rows x 32 columns,
// coalesced 128-byte row segments), do the per-element arithmetic that does not depend on the running sum
// (for layernorm: x-hat * dy, recomputed from the inputs instead of staged through the reference's scratch
// tensor, fp_kernel.cu:481-487) and park the addends in shared memory; one consumer warp (lane = column)
// walks the parked tile in row order through the rounded adds.  Tiles are double buffered: the consumer
// works on tile t while the producers fetch tile t + 1, with one barrier per tile.
constexpr int kColTile = 32;        // columns per CTA
constexpr int kRowTile = 64;        // rows per tile (two buffers of two tensors stay within 48 KB of static shared memory)
constexpr int kProducerWarps = 8;
constexpr int kColsumThreads = (kProducerWarps + 1) * 32;

// MODE 0: layernorm parameter gradients (two chains: x-hat*dy -> out0, dy -> out1).  MODE 1: plain column sum of `in`.
template <int MODE>
__global__ void __launch_bounds__(kColsumThreads) colsum_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                float* __restrict__ out0, float* __restrict__ out1, RowGeom g,
                                                                Caster facc, Caster fmul, SeqAdder seq) {
    __shared__ float sA[2][kRowTile][kColTile];
    __shared__ float sB[MODE == 0 ? 2 : 1][MODE == 0 ? kRowTile : 1][kColTile];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * kColTile + lane;
    const bool col_ok = col < g.channel;
    const int64_t st = g.inner;
    const int64_t ntiles = (g.rows + kRowTile - 1) / kRowTile;

    auto produce = [&](int64_t t) {      // producer warps: rows warp, warp + 8, ... of the tile
        const int buf = (int)(t & 1);
        const int64_t r0 = t * kRowTile;
        constexpr int PER = kRowTile / kProducerWarps;     // rows per producer warp, in batches of 8
#pragma unroll
        for (int h = 0; h < PER / 8; ++h) {
            float xv[8], gv[8], mv[8], rv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int lr = warp * PER + h * 8 + u;
                const int64_t row = r0 + lr;
                const bool ok = col_ok && row < g.rows;
                const int64_t idx = ok ? row_base(g, row) + col * st : 0;
                xv[u] = ok ? in[idx] : 0.f;
                if (MODE == 0) { gv[u] = ok ? gout[idx] : 0.f; mv[u] = ok ? mean[row] : 0.f; rv[u] = ok ? rstd[row] : 0.f; }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int lr = warp * PER + h * 8 + u;
                if (MODE == 0) {
                    const float xhat = fmul(__fmul_rn(facc(__fsub_rn(xv[u], mv[u])), rv[u]));
                    sA[buf][lr][lane] = fmul(__fmul_rn(xhat, gv[u]));
                    sB[buf][lr][lane] = gv[u];
                } else {
                    sA[buf][lr][lane] = xv[u];
                }
            }
        }
    };

    float acc0 = 0.f, acc1 = 0.f;
    if (warp < kProducerWarps && ntiles > 0) produce(0);
    __syncthreads();
    for (int64_t t = 0; t < ntiles; ++t) {
        if (warp < kProducerWarps) {
            if (t + 1 < ntiles) produce(t + 1);
        } else {
            const int buf = (int)(t & 1);
            const int64_t left = g.rows - t * kRowTile;
            const int nrows = left < kRowTile ? (int)left : kRowTile;
            int r = 0;
            for (; r + 8 <= nrows; r += 8) {
                float a[8], b[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) { a[u] = sA[buf][r + u][lane]; if (MODE == 0) b[u] = sB[buf][r + u][lane]; }
                acc0 = seq.add(acc0, a);
                if (MODE == 0) acc1 = seq.add(acc1, b);
            }
            for (; r < nrows; ++r) {
                const float a[1] = {sA[buf][r][lane]};
                acc0 = seq.add(acc0, a);
                if (MODE == 0) { const float b[1] = {sB[buf][r][lane]}; acc1 = seq.add(acc1, b); }
            }
        }
        __syncthreads();
    }
    if (warp == kProducerWarps && col_ok) {
        out0[col] = acc0;
        if (MODE == 0) out1[col] = acc1;
    }
}

int check_geom(const char* who, int64_t outer, int channel, int64_t inner) {
    MPT_REQUIRE(outer >= 0 && channel >= 0 && inner >= 0, "%s: negative extent", who);
    return MPT_OK;
}

unsigned row_blocks(int64_t rows, bool tree) {
    const int64_t per = tree ? kWarpsPerBlock : kWarpsPerBlock * 32;
    return (unsigned)((rows + per - 1) / per);
}

// ---- host side of the register-resident row kernels
bool rows_shape_ok(const RowGeom& g, int max_channel) {
    return g.inner == 1 && g.channel % 64 == 0 && g.channel <= max_channel;
}
float top_of(const Caster& c) { return ldexpf(1.0f, fast_rn_exp_limit(c.any.fp) + 1); }
double step_growth(const Caster& c) { return 1.0 + ldexp(1.0, -(c.any.fp.man + 1)); }
bool small_exp(const Caster& c) { return c.use_fast && c.any.fp.exp < 8; }

RowLimits ln_limits(const LnFmt& f, int channel) {
    RowLimits lim{};
    lim.top[0] = top_of(f.acc); lim.top[1] = top_of(f.mul); lim.top[2] = top_of(f.div);
    lim.growth = (float)(pow(step_growth(f.acc), channel / 64 + 6) * 1.001);
    double sg = step_growth(f.acc);
    if (step_growth(f.mul) > sg) sg = step_growth(f.mul);
    if (step_growth(f.div) > sg) sg = step_growth(f.div);
    lim.slack = (float)(sg * sg * 1.001);
    return lim;
}

#define MPT_ROWS_DISPATCH(KERNEL, MAXJ, TRUSTED, ...)                                                                       \
    do {                                                                                                                    \
        const int nj_ = g.channel / 32;                                                                                     \
        const unsigned grid_ = row_blocks(g.rows, true);                                                                    \
        const unsigned thr_ = kWarpsPerBlock * 32;                                                                          \
        cudaStream_t st_ = as_stream(stream);                                                                               \
        if (TRUSTED) {                                                                                                      \
            if (nj_ <= 8) KERNEL<8, true><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                            \
            else if (nj_ <= 16) KERNEL<16, true><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                     \
            else if (nj_ <= 32 || MAXJ == 32) KERNEL<32, true><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                       \
            else KERNEL<MAXJ, true><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                                  \
        } else {                                                                                                            \
            if (nj_ <= 8) KERNEL<8, false><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                           \
            else if (nj_ <= 16) KERNEL<16, false><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                    \
            else if (nj_ <= 32 || MAXJ == 32) KERNEL<32, false><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                      \
            else KERNEL<MAXJ, false><<<grid_, thr_, 0, st_>>>(__VA_ARGS__);                                                 \
        }                                                                                                                   \
    } while (0)

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
        const bool trusted = small_exp(fe) && small_exp(fo) && small_exp(fa) && fast_rn_exp_limit(fe.any.fp) >= 0;
        RowLimits lim{};
        lim.top[1] = top_of(fo); lim.top[2] = top_of(fa);
        MPT_ROWS_DISPATCH(softmax_fwd_rows_kernel, 64, trusted, in, out, g.rows, g.channel, fe, fo, fa, lim);
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
        const bool trusted = small_exp(fa) && small_exp(fm);
        RowLimits lim{};
        lim.top[0] = top_of(fa); lim.top[1] = top_of(fm);
        lim.growth = (float)(pow(step_growth(fa), channel / 64 + 6) * 1.001);
        const double sg = step_growth(fa) > step_growth(fm) ? step_growth(fa) : step_growth(fm);
        lim.slack = (float)(sg * sg * 1.001);
        MPT_ROWS_DISPATCH(softmax_bwd_rows_kernel, 32, trusted, y, grad, out, g.rows, g.channel, fa, fm, lim);
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
        const bool trusted = small_exp(f.acc) && small_exp(f.mul) && small_exp(f.div);
        const RowLimits lim = ln_limits(f, channel);
        MPT_ROWS_DISPATCH(layernorm_fwd_rows_kernel, 64, trusted, in, weight, bias, out, mean, rstd, eps, g.rows, g.channel, f, lim);
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
            const bool trusted = small_exp(f.acc) && small_exp(f.mul);
            const RowLimits lim = ln_limits(f, channel);
            MPT_ROWS_DISPATCH(layernorm_bwd_rows_kernel, 32, trusted, in, grad_out, weight, mean, rstd, grad_in, g.rows, g.channel, f, lim);
        } else
        if (tree) layernorm_bwd_dx_kernel<true><<<row_blocks(g.rows, true), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        else layernorm_bwd_dx_kernel<false><<<row_blocks(g.rows, false), kWarpsPerBlock * 32, 0, as_stream(stream)>>>(in, grad_out, weight, mean, rstd, grad_in, g, f);
        rc = check_launch("layernorm_backward (input gradient)");
        if (rc) return rc;
    }
    colsum_kernel<0><<<(channel + kColTile - 1) / kColTile, kColsumThreads, 0, as_stream(stream)>>>(in, grad_out, mean, rstd, grad_gamma, grad_beta, g,
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
    colsum_kernel<1><<<(unsigned)((cols + kColTile - 1) / kColTile), kColsumThreads, 0, as_stream(stream)>>>(in, nullptr, nullptr, nullptr, out, nullptr, g,
                                                                                                        Caster::make(f), Caster::make(f), SeqAdder::make(f));
    return check_launch("qsum_rows");
}

}
