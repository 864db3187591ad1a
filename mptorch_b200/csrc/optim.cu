// Quantized optimizer steps as one launch over many tensors: the arithmetic of the reference's QSGD
// (mptorch/optim/sgd.py:63-150) and QAdamW (mptorch/optim/adamw.py:44-150) with their quantizer callables of the form
// Q(x + y * z), momentum / moment buffers, and the Kahan compensation buffer of the weight update.
//
// The reference walks the parameters in Python and issues a dozen small torch kernels plus several quantizer
// launches per tensor; here a launch carries a table of up to kOptMax tensors in its kernel parameters (nothing is
// allocated), a CTA finds the tensor its block index falls into and updates one contiguous chunk of it in place.
// HBM-bound: per element the SGD step reads and writes parameter, gradient, momentum and compensation once each.
//
// Every fp32 operation is written out as the separately rounded operation the reference's torch expression performs on a
// CUDA tensor: `a.add_(b, alpha=s)` and `addcdiv_` are one fused multiply-add, a tensor divided by a Python scalar is a
// multiplication by the reciprocal (taken in double precision, rounded to fp32), `x + y * z` inside a quantizer callable is a multiplication then an addition.
#include "cast.cuh"
#include "common.cuh"

namespace mpt {
namespace {

constexpr int kThreads = 256;
constexpr int kOptMax = 40;
constexpr int kOptChunk = kThreads * 8;      // elements per CTA

struct OptTable {
    float* param[kOptMax];
    float* grad[kOptMax];
    float* buf0[kOptMax];    // SGD: momentum buffer            AdamW: exp_avg
    float* buf1[kOptMax];    // SGD: compensation buffer        AdamW: exp_avg_sq
    float* buf2[kOptMax];    //                                 AdamW: compensation buffer
    float* buf3[kOptMax];    //                                 AdamW: max_exp_avg_sq (amsgrad)
    int64_t n[kOptMax];
    int first_block[kOptMax + 1];
    int flags[kOptMax];      // per tensor: MPT_OPT_FIRST_STEP
    int count;
};

// The exact caster as a function call: it is rarely taken, and a copy inlined at every rounding of an unrolled
// update would push the kernel out of the instruction cache.
__device__ __noinline__ float exact_nearest(float x, FpFmt fmt) { return cast_fp_nearest(x, fmt); }

// One quantizer Q of the optimizer: identity (no quantizer given), the FP-pipe rounding, or the exact caster.
struct Rounder {
    FullRn fast;
    FpFmt fmt;
    int mode;                // 0 identity, 1 fast, 2 exact, 3 a float format without subnormals (fast in line<true> only)
    __device__ __forceinline__ float operator()(float x) const {
        if (mode == 0) return x;
        if (mode >= 2) return exact_nearest(x, fmt);
        if (fmt.exp == 8) {
            // formats with an 8-bit exponent: fp32 denormals and the largest magnitudes go to the exact caster; a
            // positive zero (the usual gradient of an unused embedding row) is its own rounding
            const uint32_t t = f2u(x), a = t & 0x7FFFFFFFu;
            if (t == 0u) return x;
            if (a >= fast.exact_from || a < 0x00800000u) return exact_nearest(x, fmt);
        }
        return fast.line(x);
    }
    // the reference's callable: Q(x + y * z), the product rounded to fp32 before the sum
    __device__ __forceinline__ float fma3(float x, float y, float z) const { return (*this)(add_rn(x, mul_rn(y, z))); }

    // The same without a branch, for modes 0 and 1: the FP-pipe rounding is always computed, and an input the exact
    // caster would have to handle (8-bit exponent: an fp32 denormal or a magnitude near the top of the range) only
    // sets `rare`; the caller then recomputes that element through operator().  Straight-line code lets the compiler
    // interleave the roundings of independent elements.
    uint32_t span;           // rare when (|x| bits - 0x00800000) >= span, zero excepted
    uint32_t check;          // 1 where that test applies (mode 1 with an 8-bit exponent; mode 3)
    // NS: the kernel instantiation for formats without subnormals (modes 0 and 3): the settling rounding, with fp32
    // denormals, -0, overflow, infinities and NaN left to the redo.
    template <bool NS>
    __device__ __forceinline__ float line(float x, uint32_t& rare) const {
        const uint32_t t = f2u(x), a = t & 0x7FFFFFFFu;
        rare |= ((a - 0x00800000u >= span) && t != 0u) ? check : 0u;
        const float y = (t == 0u) ? x : (NS ? fast_rn_nosub(fast.fast, x) : fast.line(x));
        return mode == 0 ? x : y;
    }
    template <bool NS>
    __device__ __forceinline__ float line3(float x, float y, float z, uint32_t& rare) const { return line<NS>(add_rn(x, mul_rn(y, z)), rare); }
};

Rounder make_rounder(int enabled, int man, int exp, int sub, int sat) {
    Rounder r;
    r.fmt = make_fmt(enabled ? man : 23, enabled ? exp : 8, sub, sat);
    r.fast = FullRn::make(r.fmt);
    const bool nosub = !r.fmt.sub && r.fmt.man <= 21 && r.fmt.exp >= 2;
    r.mode = !enabled ? 0 : (fast_rn_supported(r.fmt) ? 1 : (nosub ? 3 : 2));
    r.check = ((r.mode == 1 && r.fmt.exp == 8) || r.mode == 3) ? 1u : 0u;
    const uint32_t top = r.fast.ovf_from < r.fast.exact_from ? r.fast.ovf_from : r.fast.exact_from;
    r.span = r.mode == 3 ? top - 0x00800000u : (r.check ? r.fast.exact_from - 0x00800000u : 0xFFFFFFFFu);
    return r;
}

struct SgdArgs {
    float lr, neg_lr, momentum, one_minus_dampening, weight_decay;
    int nesterov, compensated, has_momentum_quant, has_acc_quant;
    Rounder qm, qa;
};

struct AdamArgs {
    float beta1, beta2, one_minus_beta1, one_minus_beta2, inv_sqrt_bc2, eps, step_size, neg_step_size;
    int amsgrad, compensated, has_momentum_quant, has_acc_quant;
    Rounder qm, qa;
};

__device__ __forceinline__ int find_tensor(const OptTable& t, int b) {
    int lo = 0, hi = t.count;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (t.first_block[mid] <= b) lo = mid; else hi = mid;
    }
    return lo;
}

// Kahan-compensated weight update shared by both optimizers (sgd.py:121-138, adamw.py:131-146): `update` is the
// step before the sign flip (lr * d_p, or step_size * u).
__device__ __forceinline__ void compensated_update(float& p, float& comp, float d, float scale, const Rounder& qa) {
    const float y = -qa.fma3(comp, d, scale);
    const float s = qa.fma3(p, y, 1.0f);
    comp = qa.fma3(qa.fma3(s, p, -1.0f), y, -1.0f);
    p = s;
}

// Internal per-tensor flag (set by launch_optim, never by the caller): every buffer of the tensor starts on a 16-byte
// boundary, so full chunks move as float4.
constexpr int kOptAligned = 1 << 30;

// One element of the QSGD step.  m and c are read only where the configuration uses them.
__device__ __forceinline__ void sgd_elem(float& p, float& g, float& m, float& c, bool first, const SgdArgs& a) {
    if (a.weight_decay != 0.0f) g = fma_rn(p, a.weight_decay, g);      // d_p.add_(p.data, alpha=weight_decay), in place on the gradient
    float d = g;
    if (a.momentum != 0.0f) {
        float buf;
        if (first) {
            // momentum_quant(clone(d_p), zeros, zeros), or a plain clone
            buf = a.has_momentum_quant ? a.qm.fma3(g, 0.0f, 0.0f) : g;
        } else {
            const float scaled = mul_rn(m, a.momentum);                // buf.mul_(momentum)
            buf = a.has_momentum_quant ? a.qm.fma3(scaled, g, a.one_minus_dampening)
                                       : fma_rn(g, a.one_minus_dampening, scaled);   // .add_(d_p, alpha=1 - dampening)
        }
        m = buf;
        d = a.nesterov ? fma_rn(buf, a.momentum, g) : buf;             // d_p.add(buf, alpha=momentum)
    }
    if (a.has_acc_quant) {
        if (!a.compensated) p = a.qa.fma3(p, d, a.neg_lr);
        else compensated_update(p, c, d, a.lr, a.qa);
    } else if (!a.compensated) {
        p = fma_rn(d, a.neg_lr, p);                                    // p.add_(d_p, alpha=-lr)
    } else {
        // u = -lr * d_p; y = u - comp; s = p + y; comp = (s - p) - y
        const float u = mul_rn(a.neg_lr, d), y = add_rn(u, -c), s = add_rn(p, y);
        c = add_rn(add_rn(s, -p), -y);
        p = s;
    }
}

constexpr int kOptPer = kOptChunk / kThreads;            // elements per thread and chunk
constexpr int kOptVecs = kOptPer / 4;                    // float4 groups per thread and chunk

__device__ __forceinline__ void ld4(const float* src, float* dst) {
    const float4 v = *reinterpret_cast<const float4*>(src);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void st4(float* dst, const float* src) { *reinterpret_cast<float4*>(dst) = make_float4(src[0], src[1], src[2], src[3]); }
__device__ __forceinline__ void zero4(float* dst) { dst[0] = dst[1] = dst[2] = dst[3] = 0.0f; }

#define MPT_EACH for (int e = 0; e < kOptPer; ++e)

template <bool NS>
__device__ __forceinline__ void compensated_line(float& p, float& comp, float d, float scale, const Rounder& qa, uint32_t& rare) {
    const float y = -qa.line3<NS>(comp, d, scale, rare);
    const float s = qa.line3<NS>(p, y, 1.0f, rare);
    comp = qa.line3<NS>(qa.line3<NS>(s, p, -1.0f, rare), y, -1.0f, rare);
    p = s;
}

// The QSGD step over the kOptPer elements a thread holds, one phase at a time: the configuration's branches sit
// between the phases, each phase is straight-line code over independent elements.  Same operations as sgd_elem.
template <bool NS>
__device__ __forceinline__ uint32_t sgd_block(float (&p)[kOptPer], float (&g)[kOptPer], float (&m)[kOptPer], float (&c)[kOptPer], bool first,
                                              const SgdArgs& a) {
    uint32_t rare = 0u;
    float d[kOptPer];
    if (a.weight_decay != 0.0f) {
#pragma unroll
        MPT_EACH g[e] = fma_rn(p[e], a.weight_decay, g[e]);
    }
    if (a.momentum != 0.0f) {
        if (first) {
            if (a.has_momentum_quant) {
#pragma unroll
                MPT_EACH m[e] = a.qm.line3<NS>(g[e], 0.0f, 0.0f, rare);
            } else {
#pragma unroll
                MPT_EACH m[e] = g[e];
            }
        } else if (a.has_momentum_quant) {
#pragma unroll
            MPT_EACH m[e] = a.qm.line3<NS>(mul_rn(m[e], a.momentum), g[e], a.one_minus_dampening, rare);
        } else {
#pragma unroll
            MPT_EACH m[e] = fma_rn(g[e], a.one_minus_dampening, mul_rn(m[e], a.momentum));
        }
        if (a.nesterov) {
#pragma unroll
            MPT_EACH d[e] = fma_rn(m[e], a.momentum, g[e]);
        } else {
#pragma unroll
            MPT_EACH d[e] = m[e];
        }
    } else {
#pragma unroll
        MPT_EACH d[e] = g[e];
    }
    if (a.has_acc_quant) {
        if (!a.compensated) {
#pragma unroll
            MPT_EACH p[e] = a.qa.line3<NS>(p[e], d[e], a.neg_lr, rare);
        } else {
#pragma unroll
            MPT_EACH compensated_line<NS>(p[e], c[e], d[e], a.lr, a.qa, rare);
        }
    } else if (!a.compensated) {
#pragma unroll
        MPT_EACH p[e] = fma_rn(d[e], a.neg_lr, p[e]);
    } else {
#pragma unroll
        MPT_EACH {
            const float u = mul_rn(a.neg_lr, d[e]), y = add_rn(u, -c[e]), s = add_rn(p[e], y);
            c[e] = add_rn(add_rn(s, -p[e]), -y);
            p[e] = s;
        }
    }
    return rare;
}

// A thread's elements of one chunk again, from memory, through the branching rounder: taken when sgd_block met an
// input its straight-line rounding does not cover (nothing of the chunk has been stored yet at that point).
__device__ __noinline__ void sgd_redo(float* P, float* G, float* M, float* C, int64_t base, bool first, const SgdArgs& a) {
    const bool use_m = a.momentum != 0.0f, rd_m = use_m && !first, use_c = a.compensated != 0, wr_g = a.weight_decay != 0.0f;
#pragma unroll 1
    for (int e = 0; e < kOptPer; ++e) {
        const int64_t i = base + (int64_t)(e >> 2) * (kThreads * 4) + (e & 3);
        float p = P[i], g = G[i], m = rd_m ? M[i] : 0.0f, c = use_c ? C[i] : 0.0f;
        sgd_elem(p, g, m, c, first, a);
        P[i] = p;
        if (wr_g) G[i] = g;
        if (use_m) M[i] = m;
        if (use_c) C[i] = c;
    }
}

// LINE: neither quantizer needs the exact caster throughout (the host decides), so aligned full chunks take the
// vector path with straight-line roundings.
template <bool LINE, bool NS = false>
__global__ void __launch_bounds__(kThreads) qsgd_kernel(const __grid_constant__ OptTable t, const __grid_constant__ SgdArgs a) {
    const int k = find_tensor(t, blockIdx.x);
    float* __restrict__ P = t.param[k];
    float* __restrict__ G = t.grad[k];
    float* __restrict__ M = t.buf0[k];
    float* __restrict__ C = t.buf1[k];
    const bool first = (t.flags[k] & MPT_OPT_FIRST_STEP) != 0;
    const bool use_m = a.momentum != 0.0f, rd_m = use_m && !first, use_c = a.compensated != 0, wr_g = a.weight_decay != 0.0f;
    const int64_t begin = (int64_t)(blockIdx.x - t.first_block[k]) * kOptChunk;
    const int64_t end = begin + kOptChunk < t.n[k] ? begin + kOptChunk : t.n[k];
    if (LINE && (t.flags[k] & kOptAligned) && end - begin == kOptChunk) {
        // all loads of the chunk first, so that every thread has its elements of each buffer in flight at once
        const int64_t base = begin + (int64_t)threadIdx.x * 4;
        float p[kOptPer], g[kOptPer], m[kOptPer], c[kOptPer];
#pragma unroll
        for (int h = 0; h < kOptVecs; ++h) {
            const int64_t i = base + (int64_t)h * (kThreads * 4);
            ld4(P + i, p + 4 * h);
            ld4(G + i, g + 4 * h);
            if (rd_m) ld4(M + i, m + 4 * h); else zero4(m + 4 * h);
            if (use_c) ld4(C + i, c + 4 * h); else zero4(c + 4 * h);
        }
        if (sgd_block<NS>(p, g, m, c, first, a)) { sgd_redo(P, G, M, C, base, first, a); return; }
#pragma unroll
        for (int h = 0; h < kOptVecs; ++h) {
            const int64_t i = base + (int64_t)h * (kThreads * 4);
            st4(P + i, p + 4 * h);
            if (wr_g) st4(G + i, g + 4 * h);
            if (use_m) st4(M + i, m + 4 * h);
            if (use_c) st4(C + i, c + 4 * h);
        }
        return;
    }
    for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
        float p = P[i], g = G[i], m = rd_m ? M[i] : 0.0f, c = use_c ? C[i] : 0.0f;
        sgd_elem(p, g, m, c, first, a);
        P[i] = p;
        if (wr_g) G[i] = g;
        if (use_m) M[i] = m;
        if (use_c) C[i] = c;
    }
}

// One element of the QAdamW step.  c and vm are read only where the configuration uses them.
__device__ __forceinline__ void adam_elem(float& p, float g, float& m, float& v, float& c, float& vm, const AdamArgs& a) {
    m = mul_rn(m, a.beta1);                                 // exp_avg.mul_(beta1)
    v = mul_rn(v, a.beta2);                                 // exp_avg_sq.mul_(beta2)
    const float gg = mul_rn(g, g);
    if (a.has_momentum_quant) {
        m = a.qm.fma3(m, g, a.one_minus_beta1);
        v = a.qm.fma3(v, gg, a.one_minus_beta2);
    } else {
        m = fma_rn(g, a.one_minus_beta1, m);                // .add_(d_p, alpha=1 - beta1)
        v = fma_rn(a.one_minus_beta2, gg, v);               // .addcmul_(d_p, d_p, value=1 - beta2)
    }
    float vv = v;
    if (a.amsgrad) {
        vv = fmaxf(vm, v);
        if (vm != vm || v != v) vv = __uint_as_float(0x7FC00000u);   // torch.max propagates NaN
        vm = vv;
    }
    // (sqrt(v) / sqrt(bias_correction2)).add_(eps): a tensor over a Python scalar multiplies by the reciprocal
    const float denom = add_rn(mul_rn(__fsqrt_rn(vv), a.inv_sqrt_bc2), a.eps);
    if (a.has_acc_quant) {
        if (!a.compensated) {
            p = fma_rn(a.neg_step_size, __fdiv_rn(m, denom), p);    // addcdiv_(exp_avg, denom, value=-step_size)
            p = a.qa.fma3(p, 0.0f, 0.0f);
        } else {
            const float u = a.qa.fma3(__fdiv_rn(m, denom), 0.0f, 0.0f);
            compensated_update(p, c, u, a.step_size, a.qa);
        }
    } else if (!a.compensated) {
        p = fma_rn(a.neg_step_size, __fdiv_rn(m, denom), p);
    } else {
        // u = -step_size * exp_avg / denom; y = u - comp; s = p + y; comp = (s - p) - y
        const float u = __fdiv_rn(mul_rn(a.neg_step_size, m), denom), y = add_rn(u, -c), s = add_rn(p, y);
        c = add_rn(add_rn(s, -p), -y);
        p = s;
    }
}

// The QAdamW step over a thread's elements, phase by phase (see sgd_block).  Same operations as adam_elem.
template <bool NS>
__device__ __forceinline__ uint32_t adam_block(float (&p)[kOptPer], const float (&g)[kOptPer], float (&m)[kOptPer], float (&v)[kOptPer],
                                               float (&c)[kOptPer], float (&vm)[kOptPer], const AdamArgs& a) {
    uint32_t rare = 0u;
    float q[kOptPer];                                      // exp_avg / denom
    if (a.has_momentum_quant) {
#pragma unroll
        MPT_EACH {
            m[e] = a.qm.line3<NS>(mul_rn(m[e], a.beta1), g[e], a.one_minus_beta1, rare);
            v[e] = a.qm.line3<NS>(mul_rn(v[e], a.beta2), mul_rn(g[e], g[e]), a.one_minus_beta2, rare);
        }
    } else {
#pragma unroll
        MPT_EACH {
            m[e] = fma_rn(g[e], a.one_minus_beta1, mul_rn(m[e], a.beta1));
            v[e] = fma_rn(a.one_minus_beta2, mul_rn(g[e], g[e]), mul_rn(v[e], a.beta2));
        }
    }
    if (a.amsgrad) {
#pragma unroll
        MPT_EACH {
            float vv = fmaxf(vm[e], v[e]);
            if (vm[e] != vm[e] || v[e] != v[e]) vv = __uint_as_float(0x7FC00000u);
            vm[e] = vv;
            q[e] = vv;
        }
    } else {
#pragma unroll
        MPT_EACH q[e] = v[e];
    }
    const bool scale_first = !a.has_acc_quant && a.compensated;      // that branch multiplies by -step_size before dividing
#pragma unroll
    MPT_EACH {
        const float denom = add_rn(mul_rn(__fsqrt_rn(q[e]), a.inv_sqrt_bc2), a.eps);
        q[e] = __fdiv_rn(scale_first ? mul_rn(a.neg_step_size, m[e]) : m[e], denom);
    }
    if (a.has_acc_quant) {
        if (!a.compensated) {
#pragma unroll
            MPT_EACH p[e] = a.qa.line3<NS>(fma_rn(a.neg_step_size, q[e], p[e]), 0.0f, 0.0f, rare);
        } else {
#pragma unroll
            MPT_EACH compensated_line<NS>(p[e], c[e], a.qa.line3<NS>(q[e], 0.0f, 0.0f, rare), a.step_size, a.qa, rare);
        }
    } else if (!a.compensated) {
#pragma unroll
        MPT_EACH p[e] = fma_rn(a.neg_step_size, q[e], p[e]);
    } else {
#pragma unroll
        MPT_EACH {
            const float y = add_rn(q[e], -c[e]), s = add_rn(p[e], y);
            c[e] = add_rn(add_rn(s, -p[e]), -y);
            p[e] = s;
        }
    }
    return rare;
}

__device__ __noinline__ void adam_redo(float* P, const float* G, float* M, float* V, float* C, float* VM, int64_t base, const AdamArgs& a) {
    const bool use_c = a.compensated != 0, use_vm = a.amsgrad != 0;
#pragma unroll 1
    for (int e = 0; e < kOptPer; ++e) {
        const int64_t i = base + (int64_t)(e >> 2) * (kThreads * 4) + (e & 3);
        float p = P[i], m = M[i], v = V[i], c = use_c ? C[i] : 0.0f, vm = use_vm ? VM[i] : 0.0f;
        adam_elem(p, G[i], m, v, c, vm, a);
        P[i] = p;
        M[i] = m;
        V[i] = v;
        if (use_c) C[i] = c;
        if (use_vm) VM[i] = vm;
    }
}

template <bool LINE, bool NS = false>
__global__ void __launch_bounds__(kThreads) qadamw_kernel(const __grid_constant__ OptTable t, const __grid_constant__ AdamArgs a) {
    const int k = find_tensor(t, blockIdx.x);
    float* __restrict__ P = t.param[k];
    const float* __restrict__ G = t.grad[k];
    float* __restrict__ M = t.buf0[k];
    float* __restrict__ V = t.buf1[k];
    float* __restrict__ C = t.buf2[k];
    float* __restrict__ VM = t.buf3[k];
    const bool use_c = a.compensated != 0, use_vm = a.amsgrad != 0;
    const int64_t begin = (int64_t)(blockIdx.x - t.first_block[k]) * kOptChunk;
    const int64_t end = begin + kOptChunk < t.n[k] ? begin + kOptChunk : t.n[k];
    if (LINE && (t.flags[k] & kOptAligned) && end - begin == kOptChunk) {
        const int64_t base = begin + (int64_t)threadIdx.x * 4;
        float p[kOptPer], g[kOptPer], m[kOptPer], v[kOptPer], c[kOptPer], vm[kOptPer];
#pragma unroll
        for (int h = 0; h < kOptVecs; ++h) {
            const int64_t i = base + (int64_t)h * (kThreads * 4);
            ld4(P + i, p + 4 * h);
            ld4(G + i, g + 4 * h);
            ld4(M + i, m + 4 * h);
            ld4(V + i, v + 4 * h);
            if (use_c) ld4(C + i, c + 4 * h); else zero4(c + 4 * h);
            if (use_vm) ld4(VM + i, vm + 4 * h); else zero4(vm + 4 * h);
        }
        if (adam_block<NS>(p, g, m, v, c, vm, a)) { adam_redo(P, G, M, V, C, VM, base, a); return; }
#pragma unroll
        for (int h = 0; h < kOptVecs; ++h) {
            const int64_t i = base + (int64_t)h * (kThreads * 4);
            st4(P + i, p + 4 * h);
            st4(M + i, m + 4 * h);
            st4(V + i, v + 4 * h);
            if (use_c) st4(C + i, c + 4 * h);
            if (use_vm) st4(VM + i, vm + 4 * h);
        }
        return;
    }
    for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
        float p = P[i], m = M[i], v = V[i], c = use_c ? C[i] : 0.0f, vm = use_vm ? VM[i] : 0.0f;
        adam_elem(p, G[i], m, v, c, vm, a);
        P[i] = p;
        M[i] = m;
        V[i] = v;
        if (use_c) C[i] = c;
        if (use_vm) VM[i] = vm;
    }
}

#undef MPT_EACH

template <class Args, class Kernel>
int launch_optim(const mpt_optim_tensor* tensors, int count, const Args& args, Kernel kern, bool need0, bool need1, bool need2, bool need3,
                 cudaStream_t st, const char* who) {
    int i = 0;
    while (i < count) {
        OptTable t{};
        int blocks = 0, k = 0;
        for (; i < count && k < kOptMax; ++i) {
            const mpt_optim_tensor& x = tensors[i];
            if (x.n == 0) continue;
            const int64_t nb = (x.n + kOptChunk - 1) / kOptChunk;
            if (nb > 0x3FFFFFFF - blocks) break;
            t.param[k] = x.param; t.grad[k] = x.grad; t.buf0[k] = x.buf0; t.buf1[k] = x.buf1; t.buf2[k] = x.buf2; t.buf3[k] = x.buf3;
            const uintptr_t bits = (uintptr_t)x.param | (uintptr_t)x.grad | (uintptr_t)x.buf0 | (uintptr_t)x.buf1 | (uintptr_t)x.buf2 | (uintptr_t)x.buf3;
            t.n[k] = x.n; t.flags[k] = (x.flags & ~kOptAligned) | ((bits & 15) == 0 ? kOptAligned : 0); t.first_block[k] = blocks;
            blocks += (int)nb;
            ++k;
        }
        if (k == 0) {
            if (i < count) { set_error("%s: tensor %d is too large for one launch", who, i); return MPT_ERR_INVALID_ARGUMENT; }
            break;
        }
        t.first_block[k] = blocks;
        t.count = k;
        kern<<<(unsigned)blocks, kThreads, 0, st>>>(t, args);
        const int rc = check_launch(who);
        if (rc) return rc;
    }
    (void)need0; (void)need1; (void)need2; (void)need3;
    return MPT_OK;
}

int check_tensors(const char* who, const mpt_optim_tensor* tensors, int count, bool need0, bool need1, bool need2, bool need3) {
    MPT_REQUIRE(count >= 0, "%s: negative tensor count", who);
    MPT_REQUIRE(count == 0 || tensors, "%s: null tensor table", who);
    for (int i = 0; i < count; ++i) {
        const mpt_optim_tensor& x = tensors[i];
        MPT_REQUIRE(x.n >= 0, "%s: tensor %d has a negative size", who, i);
        if (x.n == 0) continue;
        MPT_REQUIRE(x.param && x.grad, "%s: tensor %d: null parameter or gradient", who, i);
        MPT_REQUIRE((!need0 || x.buf0) && (!need1 || x.buf1) && (!need2 || x.buf2) && (!need3 || x.buf3),
                    "%s: tensor %d: a state buffer this configuration needs is null", who, i);
    }
    return MPT_OK;
}

// ---- tensor scaling fused into the quantizer ------------------------------------------------------------------------
// compute_bias / scale / quantize of the reference layers (mptorch/quant/functional.py:39-59): per matrix (the last two
// dimensions) amax -> s = floor(log2(normal_max / amax)) - margin -> Q(x * 2^s).  Pass 1 takes the maxima, pass 2
// derives the exponent per matrix in double precision, as the reference does, scales and rounds.
__global__ void __launch_bounds__(kThreads) amax_rows_kernel(const float* __restrict__ x, int64_t per_matrix, uint32_t* __restrict__ amax_bits) {
    const float* base = x + (int64_t)blockIdx.y * per_matrix;
    uint32_t m = 0u;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < per_matrix; i += (int64_t)gridDim.x * kThreads) {
        const uint32_t a = __float_as_uint(base[i]) & 0x7FFFFFFFu;
        m = max(m, a);               // NaN patterns order above infinity: a NaN anywhere makes the maximum a NaN, as torch's amax
    }
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + blockIdx.y, m);
}

__global__ void zero_u32_kernel(uint32_t* p, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 0u;
}

// floor(log2(normal_max / amax)) - margin in double precision, then 2^s as the reference's torch.pow(2.0, s) yields it
__device__ __forceinline__ float scale_exponent(uint32_t amax_bits, double normal_max, int margin) {
    const double amax = (double)__uint_as_float(amax_bits);
    return (float)floor(log2(normal_max / amax)) - (float)margin;
}

__global__ void __launch_bounds__(kThreads) scale_quantize_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t per_matrix,
                                                                  const uint32_t* __restrict__ amax_bits, double normal_max, int margin,
                                                                  float* __restrict__ scale_out, Rounder q) {
    const float s = scale_exponent(amax_bits[blockIdx.y], normal_max, margin);
    if (scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) scale_out[blockIdx.y] = s;
    const float f = powf(2.0f, s);    // the reference's torch.pow(2.0, s); inf / 0 / NaN exponents flow through the same way
    const float* xi = x + (int64_t)blockIdx.y * per_matrix;
    float* oi = out + (int64_t)blockIdx.y * per_matrix;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < per_matrix; i += (int64_t)gridDim.x * kThreads)
        oi[i] = q(mul_rn(xi[i], f));
}

}  // namespace
}  // namespace mpt

using namespace mpt;

extern "C" {

int mpt_qsgd_step(const mpt_optim_tensor* tensors, int count, float lr, float momentum, float one_minus_dampening,
                  float weight_decay, int nesterov, int compensated, int momentum_quant, int man_mom, int exp_mom, int acc_quant,
                  int man_acc, int exp_acc, int subnormals, int saturate, void* stream) {
    const char* who = "qsgd_step";
    MPT_REQUIRE(!momentum_quant || valid_format(man_mom, exp_mom), "%s: unsupported momentum format", who);
    MPT_REQUIRE(!acc_quant || valid_format(man_acc, exp_acc), "%s: unsupported accumulator format", who);
    const bool need_m = momentum != 0.0f, need_c = compensated != 0;
    int rc = check_tensors(who, tensors, count, need_m, need_c, false, false);
    if (rc) return rc;
    SgdArgs a;
    a.lr = lr; a.neg_lr = -lr; a.momentum = momentum; a.one_minus_dampening = one_minus_dampening; a.weight_decay = weight_decay;
    a.nesterov = nesterov != 0; a.compensated = compensated != 0;
    a.has_momentum_quant = momentum_quant != 0; a.has_acc_quant = acc_quant != 0;
    a.qm = make_rounder(momentum_quant, man_mom, exp_mom, subnormals, saturate);
    a.qa = make_rounder(acc_quant, man_acc, exp_acc, subnormals, saturate);
    const bool line = a.qm.mode <= 1 && a.qa.mode <= 1;
    const bool ns = (a.qm.mode == 0 || a.qm.mode == 3) && (a.qa.mode == 0 || a.qa.mode == 3) && !line;
    return launch_optim(tensors, count, a, line ? qsgd_kernel<true> : (ns ? qsgd_kernel<true, true> : qsgd_kernel<false>), need_m, need_c, false, false, as_stream(stream), who);
}

int mpt_qadamw_step(const mpt_optim_tensor* tensors, int count, float beta1, float beta2, float one_minus_beta1,
                    float one_minus_beta2, float inv_sqrt_bias_correction2, float eps, float step_size, int amsgrad, int compensated,
                    int momentum_quant, int man_mom, int exp_mom, int acc_quant, int man_acc, int exp_acc, int subnormals,
                    int saturate, void* stream) {
    const char* who = "qadamw_step";
    MPT_REQUIRE(!momentum_quant || valid_format(man_mom, exp_mom), "%s: unsupported moment format", who);
    MPT_REQUIRE(!acc_quant || valid_format(man_acc, exp_acc), "%s: unsupported accumulator format", who);
    int rc = check_tensors(who, tensors, count, true, true, compensated != 0, amsgrad != 0);
    if (rc) return rc;
    AdamArgs a;
    a.beta1 = beta1; a.beta2 = beta2; a.one_minus_beta1 = one_minus_beta1; a.one_minus_beta2 = one_minus_beta2;
    a.inv_sqrt_bc2 = inv_sqrt_bias_correction2; a.eps = eps; a.step_size = step_size; a.neg_step_size = -step_size;
    a.amsgrad = amsgrad != 0; a.compensated = compensated != 0;
    a.has_momentum_quant = momentum_quant != 0; a.has_acc_quant = acc_quant != 0;
    a.qm = make_rounder(momentum_quant, man_mom, exp_mom, subnormals, saturate);
    a.qa = make_rounder(acc_quant, man_acc, exp_acc, subnormals, saturate);
    const bool line = a.qm.mode <= 1 && a.qa.mode <= 1;
    const bool ns = (a.qm.mode == 0 || a.qm.mode == 3) && (a.qa.mode == 0 || a.qa.mode == 3) && !line;
    return launch_optim(tensors, count, a, line ? qadamw_kernel<true> : (ns ? qadamw_kernel<true, true> : qadamw_kernel<false>), true, true, compensated != 0, amsgrad != 0, as_stream(stream), who);
}

size_t mpt_scale_quantize_workspace_bytes(int64_t matrices) { return sizeof(uint32_t) * (size_t)(matrices < 1 ? 1 : matrices); }

int mpt_scale_quantize(const float* in, float* out, int64_t matrices, int64_t per_matrix, double normal_max, int margin, int quantize,
                       int man, int exp, int subnormals, int saturate, float* scale_out, void* workspace, size_t workspace_bytes,
                       void* stream) {
    const char* who = "scale_quantize";
    MPT_REQUIRE(matrices >= 0 && per_matrix >= 0, "%s: negative extent", who);
    if (matrices == 0 || per_matrix == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "%s: null pointer", who);
    MPT_REQUIRE(matrices <= 65535, "%s: more than 65535 matrices", who);
    MPT_REQUIRE(!quantize || valid_format(man, exp), "%s: unsupported format", who);
    MPT_REQUIRE(workspace && workspace_bytes >= sizeof(uint32_t) * (size_t)matrices, "%s: workspace of %zu bytes needed", who,
                sizeof(uint32_t) * (size_t)matrices);
    cudaStream_t st = as_stream(stream);
    uint32_t* amax = static_cast<uint32_t*>(workspace);
    zero_u32_kernel<<<(unsigned)((matrices + 255) / 256), 256, 0, st>>>(amax, matrices);
    int64_t gx = (per_matrix + kThreads * 4 - 1) / (kThreads * 4);
    const int64_t cap = ((int64_t)sm_count() * 16 + matrices - 1) / matrices;
    if (gx > cap) gx = cap;
    if (gx < 1) gx = 1;
    amax_rows_kernel<<<dim3((unsigned)gx, (unsigned)matrices), kThreads, 0, st>>>(in, per_matrix, amax);
    scale_quantize_kernel<<<dim3((unsigned)gx, (unsigned)matrices), kThreads, 0, st>>>(in, out, per_matrix, amax, normal_max, margin, scale_out,
                                                                                 make_rounder(quantize, man, exp, subnormals, saturate));
    return check_launch(who);
}

}
