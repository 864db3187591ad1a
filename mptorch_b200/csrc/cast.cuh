// Device-side rounding primitives for simulated low-precision arithmetic.
//
// Two families live here:
//   * exact casters (`cast_fp_nearest`, `cast_fp_truncate`, `cast_fp_stochastic`,
//     `cast_binary8`, `cast_superfp`): complete restatements of the reference
//     semantics (mptorch quant_cuda/fp_kernel.cu:12-129, binary8_kernel.cu:11-276,
//     superfp_kernel.cu:12-68, bit_helper.cu), valid for every input pattern and
//     every format, including the reference's corner-case behaviour.
//   * the "magic add" fast path (`FastRn`): round-to-nearest-even on the FP32 pipe,
//     bit-identical to the exact caster on the value range its caller guarantees.
#pragma once
#include <cfenv>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cuda_runtime.h>

namespace mpt {

// Every caster is __host__ __device__ so that the identical source can be swept on the CPU
// against the oracle (tests/host_cast_check.cu); the library only ever runs the device side.
#define MPT_HD __host__ __device__ __forceinline__

MPT_HD uint32_t f2u(float x) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(x);
#else
    uint32_t u; memcpy(&u, &x, 4); return u;
#endif
}
MPT_HD float u2f(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float x; memcpy(&x, &u, 4); return x;
#endif
}
// fp32 operations that must never be contracted or reassociated
MPT_HD float fma_rn(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return __fmaf_rn(a, b, c);
#else
    return fmaf(a, b, c);
#endif
}
// fused multiply-add rounded toward zero (host side: through the floating-point environment)
MPT_HD float fma_rz(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return __fmaf_rz(a, b, c);
#else
    const int old = fegetround();
    fesetround(FE_TOWARDZERO);
    volatile float r = fmaf(a, b, c);
    fesetround(old);
    return r;
#endif
}
MPT_HD float add_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fadd_rn(a, b);
#else
    volatile float r = a + b; return r;
#endif
}
MPT_HD float mul_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fmul_rn(a, b);
#else
    volatile float r = a * b; return r;
#endif
}

// Format descriptor for IEEE-like (exp, man) targets; derived fields are filled on the host.
struct FpFmt {
    int man;         // mantissa bits kept (0..23)
    int exp;         // exponent bits (1..8)
    int min_exp;     // smallest normal exponent: 2 - 2^(exp-1)
    int max_store;   // biased fp32 exponent of the largest binade: 2^(exp-1) - 1 + 127
    int sub;         // subnormals supported
    int sat;         // saturate to max finite instead of overflowing to inf
};

__host__ __device__ inline FpFmt make_fmt(int man, int exp, int sub, int sat) {
    FpFmt f;
    f.man = man; f.exp = exp; f.sub = sub; f.sat = sat;
    f.min_exp = 2 - (1 << (exp - 1));
    f.max_store = (1 << (exp - 1)) - 1 + 127;
    return f;
}

MPT_HD uint32_t low_mask(int nbits) {       // nbits in 0..32
    return nbits >= 32 ? 0xFFFFFFFFu : ((1u << nbits) - 1u);
}

// Round the fp32 pattern t to m mantissa bits, nearest-even; m in -1..23.
// With m <= 0 at most 23 bits are cleared (cap23), so a tie moves away from zero; the
// binary8 P=1 format lifts that cap and resolves the tie on the exponent's low bit.
MPT_HD uint32_t rne_bits(uint32_t t, int m, bool cap23 = true) {
    if (m >= 23) return t;
    const int drop = 23 - m;                       // 1..24 bits to discard
    const uint32_t half = 1u << (drop - 1);
    if (m >= 1 || !cap23) {
        // classic integer RNE: add (half - 1) plus the parity of the kept part
        const uint32_t odd = (t >> drop) & 1u;
        return (t + (half - 1u) + odd) & ~low_mask(drop);
    }
    return (t + half) & ~0x7FFFFFu;
}

MPT_HD uint32_t max_finite_bits(const FpFmt& f, uint32_t sign) {
    const uint32_t man_field = (0x7FFFFFu >> (23 - f.man)) << (23 - f.man);
    return sign | ((uint32_t)f.max_store << 23) | man_field;
}

// After rounding in the subnormal range: anything that landed below the smallest
// subnormal's binade is bumped up one binade (if adjacent) or flushed.
MPT_HD uint32_t settle_subnormal(const FpFmt& f, uint32_t t, uint32_t q) {
    if (q == 0u) return 0u;
    const int qe = (int)((q << 1) >> 24);
    const int floor_store = f.min_exp - f.man + 127;
    if (qe < floor_store) {
        if (qe != floor_store - 1) return 0u;
        q = (q + 0x00800000u) | (t & 0x80000000u);
    }
    return q;
}

// After rounding in the normal range: overflow to inf / max finite; values below the
// smallest normal (only reachable without subnormals) snap to it or to signed zero.
MPT_HD uint32_t settle_normal(const FpFmt& f, uint32_t t, uint32_t q) {
    if (q == 0u) return 0u;
    const int qe = (int)((q << 1) >> 24);
    const uint32_t sign = t & 0x80000000u;
    const int min_store = f.min_exp + 127;
    if (qe > f.max_store) return f.sat ? max_finite_bits(f, sign) : (sign | 0x7F800000u);
    if (qe < min_store) {
        const bool up = (qe == min_store - 1) && ((t & 0x7FFFFFu) > 0x400000u);
        return (up ? ((uint32_t)min_store << 23) : 0u) | sign;
    }
    return q;
}

template <bool TRUNC>
MPT_HD float cast_fp_exact(float x, const FpFmt& f) {
    if (f.man >= 23 && f.exp >= 8) return x;
    const uint32_t t = f2u(x);
    const int E = (int)((t << 1) >> 24) - 127;
    if (f.sub && E < f.min_exp) {
        const int d = f.man - (f.min_exp - E);       // mantissa bits left in this binade
        uint32_t q;
        if (TRUNC) q = (d >= 0) ? (t & ~low_mask(23 - d)) : 0u;
        else {
            const bool keep = (d >= 0) || (d == -1 && (t << 9) != 0u);
            q = keep ? rne_bits(t, d) : 0u;
        }
        return u2f(settle_subnormal(f, t, q));
    }
    if (E == 128) return x;
    const uint32_t q = TRUNC ? (t & ~low_mask(23 - f.man)) : rne_bits(t, f.man);
    return u2f(settle_normal(f, t, q));
}

MPT_HD float cast_fp_nearest(float x, const FpFmt& f) { return cast_fp_exact<false>(x, f); }
MPT_HD float cast_fp_truncate(float x, const FpFmt& f) { return cast_fp_exact<true>(x, f); }

// Stochastic rounding with an explicit 32-bit random word.  No NaN/inf early-out exists on
// this path in the reference: the exponent clip decides.
MPT_HD float cast_fp_stochastic(float x, uint32_t r, int rbits, const FpFmt& f) {
    const uint32_t t = f2u(x);
    const int E = (int)((t << 1) >> 24) - 127;
    r &= 0x7FFFFFu;
    const int sh = 23 - f.man - rbits - 1;           // the reference clears this single bit
    if (sh >= 0 && sh <= 31) r &= ~(1u << sh);
    const uint32_t mask = low_mask(23 - f.man);
    if (f.sub && E < f.min_exp) {
        // lift into the smallest normal binade, round there, and come back down
        const float lift = u2f(((uint32_t)(127 + f.min_exp) << 23) | (t & 0x80000000u));
        const uint32_t v = f2u(add_rn(x, lift));
        const uint32_t q = (v + (r & mask)) & ~mask;
        return add_rn(u2f(q), -lift);
    }
    uint32_t q = (t + (r & mask)) & ~mask;
    if (q == 0u) return 0.0f;
    const int qe = (int)((q << 1) >> 24);
    const uint32_t sign = t & 0x80000000u;
    const int min_store = f.min_exp + 127;
    if (qe > f.max_store) q = f.sat ? max_finite_bits(f, sign) : (sign | 0x7F800000u);
    else if (qe < min_store) {
        const uint32_t middle = (uint32_t)(min_store - 1) << 23;
        q = ((q & 0x7FFFFFFFu) > middle) ? (sign | ((uint32_t)min_store << 23)) : 0u;
    }
    return u2f(q);
}

// ---- P3109 binary8 ------------------------------------------------------------------
enum : int { B8_INFTY = 0, B8_MAXFLOAT = 1, B8_MAXFLOAT2 = 2 };
enum : int { RND_NEAREST = 0, RND_STOCHASTIC = 1, RND_TRUNCATE = 2 };

MPT_HD uint32_t binary8_settle(int exp_bits, int man_bits, uint32_t t, uint32_t q,
                                                   int policy, bool sub) {
    if (q == 0u) return 0u;
    const uint32_t qman = q & 0x7FFFFFu;
    const uint32_t sign = t & 0x80000000u;
    const uint32_t ones = (1u << man_bits) - 1u;
    const int up = 23 - man_bits;
    uint32_t top_man = (ones & ~1u) << up;           // all-ones pattern is reserved
    int reserve_exp = 0;
    if (policy == B8_MAXFLOAT2) {
        if (exp_bits + man_bits == 7) top_man = ones << up;
    } else if (exp_bits == 8) {
        reserve_exp = 1;
    } else if (exp_bits == 7 && man_bits == 1) {
        reserve_exp = 1; top_man = ones << up;
    } else if (exp_bits + man_bits == 8) {
        top_man = (ones - 2u) << up;                 // wraps for man_bits < 2, as the reference does
    }
    const int qe = (int)((q << 1) >> 24);
    const int hi = (1 << (exp_bits - 1)) - 1 + 127 - reserve_exp;
    const int lo = 127 - ((1 << (exp_bits - 1)) - 1) + (man_bits == 0 ? 1 : 0) - (sub ? 0 : 1);
    if (qe > hi || (qe == hi && qman > top_man)) {
        if (policy == B8_INFTY) return sign | 0x7F800000u;
        q = sign | ((uint32_t)hi << 23) | top_man;
    }
    const uint32_t unit = 1u << up;
    if (qe < lo || (qe == lo && qman < unit)) {      // decided on the pre-overflow fields
        const uint32_t mag = t & 0x7FFFFFFFu;
        if (sub) {
            if (lo - qe > man_bits) {
                const int tiny = lo - man_bits;
                q = (mag > ((uint32_t)(tiny - 1) << 23)) ? (sign | ((uint32_t)tiny << 23)) : 0u;
            }
        } else {
            const uint32_t floor_num = ((uint32_t)lo << 23) | unit;
            const uint32_t mid = ((uint32_t)(lo - 1) << 23) | unit;
            if (mag > mid) return sign | floor_num;
            q = 0u;
        }
    }
    return q;
}

MPT_HD float cast_binary8(float x, int P, bool is_signed, int policy, bool sub,
                                              int mode, uint32_t r, int prng_bits) {
    if (!is_signed && x < 0.0f) return u2f(0x7FC00000u);   // NaN
    const uint32_t t = f2u(x);
    const int E = (int)((t << 1) >> 24) - 127;
    const uint32_t tman = t & 0x7FFFFFu;
    if (E == 128 && (tman != 0u || policy == B8_INFTY)) return x;
    const int man = P - 1;
    // the unsigned truncating cast keeps the signed exponent width, as the reference does
    const int exp = (is_signed || mode == RND_TRUNCATE) ? 8 - P : 9 - P;
    int shift = 0;
    if (sub) {
        const int max_exp = (1 << (exp - 1)) - 1;
        const int min_exp = (P == 1 ? 1 : 0) - max_exp;
        if (E < min_exp && min_exp - E <= man) shift = min_exp - E;
    }
    const int mb = man - shift;
    uint32_t q;
    if (mode == RND_NEAREST) q = rne_bits(t, mb, P != 1);
    else if (mode == RND_TRUNCATE) q = t & ~low_mask(23 - mb);
    else {
        r &= 0x7FFFFFu;
        const int sh = 23 - man - prng_bits - 1;
        if (sh >= 0 && sh <= 31) r &= ~(1u << sh);
        const uint32_t mask = low_mask(23 - mb);
        q = (t + (r & mask)) & ~mask;
    }
    return u2f(binary8_settle(exp, man, t, q, policy, sub));
}

// ---- supernormal floats -------------------------------------------------------------------
MPT_HD float cast_superfp(float x, int man, int exp, int bl, int bu, bool sat) {
    const uint32_t t = f2u(x);
    const int E = (int)((t << 1) >> 24) - 127;
    const int lo = 1 - (1 << (exp - 1)) + (bl - 1);
    const int hi = ((1 << (exp - 1)) - 2) - (bu - 1);
    const uint32_t sign = t & 0x80000000u;
    const uint32_t pow2 = (t + 0x400000u) & ~0x7FFFFFu;   // nearest power of two in the log sense
    if (E < lo) return (E < lo - bl * (1 << man) + 1) ? 0.0f : u2f(pow2);
    if (E > hi) {
        const int top = hi + bu * (1 << man);
        const uint32_t topnum = sign | ((uint32_t)(top + 127) << 23);
        if (E == 128) return (sat && (t & 0x7FFFFFFFu) == 0x7F800000u) ? u2f(topnum) : x;
        if (E >= top - 1 + (sat ? 1 : 0)) {
            if (sat) return u2f(topnum);
            if ((t << 9) == 0u && E == top - 1) return x;
            return u2f(sign | 0x7F800000u);
        }
        return u2f(pow2);
    }
    return u2f(rne_bits(t, man));
}

// ---- one descriptor for the three nearest-rounding format families ---------------------------------
// The reference instantiates its GEMM, softmax and layernorm templates once per family (float, supernormal
// float, binary8); here the exact arithmetic paths take this descriptor instead.
enum : int { FMT_FLOAT = 0, FMT_SUPERFP = 1, FMT_BINARY8 = 2 };
struct AnyFmt {
    int kind;
    FpFmt fp;                   // float: all fields; superfp: man, exp, sat; binary8: sub
    int bl, bu;                 // superfp binades
    int P, is_signed, policy;   // binary8
};
MPT_HD float cast_any(float x, const AnyFmt& f) {
    if (f.kind == FMT_SUPERFP) return cast_superfp(x, f.fp.man, f.fp.exp, f.bl, f.bu, f.fp.sat != 0);
    if (f.kind == FMT_BINARY8) return cast_binary8(x, f.P, f.is_signed != 0, f.policy, f.fp.sub != 0, RND_NEAREST, 0u, 0);
    return cast_fp_nearest(x, f.fp);
}
__host__ __device__ inline AnyFmt any_float(const FpFmt& f) {
    AnyFmt a;
    a.kind = FMT_FLOAT; a.fp = f; a.bl = a.bu = 1; a.P = 1; a.is_signed = 1; a.policy = 0;
    return a;
}

// ---- fast round-to-nearest-even on the FP32 pipe ---------------------------------------------
// For a finite x whose rounded value stays below the format's overflow threshold, and a
// format with subnormals and man <= 21:
//     q = 2^(max(E_x, min_exp) - man)            (the rounding quantum)
//     C = 1.5 * 2^23 * q
//     round(x) = (x + C) - C                      (both adds in fp32 round-to-nearest-even)
// x + C lies in [2^23 q, 2^24 q) where one ulp equals q, and C is an even multiple of q, so
// the hardware's tie-to-even coincides with tie-to-even on x/q; the subtraction is exact.
// Zero results come out as +0, as in the reference's subnormal branch.  The two adds are
// issued as FFMA(m, K, x) and FFMA(m, -K, y) with m = 2^max(E_x, min_exp) taken from the
// exponent field, so the cast costs 2 ALU + 2 FMA instructions.
struct FastRn {
    int   min_e_bits;   // (min_exp + 127) << 23
    float k;            // 1.5 * 2^(23 - man)
    __host__ __device__ static FastRn make(const FpFmt& f) {
        FastRn r;
        r.min_e_bits = (f.min_exp + 127) << 23;
        union { uint32_t u; float v; } c;
        c.u = ((uint32_t)(127 + 23 - f.man) << 23) | 0x400000u;
        r.k = c.v;
        return r;
    }
    MPT_HD float operator()(float x) const {
        const int e = (int)(f2u(x) & 0x7F800000u);
        const float m = u2f((uint32_t)(e > min_e_bits ? e : min_e_bits));
        const float y = fma_rn(m, k, x);
        return fma_rn(m, -k, y);
    }
};

// The same rounding for a format WITHOUT subnormals (the reference's default for FloatingPoint), for a finite x that is
// zero or a normal fp32 number and whose rounded value stays below the format's overflow threshold.  The reference
// rounds every value at its own exponent (no fixed quantum below the smallest normal) and then settles what landed
// below 2^min_exp (bit_helper.cu:193-198): the smallest normal value if the ROUNDED value is in the binade just below
// it and the ORIGINAL mantissa field exceeds one half, zero otherwise, with the sign of the input either way.  Here: the
// FP-pipe rounding without the exponent clamp, then that rule on the bits with two compares and two selects.
MPT_HD float nosub_settle(uint32_t min_norm, uint32_t t, float q) {
    const uint32_t a = f2u(q) & 0x7FFFFFFFu;
    const bool up = a >= min_norm - 0x00800000u && (t & 0x007FFFFFu) > 0x00400000u;
    const uint32_t settled = (t & 0x80000000u) | (up ? min_norm : 0u);
    return a < min_norm ? u2f(settled) : q;
}
MPT_HD float fast_rn_nosub(const FastRn& r, float x) {
    const uint32_t t = f2u(x);
    const float m = u2f(t & 0x7F800000u);
    const float y = fma_rn(m, r.k, x);
    const float q = fma_rn(m, -r.k, y);
    return nosub_settle((uint32_t)r.min_e_bits, t, q);                 // min_e_bits: the bit pattern of 2^min_exp
}
// The same function for roundings whose result is rarely a nonzero value below the smallest normal one (a sum of
// rounded products: it is zero, or at least one quantum of the product format): the settling rule sits behind a
// branch (a call, so that the compiler does not turn it back into selects), which leaves three integer instructions
// on the common path instead of nine.  A zero result (from a zero input only: a normal value rounded at its own exponent
// is never zero) needs no settling beyond the input's sign, which the magic addition drops and one OR puts back.
#ifdef __CUDA_ARCH__
static __device__ __noinline__ float nosub_settle_cold(uint32_t min_norm, uint32_t t, float q) { return nosub_settle(min_norm, t, q); }
#endif
MPT_HD float fast_rn_nosub_rare(const FastRn& r, float x) {
    const uint32_t t = f2u(x);
    const float m = u2f(t & 0x7F800000u);
    const float y = fma_rn(m, r.k, x);
    const float q = fma_rn(m, -r.k, y);
    const uint32_t qb = f2u(q) | (t & 0x80000000u);
    if (qb + qb - 1u < 2u * (uint32_t)r.min_e_bits - 1u) {             // 0 < |q| < 2^min_exp
#ifdef __CUDA_ARCH__
        return nosub_settle_cold((uint32_t)r.min_e_bits, t, q);
#else
        return nosub_settle((uint32_t)r.min_e_bits, t, q);
#endif
    }
    return u2f(qb);
}

// Third form, with no branch at all: the rounding without the settling rule, and a flag that the result was a nonzero
// value below the smallest normal one, in which case the caller discards what it computed and redoes it on the exact
// casters.  For the sum roundings of the GEMM's inner sums, which start from zero every eight steps: nothing has to be
// saved to redo a group, and straight-line code lets the compiler interleave the thread's 32 independent chains.
MPT_HD float fast_rn_nosub_flag(const FastRn& r, float x, uint32_t& rare) {
    const uint32_t t = f2u(x);
    const float m = u2f(t & 0x7F800000u);
    const float y = fma_rn(m, r.k, x);
    const float q = fma_rn(m, -r.k, y);
    const uint32_t qb = f2u(q) | (t & 0x80000000u);                    // a zero keeps the input's sign
    rare |= (qb + qb - 1u < 2u * (uint32_t)r.min_e_bits - 1u) ? 1u : 0u;
    return u2f(qb);
}

// a / b rounded to nearest even, given r = RN(1 / b) (the correctly rounded reciprocal): the quotient estimate
// a * r is within one ulp, the remainder a - b * q is exact in one FMA, and the correction FMA lands on the correctly
// rounded quotient (Markstein's correction step).  Exact while 1 / b, the quotient and the remainder are normal
// numbers: callers keep 2^-20 <= |b| <= 2^20 and |a| either zero or in [2^-83, 2^64).
MPT_HD float div_with_rcp(float a, float b, float r) {
    const float q = mul_rn(a, r);
    const float rem = fma_rn(-b, q, a);
    return fma_rn(rem, r, q);
}

// Largest unbiased exponent E such that every |x| < 2^(E+1) is safe on the fast path of format
// f: the top binade is excluded because its upper part rounds up into overflow, and
// C = 1.5 * 2^(E - man + 23) must stay finite.
__host__ __device__ inline int fast_rn_exp_limit(const FpFmt& f) {
    const int top = f.max_store - 127 - 1;
    const int magic = 103 + f.man;
    return top < magic ? top : magic;
}

__host__ __device__ inline bool fast_rn_supported(const FpFmt& f) {
    // exp == 1 is degenerate (its largest binade lies below its smallest normal one): exact caster only
    return f.sub && f.man <= 21 && f.exp >= 2;
}


// Round-to-nearest-even over the WHOLE fp32 input domain, built on FastRn: the elementwise
// quantizer's inner step.  Finite inputs below the overflow threshold take the 4-instruction
// FP-pipe rounding; overflow, infinities and NaN are patched in with two compares and two selects
// (the FastRn result computed for them is simply discarded).  Only formats with an 8-bit exponent
// keep a data-dependent branch to the exact caster, for magnitudes where 1.5 * 2^23 * quantum would
// overflow fp32 and for zero and fp32-denormal inputs (which the reference rounds one bit coarser,
// keeping the sign of a negative zero).
struct FullRn {
    FastRn fast;
    FpFmt fmt;
    uint32_t ovf_from;    // smallest |x| pattern whose rounding overflows the format
    uint32_t ovf_value;   // what overflow yields (without sign): max finite, or infinity
    uint32_t exact_from;  // 8-bit-exponent formats: smallest |x| pattern that must take the exact caster
    __host__ __device__ static FullRn make(const FpFmt& f) {
        FullRn r;
        r.fast = FastRn::make(f);
        r.fmt = f;
        const uint32_t maxf = ((uint32_t)f.max_store << 23) | ((0x7FFFFFu >> (23 - f.man)) << (23 - f.man));
        r.ovf_from = maxf + (1u << (22 - f.man));       // max finite plus half a quantum: a tie rounds up
        r.ovf_value = f.sat ? maxf : 0x7F800000u;
        r.exact_from = (f.exp == 8) ? ((uint32_t)(103 + f.man + 1 + 127) << 23) : 0xFFFFFFFFu;
        return r;
    }
    MPT_HD float operator()(float x) const {
        const uint32_t t = f2u(x);
        const uint32_t a = t & 0x7FFFFFFFu;
        if (fmt.exp == 8 && (a >= exact_from || a < 0x00800000u)) return cast_fp_nearest(x, fmt);
        float y = fast(x);
        const float over = (a >= 0x7F800000u) ? x : u2f((t & 0x80000000u) | ovf_value);
        return (a >= ovf_from) ? over : y;
    }
    // The same for formats with fewer than 8 exponent bits, without the test for them: straight-line code (no branch),
    // so that a compiler can interleave several independent roundings.
    MPT_HD float line(float x) const {
        const uint32_t t = f2u(x);
        const uint32_t a = t & 0x7FFFFFFFu;
        const float y = fast(x);
        const float over = (a >= 0x7F800000u) ? x : u2f((t & 0x80000000u) | ovf_value);
        return (a >= ovf_from) ? over : y;
    }
};


// Truncation toward zero over the whole fp32 input domain, the counterpart of FullRn: the magic
// constant carries the sign of x and the first FFMA rounds toward zero, so |x| + C is cut down to a
// multiple of the quantum; the second FFMA (exact) removes C again.
struct FullRz {
    FastRn fast;
    FpFmt fmt;
    uint32_t ovf_from, ovf_value, exact_from;
    __host__ __device__ static FullRz make(const FpFmt& f) {
        FullRz r;
        r.fast = FastRn::make(f);
        r.fmt = f;
        const uint32_t maxf = ((uint32_t)f.max_store << 23) | ((0x7FFFFFu >> (23 - f.man)) << (23 - f.man));
        r.ovf_from = (uint32_t)(f.max_store + 1) << 23;   // truncation never rounds up into overflow
        r.ovf_value = f.sat ? maxf : 0x7F800000u;
        r.exact_from = (f.exp == 8) ? ((uint32_t)(103 + f.man + 1 + 127) << 23) : 0xFFFFFFFFu;
        return r;
    }
    MPT_HD float operator()(float x) const {
        const uint32_t t = f2u(x);
        const uint32_t a = t & 0x7FFFFFFFu;
        if (fmt.exp == 8 && (a >= exact_from || a < 0x00800000u)) return cast_fp_truncate(x, fmt);
        const int e = (int)(t & 0x7F800000u);
        const float m = u2f((uint32_t)(e > fast.min_e_bits ? e : fast.min_e_bits) | (t & 0x80000000u));
        const float y = fma_rz(m, fast.k, x);
        const float r = fma_rn(m, -fast.k, y);
        // a negative input that truncates to zero leaves -0 here; the reference's subnormal branch returns +0
        const float rz = (f2u(r) == 0x80000000u) ? 0.0f : r;
        const float over = (a >= 0x7F800000u) ? x : u2f((t & 0x80000000u) | ovf_value);
        return (a >= ovf_from) ? over : rz;
    }
};

// Stochastic rounding with an explicit random word over the whole input domain, for formats with
// subnormals: the two branches of the exact caster (lift sub-minimum inputs into the smallest normal
// binade, round there, come back) collapse into one straight line with a conditional lift of zero.
struct FullSr {
    FpFmt fmt;
    uint32_t rmask;       // random bits that take part: low (23 - man) bits, minus the one bit the reference clears
    uint32_t keep;        // ~((1 << (23 - man)) - 1)
    uint32_t min_norm;    // bit pattern of the smallest normal value 2^min_exp
    uint32_t ovf_from;    // (max_store + 1) << 23
    uint32_t ovf_value;
    int rbits;
    __host__ __device__ static bool supported(const FpFmt& f) { return f.sub && f.exp >= 2; }
    __host__ __device__ static FullSr make(const FpFmt& f, int rbits) {
        FullSr r;
        r.fmt = f;
        r.rbits = rbits;
        const uint32_t low = (f.man >= 23) ? 0u : ((1u << (23 - f.man)) - 1u);
        r.keep = ~low;
        uint32_t rm = 0x7FFFFFu & low;
        const int sh = 23 - f.man - rbits - 1;
        if (sh >= 0 && sh <= 31) rm &= ~(1u << sh);
        r.rmask = rm;
        r.min_norm = (uint32_t)(f.min_exp + 127) << 23;
        r.ovf_from = (uint32_t)(f.max_store + 1) << 23;
        r.ovf_value = f.sat ? (((uint32_t)f.max_store << 23) | ((0x7FFFFFu >> (23 - f.man)) << (23 - f.man))) : 0x7F800000u;
        return r;
    }
    MPT_HD float operator()(float x, uint32_t rnd) const {
        const uint32_t t = f2u(x);
        const uint32_t a = t & 0x7FFFFFFFu;
        const uint32_t sign = t & 0x80000000u;
        // NaN payloads can carry into the sign bit when the random word is added; the reference has no NaN
        // early-out on this path, so whatever its clip makes of the wrapped pattern is reproduced by the exact caster
        if (a > 0x7F800000u) return cast_fp_stochastic(x, rnd, rbits, fmt);
        const bool small = a < min_norm;
        const float lift = u2f(small ? (min_norm | sign) : 0u);
        const uint32_t v = small ? f2u(add_rn(x, lift)) : t;
        const uint32_t q = (v + (rnd & rmask)) & keep;
        const float r = small ? add_rn(u2f(q), -lift) : u2f(q);
        // the exponent clip of the normal branch: anything at or above 2^(max_exp+1), infinities and NaN included
        return (!small && (q & 0x7FFFFFFFu) >= ovf_from) ? u2f(sign | ovf_value) : r;
    }
};

// Round-to-nearest-even for P3109 binary8 (P >= 2, subnormals on) over the whole input domain, on the
// same FP-pipe rounding.  The format's largest finite value depends on signedness and overflow policy,
// so the overflow threshold is worked out on the host: the smallest |x| pattern that rounds above it.
struct FullRnB8 {
    FastRn fast;
    uint32_t ovf_from;    // smallest |x| pattern that rounds above the largest finite value
    uint32_t ovf_value;   // largest finite value, or infinity for the SATURATE_INFTY policy
    int is_signed, keep_inf;
    __host__ __device__ static bool supported(int P, bool sub) { return sub && P >= 2 && P <= 7; }
    __host__ __device__ static FullRnB8 make(int P, bool is_signed, int policy) {
        FullRnB8 r;
        const int man = P - 1, exp = is_signed ? 8 - P : 9 - P;
        const int max_exp = (1 << (exp - 1)) - 1;
        FpFmt f = make_fmt(man, 8, 1, 0);
        f.min_exp = -max_exp;                           // P >= 2
        r.fast = FastRn::make(f);
        const uint32_t ones = (1u << man) - 1u;
        const int up = 23 - man;
        uint32_t top_man = (ones & ~1u) << up;
        int reserve = 0;
        if (policy == B8_MAXFLOAT2) { if (exp + man == 7) top_man = ones << up; }
        else if (exp == 8) reserve = 1;
        else if (exp == 7 && man == 1) { reserve = 1; top_man = ones << up; }
        else if (exp + man == 8) top_man = (ones - 2u) << up;
        const uint32_t maxf = ((uint32_t)(max_exp + 127 - reserve) << 23) | top_man;
        const bool max_is_odd = ((top_man >> up) & 1u) != 0u;
        r.ovf_from = maxf + (1u << (up - 1)) + (max_is_odd ? 0u : 1u);   // a tie goes to the even neighbour
        r.ovf_value = policy == B8_INFTY ? 0x7F800000u : maxf;
        r.is_signed = is_signed;
        r.keep_inf = policy == B8_INFTY;
        return r;
    }
    MPT_HD float operator()(float x) const {
        const uint32_t t = f2u(x);
        const uint32_t a = t & 0x7FFFFFFFu;
        float y = fast(x);
        const bool passthrough = a > 0x7F800000u || (a == 0x7F800000u && keep_inf);
        const float over = passthrough ? x : u2f((t & 0x80000000u) | ovf_value);
        y = (a >= ovf_from) ? over : y;
        if (!is_signed && x < 0.0f) y = u2f(0x7FC00000u);
        return y;
    }
};

}  // namespace mpt
