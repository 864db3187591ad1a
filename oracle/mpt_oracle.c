/*
 * mpt_oracle.c -- CPU restatement of the simulated-arithmetic hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package links, loads or
 * calls this file; it exists so that the CUDA kernels can be compared, bit for
 * bit, with an independent scalar statement of the same arithmetic.
 *
 * Every function restates the algorithm of the reference implementation
 * (mptorch) and cites the reference file:line it follows.  The restatement is
 * pinned against the compiled, unmodified reference CPU extension
 * (oracle/_ref/quant_cpu) and against the reference's own known-answer test
 * vectors by tests/test_oracle_pins.py.
 *
 * Parity status per group:
 *   - float / binary8 / superfp casters, mm (sequential order), softmax and
 *     layernorm (sequential order): pinned against the reference CPU build.
 *   - "tile8" GEMM order and "tree64" reduction order restate the reference
 *     CUDA kernels; they are pinned by composing the (pinned) scalar casters
 *     in the order the CUDA source prescribes.
 *   - float truncate, MX (MXFP8/MXFP4) and NVFP4 block quantizers, and the
 *     counter-based stochastic GEMM: the reference has no implementation;
 *     PARITY UNPINNED (definitions frozen here).
 *
 * All integer arithmetic is uint32 with wrap-around, as in the reference.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* ------------------------------------------------------------------------- */
/* rounding primitives on fp32 bit patterns                                  */
/* ------------------------------------------------------------------------- */

/* Round-to-nearest-even of the fp32 pattern t to m mantissa bits.
 * reference: quant_cpu/bit_helper.cpp:42-50 (round_bitwise_nearest).
 * m ranges over -1..23.  The number of cleared bits is capped at 23, so with
 * m <= 0 an exact tie is rounded away from zero instead of to even.       */
static uint32_t rne_bits(uint32_t t, int m, int cap23)
{
    uint32_t keep_sh = (uint32_t)(8 + m);                 /* 7..31 */
    uint32_t down = (t << keep_sh) >> keep_sh;            /* discarded field (+1 bit) */
    uint32_t eps = (m <= 22) ? (1u << (22 - m)) : 0u;     /* half quantum; 1<<-1 reads as 0 */
    int clear = 23 - m + (down == eps ? 1 : 0);
    if (cap23 && clear > 23) clear = 23;
    uint32_t mask = (clear >= 32) ? 0xFFFFFFFFu : ((1u << clear) - 1u);
    return (t + eps) & ~mask;
}

/* reference: quant_cpu/bit_helper.cpp:18-28 (round_bitwise_stochastic). */
static uint32_t sr_bits(uint32_t t, uint32_t r, int m)
{
    uint32_t sh = (uint32_t)(23 - m);
    uint32_t mask = (sh >= 32) ? 0xFFFFFFFFu : ((1u << sh) - 1u);
    return (t + (r & mask)) & ~mask;
}

/* reference: bit_helper.cu:144-163 (clip_exponent_with_subnormals). */
static uint32_t clip_sub(int exp_bits, int man_bits, uint32_t t, uint32_t q)
{
    if (q == 0) return 0;
    int qe = (int)((q << 1) >> 24);
    int min_store = -((1 << (exp_bits - 1)) - 2) - man_bits + 127;
    if (qe < min_store) {
        uint32_t off = (qe == min_store - 1) ? 1u : 0u;
        q += off * (1u << 23);
        q |= t & 0x80000000u;
        q = off * q;
    }
    return q;
}

static uint32_t max_finite(int exp_bits, int man_bits, uint32_t sign)
{
    uint32_t max_store = (uint32_t)((1 << (exp_bits - 1)) - 1 + 127);
    uint32_t max_man = (0x7FFFFFu >> (23 - man_bits)) << (23 - man_bits);
    return sign | (max_store << 23) | max_man;
}

/* reference: bit_helper.cu:166-200 (clip_exponent_without_subnormals). */
static uint32_t clip_nosub(int exp_bits, int man_bits, uint32_t t, uint32_t q, int saturate)
{
    if (q == 0) return 0;
    int qe = (int)((q << 1) >> 24);
    int max_store = (1 << (exp_bits - 1)) - 1 + 127;
    int min_store = -((1 << (exp_bits - 1)) - 2) + 127;
    uint32_t sign = t & 0x80000000u;
    if (qe > max_store) {
        q = saturate ? max_finite(exp_bits, man_bits, sign) : (sign | 0x7F800000u);
    } else if (qe < min_store) {
        uint32_t off = (qe == min_store - 1) && ((t & 0x7FFFFFu) > (1u << 22));
        q = off * ((uint32_t)min_store << 23);
        q |= sign;
    }
    return q;
}

/* reference: bit_helper.cu:80-126 (clip_exponent, used by the stochastic cast). */
static uint32_t clip_sr(int exp_bits, int man_bits, uint32_t t, uint32_t q, int saturate)
{
    if (q == 0) return 0;
    int qe = (int)((q << 1) >> 24);
    int max_store = (1 << (exp_bits - 1)) - 1 + 127;
    int min_store = -((1 << (exp_bits - 1)) - 2) + 127;
    uint32_t sign = t & 0x80000000u;
    if (qe > max_store) {
        q = saturate ? max_finite(exp_bits, man_bits, sign) : (sign | 0x7F800000u);
    } else if (qe < min_store) {
        uint32_t min_num = (uint32_t)min_store << 23;
        uint32_t middle = (uint32_t)(min_store - 1) << 23;
        q = ((q & 0x7FFFFFFFu) > middle) ? (sign | min_num) : 0u;
    }
    return q;
}

/* ------------------------------------------------------------------------- */
/* scalar casters                                                            */
/* ------------------------------------------------------------------------- */

/* mode 0: round to nearest even; mode 2: truncate (toward zero).
 * nearest -- reference: quant_cpu/quant.cpp:389-435, quant_cuda/fp_kernel.cu:12-58.
 * truncate -- NO reference counterpart (parity unpinned): same control flow
 * with the mantissa rounding replaced by clearing the discarded bits, as the
 * reference's binary8 truncate does (binary8_kernel.cu:99-137).            */
static float cast_fp_rn_or_rz(float x, int man, int exp, int sub, int sat, int mode)
{
    if (man >= 23 && exp >= 8) return x;
    uint32_t t = f2u(x);
    int E = (int)((t << 1) >> 24) - 127;
    int min_exp = -((1 << (exp - 1)) - 2);
    if (sub && E < min_exp) {
        int d = man - (min_exp - E);
        uint32_t q;
        if (mode == 0) {
            int keep = (d > -1) || (d == -1 && (t << 9) != 0);
            q = keep ? rne_bits(t, d, 1) : 0u;
        } else {
            q = (d > -1) ? (t & ~((1u << (23 - d)) - 1u)) : 0u;
        }
        return u2f(clip_sub(exp, man, t, q));
    }
    if (E == 128) return x;
    uint32_t q = (mode == 0) ? rne_bits(t, man, 1)
                             : (t & ~(((man >= 23) ? 1u : (1u << (23 - man))) - 1u));
    return u2f(clip_nosub(exp, man, t, q, sat));
}

ORC_API float orc_cast_fp_nearest(float x, int man, int exp, int sub, int sat)
{
    return cast_fp_rn_or_rz(x, man, exp, sub, sat, 0);
}

ORC_API float orc_cast_fp_truncate(float x, int man, int exp, int sub, int sat)
{
    return cast_fp_rn_or_rz(x, man, exp, sub, sat, 2);
}

/* reference: quant_cuda/fp_kernel.cu:94-129 / quant_cpu/quant.cpp:352-387
 * (the overload taking rand_bits, the only one reachable from Python).
 * No NaN/inf early-out exists on this path; the clip decides.              */
ORC_API float orc_cast_fp_stochastic(float x, uint32_t r, int rbits, int man, int exp, int sub, int sat)
{
    uint32_t t = f2u(x);
    int E = (int)((t << 1) >> 24) - 127;
    int min_exp = -((1 << (exp - 1)) - 2);
    r = (r << 9) >> 9;
    int sh = 23 - man - rbits - 1;         /* `1 << a - 1` parses as 1 << (a - 1) */
    if (sh >= 0 && sh <= 31) r &= ~(1u << sh);
    if (sub && E < min_exp) {
        float shift = u2f(((uint32_t)(127 + min_exp) << 23) | (t & 0x80000000u));
        volatile float val = x + shift;
        uint32_t q = sr_bits(f2u(val), r, man);
        volatile float res = u2f(q) - shift;
        return res;
    }
    return u2f(clip_sr(exp, man, t, sr_bits(t, r, man), sat));
}

/* P3109 binary8.  policy: 0 SATURATE_INFTY, 1 SATURATE_MAXFLOAT, 2 SATURATE_MAXFLOAT2.
 * reference: quant_cuda/bit_helper.cu:203-306 (binary8_clip_exponent). */
static uint32_t b8_clip(int exp_bits, int man_bits, uint32_t t, uint32_t q, int policy, int sub)
{
    if (q == 0) return 0;
    uint32_t qman = q & 0x7FFFFFu;
    uint32_t sign = t & 0x80000000u;
    uint32_t all_man = ((1u << man_bits) - 1u);
    uint32_t max_man = (all_man & ~1u) << (23 - man_bits);
    int U = 0;
    if (exp_bits + man_bits == 7 && policy == 2) max_man = all_man << (23 - man_bits);
    if (policy != 2) {
        if (exp_bits == 8) U = 1;
        else if (exp_bits == 7 && man_bits == 1) { U = 1; max_man = all_man << (23 - man_bits); }
        else if (exp_bits + man_bits == 8) max_man = ((1u << man_bits) - 3u) << (23 - man_bits);
    }
    int qe = (int)((q << 1) >> 24);
    int max_store = (1 << (exp_bits - 1)) - 1 + 127 - U;
    int min_store = -((1 << (exp_bits - 1)) - 1) + 127 + (man_bits == 0 ? 1 : 0);
    if (!sub) min_store--;

    if (qe > max_store || (qe == max_store && qman > max_man)) {
        if (policy == 0) return sign | 0x7F800000u;
        q = sign | ((uint32_t)max_store << 23) | max_man;
    }
    /* the underflow test uses the pre-overflow exponent and mantissa */
    uint32_t min_man = 1u << (23 - man_bits);
    if (qe < min_store || (qe == min_store && qman < min_man)) {
        if (sub) {
            int shift = min_store - qe;
            int min_sub_exp = min_store - man_bits;
            uint32_t min_num = (uint32_t)min_sub_exp << 23;
            uint32_t middle = (uint32_t)(min_sub_exp - 1) << 23;
            if (shift <= man_bits) { /* keep */ }
            else if ((t & 0x7FFFFFFFu) > middle) q = sign | min_num;
            else q = 0;
        } else {
            uint32_t min_num = ((uint32_t)min_store << 23) | (1u << (23 - man_bits));
            uint32_t middle = ((uint32_t)(min_store - 1) << 23) | (1u << (23 - man_bits));
            if ((t & 0x7FFFFFFFu) > middle) return sign | min_num;
            q = 0;
        }
    }
    return q;
}

/* mode: 0 nearest, 1 stochastic, 2 truncate.
 * reference: quant_cuda/binary8_kernel.cu:11-276, quant_cpu/binary8.cpp:14-308. */
ORC_API float orc_cast_binary8(float x, int P, int is_signed, int policy, int sub,
                               int mode, uint32_t r, int prng_bits)
{
    if (!is_signed && x < 0) return NAN;
    uint32_t t = f2u(x);
    int E = (int)((t << 1) >> 24) - 127;
    uint32_t tman = t & 0x7FFFFFu;
    if (E == 128 && tman != 0) return x;
    if (policy == 0 && E == 128 && tman == 0) return x;
    int man = P - 1;
    /* the unsigned truncate cast uses the signed exponent width (binary8_kernel.cu:257) */
    int exp = (is_signed || mode == 2) ? 8 - P : 9 - P;
    int shift = 0;
    if (sub) {
        int max_exp = (1 << (exp - 1)) - 1;
        int min_exp = (P == 1 ? 1 : 0) - max_exp;
        if ((min_exp - E) <= man && E < min_exp) shift = min_exp - E;
    }
    int mb = man - shift;
    uint32_t q;
    if (mode == 0) {
        q = rne_bits(t, mb, P != 1);
    } else if (mode == 2) {
        uint32_t s = (uint32_t)(23 - mb);
        q = (s >= 32) ? 0u : ((t >> s) << s);
    } else {
        r = (r << 9) >> 9;
        int sh = 23 - man - prng_bits - 1;
        if (sh >= 0 && sh <= 31) r &= ~(1u << sh);
        q = sr_bits(t, r, mb);
    }
    return u2f(b8_clip(exp, man, t, q, policy, sub));
}

/* reference: quant_cuda/superfp_kernel.cu:12-68, quant_cpu/quant.cpp:464-542. */
ORC_API float orc_cast_superfp(float x, int man, int exp, int bl, int bu, int sat)
{
    uint32_t t = f2u(x);
    int E = (int)((t << 1) >> 24) - 127;
    int min_exp = 1 - (1 << (exp - 1)) + (bl - 1);
    int max_exp = ((1 << (exp - 1)) - 2) - (bu - 1);
    uint32_t sign = t & 0x80000000u;
    int top = max_exp + bu * (1 << man);
    if (E < min_exp) {
        if (E < min_exp - bl * (1 << man) + 1) return 0.0f;
        return u2f((t + (1u << 22)) & ~0x7FFFFFu);
    }
    if (E > max_exp) {
        uint32_t topnum = sign | ((uint32_t)(top + 127) << 23);
        if (E == 128) {
            if (sat && (t & 0x7FFFFFFFu) == 0x7F800000u) return u2f(topnum);
            return x;
        }
        if (E >= top - 1 + (sat ? 1 : 0)) {
            if (sat) return u2f(topnum);
            if ((t << 9) == 0u && E == top - 1) return x;
            return u2f(sign | 0x7F800000u);
        }
        return u2f((t + (1u << 22)) & ~0x7FFFFFu);
    }
    return u2f(rne_bits(t, man, 1));
}

/* ------------------------------------------------------------------------- */
/* elementwise array entry points                                            */
/* ------------------------------------------------------------------------- */

/* reference: quant_cpu/quant.cpp:577-591 (float_quantize_nearest host loop). */
ORC_API void orc_float_quantize(const float *a, float *o, int64_t n, int man, int exp,
                                int sub, int sat, int mode, const int32_t *rnd, int rbits)
{
    for (int64_t i = 0; i < n; ++i) {
        if (mode == 1) o[i] = orc_cast_fp_stochastic(a[i], (uint32_t)rnd[i], rbits, man, exp, sub, sat);
        else o[i] = cast_fp_rn_or_rz(a[i], man, exp, sub, sat, mode);
    }
}

ORC_API void orc_binary8_quantize(const float *a, float *o, int64_t n, int P, int is_signed,
                                  int policy, int sub, int mode, const int32_t *rnd, int prng_bits)
{
    for (int64_t i = 0; i < n; ++i)
        o[i] = orc_cast_binary8(a[i], P, is_signed, policy, sub, mode,
                                rnd ? (uint32_t)rnd[i] : 0u, prng_bits);
}

ORC_API void orc_superfp_quantize(const float *a, float *o, int64_t n, int man, int exp,
                                  int bl, int bu, int sat)
{
    for (int64_t i = 0; i < n; ++i) o[i] = orc_cast_superfp(a[i], man, exp, bl, bu, sat);
}

/* ------------------------------------------------------------------------- */
/* per-MAC rounded GEMM                                                      */
/* ------------------------------------------------------------------------- */

/* A rounding format: IEEE-like float (kind 0), supernormal float (kind 1: a = binades_l, b = binades_u) or
 * P3109 binary8 (kind 2: a = P, b = is_signed, c = overflow policy).  The reference instantiates the same
 * GEMM / softmax / layernorm templates with each of the three casters (quant_cuda/superfp_kernel.cu:79-262,
 * binary8_kernel.cu:344-491; CPU quant.cpp:893-1150, binary8.cpp:370-542). */
typedef struct { int man, exp, sub, sat; int kind, a, b, c; } fmt_t;
static inline float Q(float x, fmt_t f)
{
    if (f.kind == 1) return orc_cast_superfp(x, f.man, f.exp, f.a, f.b, f.sat);
    if (f.kind == 2) return orc_cast_binary8(x, f.a, f.b, f.c, f.sub, 0, 0u, 0);
    return cast_fp_rn_or_rz(x, f.man, f.exp, f.sub, f.sat, 0);
}
/* descriptor layout shared with the loader: {kind, man, exp, sub, sat, a, b, c} */
static fmt_t fmt_from(const int *d) { fmt_t f = {d[1], d[2], d[3], d[4], d[0], d[5], d[6], d[7]}; return f; }

/* Philox4x32-10 (Salmon et al., SC'11), the counter-based generator the
 * stochastic GEMM keys by (seed; batch,row,col,k).  Published algorithm;
 * the reference's own SR GEMM draws from a racy per-block cuRAND state seeded
 * by clock64() and is not reproducible (mm_kernel.h:263, fp_kernel.cu:131). */
static void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1)
{
    for (int i = 0; i < 10; ++i) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

ORC_API void orc_philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                        uint32_t k0, uint32_t k1, uint32_t *out)
{
    uint32_t c[4] = {c0, c1, c2, c3};
    philox4x32_10(c, k0, k1);
    memcpy(out, c, 16);
}

/* order 0 "seq":  c = Qadd(c + Qmul(a*b)) for k = 0..K-1
 *                 reference: quant_cpu/mm_kernel.h:9-20 (fma: :36-45).
 * order 1 "tile8": K is walked in tiles of 8 (zero padded; one extra all-zero
 *                 tile when 8 | K); inner accumulates a tile, then
 *                 outer = Qadd(outer + inner).
 *                 reference: quant_cuda/mm_kernel.h:34-70 (fma: :134-186).
 * compensated (Kahan) and stochastic variants walk the zero padded K range
 * with a single accumulator: reference quant_cuda/mm_kernel.h:457-520, :248-295. */
static void mm_impl(const float *a, const float *b, float *c, int64_t B, int M, int K, int N,
                    fmt_t fa, fmt_t fm, int fma, int order, int compensated);

ORC_API void orc_mm(const float *a, const float *b, float *c, int64_t B, int M, int K, int N,
                    int man_add, int exp_add, int man_mul, int exp_mul,
                    int sub, int sat, int fma, int order, int compensated)
{
    fmt_t fa = {man_add, exp_add, sub, sat}, fm = {man_mul, exp_mul, sub, sat};
    mm_impl(a, b, c, B, M, K, N, fa, fm, fma, order, compensated);
}

ORC_API void orc_mm_fmt(const float *a, const float *b, float *c, int64_t B, int M, int K, int N,
                        const int *fmt_add, const int *fmt_mul, int fma, int order)
{
    mm_impl(a, b, c, B, M, K, N, fmt_from(fmt_add), fmt_from(fmt_mul), fma, order, 0);
}

static void mm_impl(const float *a, const float *b, float *c, int64_t B, int M, int K, int N,
                    fmt_t fa, fmt_t fm, int fma, int order, int compensated)
{
    int Kpad = K + 8 - K % 8;
    /* Rows of C are independent; each output still sees its k steps in the stated order.  The loops
       run k outside j (as the reference CPU kernel does) so B is read along its rows. */
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t bi = 0; bi < B; ++bi) {
        for (int i = 0; i < M; ++i) {
            const float *A = a + bi * (int64_t)M * K + (int64_t)i * K, *Bm = b + bi * (int64_t)K * N;
            float *C = c + bi * (int64_t)M * N + (int64_t)i * N;
            float *s1 = (float *)calloc((size_t)N, sizeof(float));   /* acc / inner / sum  */
            float *s2 = (float *)calloc((size_t)N, sizeof(float));   /* outer / comp       */
            if (compensated) {
                /* order 1 restates the CUDA kernel (per-output state, padded K);
                   order 0 uses the same recurrence over k < K.               */
                int kend = order ? Kpad : K;
                for (int k = 0; k < kend; ++k) {
                    float av = k < K ? A[k] : 0.f;
                    for (int j = 0; j < N; ++j) {
                        float bv = k < K ? Bm[(int64_t)k * N + j] : 0.f;
                        float sum = s1[j], comp = s2[j], y, t;
                        if (fma) y = Q(fmaf(av, bv, -comp), fa);
                        else y = Q(Q(av * bv, fm) - comp, fa);
                        t = Q(sum + y, fa);
                        s2[j] = Q(Q(t - sum, fa) - y, fa);
                        s1[j] = t;
                    }
                }
                memcpy(C, s1, (size_t)N * sizeof(float));
            } else if (order == 0) {
                for (int k = 0; k < K; ++k) {
                    float av = A[k];
                    const float *brow = Bm + (int64_t)k * N;
                    for (int j = 0; j < N; ++j)
                        s1[j] = fma ? Q(fmaf(av, brow[j], s1[j]), fa) : Q(s1[j] + Q(av * brow[j], fm), fa);
                }
                memcpy(C, s1, (size_t)N * sizeof(float));
            } else {
                /* A multiply format that rounds nothing (man >= 23, exp >= 8) leaves `inner + a * b` in the
                   CUDA kernel, and the reference's CUDA build evaluates that as one fused multiply-add
                   (measured on its unmodified build: equal to the fused variant with the add format, bit for
                   bit, and different from the separately rounded product).  Order 1 restates the CUDA
                   kernel, so it does the same; order 0, the CPU kernel, multiplies and adds separately. */
                const int fused = fma || (fa.kind == 0 && fm.kind == 0 && fm.man >= 23 && fm.exp >= 8);
                for (int k0 = 0; k0 < Kpad; k0 += 8) {
                    for (int kk = 0; kk < 8; ++kk) {
                        int k = k0 + kk;
                        float av = k < K ? A[k] : 0.f;
                        for (int j = 0; j < N; ++j) {
                            float bv = k < K ? Bm[(int64_t)k * N + j] : 0.f;
                            s1[j] = fused ? Q(fmaf(av, bv, s1[j]), fa) : Q(s1[j] + Q(av * bv, fm), fa);
                        }
                    }
                    for (int j = 0; j < N; ++j) { s2[j] = Q(s2[j] + s1[j], fa); s1[j] = 0.f; }
                }
                memcpy(C, s2, (size_t)N * sizeof(float));
            }
            free(s1); free(s2);
        }
    }
}

/* Stochastic-rounding GEMM, single accumulator over the zero padded K range
 * (structure: reference quant_cuda/mm_kernel.h:248-295; fma :358-400).
 * Random words: Philox4x32-10 with key (seed_lo, seed_hi); every word of a
 * call is used.  Two-rounding MAC: counter (k / 2, linear output index lo,
 * hi, 0), word 2 (k % 2) feeds the add rounding and word 2 (k % 2) + 1 the
 * multiply rounding.  Fused MAC: counter (k / 4, ...), word k % 4.
 * The stochastic caster has no NaN early-out: it adds the random word to the
 * NaN's bit pattern and clips whatever comes out, so the result depends on the
 * payload.  CUDA arithmetic returns the canonical NaN 0x7FFFFFFF (x86 returns
 * 0xFFC00000 for inf - inf), and the product is CUDA code, so every NaN that
 * an arithmetic step yields is replaced by 0x7FFFFFFF before it is cast.
 * PARITY UNPINNED against the reference (its generator state is racy).    */
static float cuda_nan(float x) { return x != x ? u2f(0x7FFFFFFFu) : x; }

ORC_API void orc_mm_sr(const float *a, const float *b, float *c, int64_t B, int M, int K, int N,
                       int man_add, int exp_add, int rbits_add,
                       int man_mul, int exp_mul, int rbits_mul,
                       int sub, int sat, int fma, uint64_t seed)
{
    int Kpad = K + 8 - K % 8;
    for (int64_t bi = 0; bi < B; ++bi) {
        const float *A = a + bi * (int64_t)M * K, *Bm = b + bi * (int64_t)K * N;
        float *C = c + bi * (int64_t)M * N;
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j) {
                uint64_t lin = (uint64_t)bi * M * N + (uint64_t)i * N + j;
                float acc = 0.f;
                for (int k = 0; k < Kpad; ++k) {
                    float av = k < K ? A[(int64_t)i * K + k] : 0.f;
                    float bv = k < K ? Bm[(int64_t)k * N + j] : 0.f;
                    uint32_t ctr[4] = {(uint32_t)(fma ? k / 4 : k / 2), (uint32_t)lin, (uint32_t)(lin >> 32), 0u};
                    philox4x32_10(ctr, (uint32_t)seed, (uint32_t)(seed >> 32));
                    if (fma) {
                        acc = orc_cast_fp_stochastic(cuda_nan(fmaf(av, bv, acc)), ctr[k % 4], rbits_add, man_add, exp_add, sub, sat);
                    } else {
                        volatile float prod = av * bv;
                        float p = orc_cast_fp_stochastic(cuda_nan(prod), ctr[2 * (k % 2) + 1], rbits_mul, man_mul, exp_mul, sub, sat);
                        volatile float sum = acc + p;
                        acc = orc_cast_fp_stochastic(cuda_nan(sum), ctr[2 * (k % 2)], rbits_add, man_add, exp_add, sub, sat);
                    }
                }
                C[(int64_t)i * N + j] = acc;
            }
    }
}

/* ------------------------------------------------------------------------- */
/* quantized reductions: softmax, layernorm                                  */
/* ------------------------------------------------------------------------- */

/* "tree64": the association the reference CUDA kernels use for a row
 * (softmax_kernel.h:5-21,78-93; layernorm_kernel.h:29-50): 64 threads take
 * elements tid, tid+64, ... sequentially; each warp folds with offsets
 * 16,8,4,2,1 (lane l takes lane l+off; lanes past 31 read back their own
 * value); the result is op(warp0, warp1).                                  */
typedef float (*binop_t)(float, float, const void *);

static float tree64_combine(float part[64], binop_t op, const void *ctx)
{
    for (int w = 0; w < 2; ++w) {
        float *v = part + 32 * w;
        for (int off = 16; off > 0; off >>= 1) {
            float nv[32];
            for (int l = 0; l < 32; ++l) nv[l] = op(v[l], (l + off < 32) ? v[l + off] : v[l], ctx);
            memcpy(v, nv, sizeof nv);
        }
    }
    return op(part[0], part[32], ctx);
}

static float op_qadd(float a, float b, const void *ctx) { return Q(a + b, *(const fmt_t *)ctx); }
static float op_max(float a, float b, const void *ctx) { (void)ctx; return fmaxf(a, b); }
static float op_qlse(float a, float b, const void *ctx) { return Q(logf(expf(a) + expf(b)), *(const fmt_t *)ctx); }

/* order 0 (seq): reference quant_cpu/softmax.h:11-46.
 * order 1 (tree64): reference quant_cuda/softmax_kernel.h:23-100.          */
static void softmax_forward_impl(const float *in, float *out, int64_t outer, int channel, int64_t inner, fmt_t fe, fmt_t fo, fmt_t fa, int order);

ORC_API void orc_softmax_forward(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                 int man_exp, int exp_exp, int man_off, int exp_off,
                                 int man_acc, int exp_acc, int sub, int sat, int order)
{
    fmt_t fe = {man_exp, exp_exp, sub, sat}, fo = {man_off, exp_off, sub, sat}, fa = {man_acc, exp_acc, sub, sat};
    softmax_forward_impl(in, out, outer, channel, inner, fe, fo, fa, order);
}

ORC_API void orc_softmax_forward_fmt(const float *in, float *out, int64_t outer, int channel, int64_t inner, const int *d_fe, const int *d_fo, const int *d_fa, int order)
{
    softmax_forward_impl(in, out, outer, channel, inner, fmt_from(d_fe), fmt_from(d_fo), fmt_from(d_fa), order);
}

static void softmax_forward_impl(const float *in, float *out, int64_t outer, int channel, int64_t inner, fmt_t fe, fmt_t fo, fmt_t fa, int order)
{
    for (int64_t row = 0; row < outer * inner; ++row) {
        const float *x = in + (row / inner) * channel * inner + row % inner;
        float *y = out + (row / inner) * channel * inner + row % inner;
        float mx, sum;
        if (order == 0) {
            mx = x[0];
            for (int k = 1; k < channel; ++k) mx = fmaxf(mx, x[k * inner]);
            sum = 0.f;
            for (int k = 0; k < channel; ++k) {
                float e = Q(expf(Q(x[k * inner] - mx, fo)), fe);
                y[k * inner] = e;
                sum = Q(sum + e, fa);
            }
        } else {
            float part[64];
            for (int t = 0; t < 64; ++t) {
                part[t] = -INFINITY;
                for (int k = t; k < channel; k += 64) part[t] = fmaxf(part[t], x[k * inner]);
            }
            mx = tree64_combine(part, op_max, NULL);
            for (int k = 0; k < channel; ++k) y[k * inner] = Q(expf(Q(x[k * inner] - mx, fo)), fe);
            for (int t = 0; t < 64; ++t) {
                part[t] = 0.f;
                for (int k = t; k < channel; k += 64) part[t] = Q(part[t] + y[k * inner], fa);
            }
            sum = tree64_combine(part, op_qadd, &fa);
        }
        for (int k = 0; k < channel; ++k) y[k * inner] = y[k * inner] / sum;
    }
}

/* order 0: reference quant_cpu/softmax.h:50-87; order 1: quant_cuda/softmax_kernel.h:102-171. */
static void softmax_lse_forward_impl(const float *in, float *out, int64_t outer, int channel, int64_t inner, fmt_t fo, fmt_t fl, int order);

ORC_API void orc_softmax_lse_forward(const float *in, float *out, int64_t outer, int channel, int64_t inner,
                                     int man_off, int exp_off, int man_lse, int exp_lse,
                                     int sub, int sat, int order)
{
    fmt_t fo = {man_off, exp_off, sub, sat}, fl = {man_lse, exp_lse, sub, sat};
    softmax_lse_forward_impl(in, out, outer, channel, inner, fo, fl, order);
}

ORC_API void orc_softmax_lse_forward_fmt(const float *in, float *out, int64_t outer, int channel, int64_t inner, const int *d_fo, const int *d_fl, int order)
{
    softmax_lse_forward_impl(in, out, outer, channel, inner, fmt_from(d_fo), fmt_from(d_fl), order);
}

static void softmax_lse_forward_impl(const float *in, float *out, int64_t outer, int channel, int64_t inner, fmt_t fo, fmt_t fl, int order)
{
    for (int64_t row = 0; row < outer * inner; ++row) {
        const float *x = in + (row / inner) * channel * inner + row % inner;
        float *y = out + (row / inner) * channel * inner + row % inner;
        float mx, lgs;
        if (order == 0) {
            mx = x[0];
            for (int k = 1; k < channel; ++k) mx = fmaxf(mx, x[k * inner]);
            float x0 = Q(x[0] - mx, fo);
            y[0] = x0;
            lgs = x0;
            for (int k = 1; k < channel; ++k) {
                float v = Q(x[k * inner] - mx, fo);
                y[k * inner] = v;
                lgs = Q(logf(expf(lgs) + expf(v)), fl);
            }
        } else {
            float part[64];
            for (int t = 0; t < 64; ++t) {
                part[t] = -INFINITY;
                for (int k = t; k < channel; k += 64) part[t] = fmaxf(part[t], x[k * inner]);
            }
            mx = tree64_combine(part, op_max, NULL);
            for (int t = 0; t < 64; ++t) {
                part[t] = -INFINITY;
                for (int k = t; k < channel; k += 64) {
                    float v = Q(x[k * inner] - mx, fo);
                    y[k * inner] = v;
                    part[t] = Q(logf(expf(part[t]) + expf(v)), fl);
                }
            }
            lgs = tree64_combine(part, op_qlse, &fl);
        }
        for (int k = 0; k < channel; ++k) y[k * inner] = expf(Q(y[k * inner] - lgs, fo));
    }
}

/* order 0: reference quant_cpu/softmax.h:89-114; order 1: quant_cuda/softmax_kernel.h:173-222. */
static void softmax_backward_impl(const float *yv, const float *g, float *out, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, int order);

ORC_API void orc_softmax_backward(const float *yv, const float *g, float *out, int64_t outer, int channel,
                                  int64_t inner, int man_add, int exp_add, int man_mul, int exp_mul,
                                  int sub, int sat, int order)
{
    fmt_t fa = {man_add, exp_add, sub, sat}, fm = {man_mul, exp_mul, sub, sat};
    softmax_backward_impl(yv, g, out, outer, channel, inner, fa, fm, order);
}

ORC_API void orc_softmax_backward_fmt(const float *yv, const float *g, float *out, int64_t outer, int channel, int64_t inner, const int *d_fa, const int *d_fm, int order)
{
    softmax_backward_impl(yv, g, out, outer, channel, inner, fmt_from(d_fa), fmt_from(d_fm), order);
}

static void softmax_backward_impl(const float *yv, const float *g, float *out, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, int order)
{
    for (int64_t row = 0; row < outer * inner; ++row) {
        int64_t base = (row / inner) * channel * inner + row % inner;
        const float *y = yv + base, *gr = g + base;
        float *o = out + base;
        float s;
        if (order == 0) {
            s = 0.f;
            for (int k = 0; k < channel; ++k) s = Q(s + Q(y[k * inner] * gr[k * inner], fm), fa);
        } else {
            float part[64];
            for (int t = 0; t < 64; ++t) {
                part[t] = 0.f;
                for (int k = t; k < channel; k += 64)
                    part[t] = Q(part[t] + Q(y[k * inner] * gr[k * inner], fm), fa);
            }
            s = tree64_combine(part, op_qadd, &fa);
        }
        for (int k = 0; k < channel; ++k) o[k * inner] = Q(gr[k * inner] - s, fa) * y[k * inner];
    }
}

/* order 0: reference quant_cpu/layernorm.h:10-57 (mean and variance are
 * rounded with Qdiv after the division).
 * order 1: reference quant_cuda/layernorm_kernel.h:7-100 (tree64 sums; mean
 * and variance are NOT rounded after the division).                        */
static void layernorm_forward_impl(const float *in, const float *w, const float *bias, float *out, float *mean, float *rstd, float eps, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, fmt_t fd, fmt_t fs, int order);

ORC_API void orc_layernorm_forward(const float *in, const float *w, const float *bias, float *out,
                                   float *mean, float *rstd, float eps,
                                   int64_t outer, int channel, int64_t inner,
                                   int man_acc, int exp_acc, int man_mul, int exp_mul,
                                   int man_div, int exp_div, int man_sqrt, int exp_sqrt,
                                   int sub, int sat, int order)
{
    fmt_t fa = {man_acc, exp_acc, sub, sat}, fm = {man_mul, exp_mul, sub, sat};
    fmt_t fd = {man_div, exp_div, sub, sat}, fs = {man_sqrt, exp_sqrt, sub, sat};
    layernorm_forward_impl(in, w, bias, out, mean, rstd, eps, outer, channel, inner, fa, fm, fd, fs, order);
}

ORC_API void orc_layernorm_forward_fmt(const float *in, const float *w, const float *bias, float *out, float *mean, float *rstd, float eps, int64_t outer, int channel, int64_t inner, const int *d_fa, const int *d_fm, const int *d_fd, const int *d_fs, int order)
{
    layernorm_forward_impl(in, w, bias, out, mean, rstd, eps, outer, channel, inner, fmt_from(d_fa), fmt_from(d_fm), fmt_from(d_fd), fmt_from(d_fs), order);
}

static void layernorm_forward_impl(const float *in, const float *w, const float *bias, float *out, float *mean, float *rstd, float eps, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, fmt_t fd, fmt_t fs, int order)
{
    for (int64_t row = 0; row < outer * inner; ++row) {
        int64_t base = (row / inner) * channel * inner + row % inner;
        const float *x = in + base;
        float *y = out + base;
        float m, var;
        if (order == 0) {
            m = 0.f;
            for (int k = 0; k < channel; ++k) m = Q(m + x[k * inner], fa);
            m = Q(m / channel, fd);
            var = 0.f;
            for (int k = 0; k < channel; ++k) {
                float sh = Q(x[k * inner] - m, fa);
                var = Q(var + Q(sh * sh, fm), fa);
            }
            var = Q(var / channel, fd);
        } else {
            float part[64];
            for (int t = 0; t < 64; ++t) {
                part[t] = 0.f;
                for (int k = t; k < channel; k += 64) part[t] = Q(part[t] + x[k * inner], fa);
            }
            m = tree64_combine(part, op_qadd, &fa) / channel;
            for (int t = 0; t < 64; ++t) {
                part[t] = 0.f;
                for (int k = t; k < channel; k += 64) {
                    float sh = Q(x[k * inner] - m, fa);
                    part[t] = Q(part[t] + Q(sh * sh, fm), fa);
                }
            }
            var = tree64_combine(part, op_qadd, &fa) / channel;
        }
        float sd = Q(sqrtf(Q(var + eps, fa)), fs);
        for (int k = 0; k < channel; ++k) {
            float norm = Q(Q(x[k * inner] - m, fa) / sd, fd);
            y[k * inner] = Q(w[k] * norm, fm) + bias[k];
        }
        mean[row] = m;
        rstd[row] = Q(1.0f / sd, fd);
    }
}

/* order 0: reference quant_cpu/layernorm.h:60-116 (grad_gamma/grad_beta are
 * accumulated in place, row after row).
 * order 1: reference quant_cuda/layernorm_kernel.h:105-237 (tree64 row sums;
 * second pass sums rows 0..R-1 per channel starting from zero).
 * grad_gamma/grad_beta must be zero-filled by the caller for order 0, as the
 * reference's Python wrapper does (quant_function.py:1210-1212).           */
static void layernorm_backward_impl(const float *in, const float *g, const float *w, const float *mean, const float *rstd, float *gin, float *ggamma, float *gbeta, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, fmt_t fd, int order);

ORC_API void orc_layernorm_backward(const float *in, const float *g, const float *w,
                                    const float *mean, const float *rstd,
                                    float *gin, float *ggamma, float *gbeta,
                                    int64_t outer, int channel, int64_t inner,
                                    int man_acc, int exp_acc, int man_mul, int exp_mul,
                                    int man_div, int exp_div, int sub, int sat, int order)
{
    fmt_t fa = {man_acc, exp_acc, sub, sat}, fm = {man_mul, exp_mul, sub, sat}, fd = {man_div, exp_div, sub, sat};
    layernorm_backward_impl(in, g, w, mean, rstd, gin, ggamma, gbeta, outer, channel, inner, fa, fm, fd, order);
}

ORC_API void orc_layernorm_backward_fmt(const float *in, const float *g, const float *w, const float *mean, const float *rstd, float *gin, float *ggamma, float *gbeta, int64_t outer, int channel, int64_t inner, const int *d_fa, const int *d_fm, const int *d_fd, int order)
{
    layernorm_backward_impl(in, g, w, mean, rstd, gin, ggamma, gbeta, outer, channel, inner, fmt_from(d_fa), fmt_from(d_fm), fmt_from(d_fd), order);
}

static void layernorm_backward_impl(const float *in, const float *g, const float *w, const float *mean, const float *rstd, float *gin, float *ggamma, float *gbeta, int64_t outer, int channel, int64_t inner, fmt_t fa, fmt_t fm, fmt_t fd, int order)
{
    if (order == 1) for (int k = 0; k < channel; ++k) { ggamma[k] = 0.f; gbeta[k] = 0.f; }
    for (int64_t row = 0; row < outer * inner; ++row) {
        int64_t base = (row / inner) * channel * inner + row % inner;
        const float *x = in + base, *gr = g + base;
        float *o = gin + base;
        float m = mean[row], r = rstd[row];
        float gs, gsx;
        if (order == 0) {
            gs = 0.f; gsx = 0.f;
            for (int k = 0; k < channel; ++k) {
                float xhat = Q(Q(x[k * inner] - m, fa) * r, fm);
                float ng = Q(w[k] * gr[k * inner], fm);
                gs = Q(gs + ng, fa);
                gsx = Q(gsx + Q(xhat * ng, fm), fa);
            }
        } else {
            float p1[64], p2[64];
            for (int t = 0; t < 64; ++t) {
                p1[t] = 0.f; p2[t] = 0.f;
                for (int k = t; k < channel; k += 64) {
                    float xhat = Q(Q(x[k * inner] - m, fa) * r, fm);
                    float ng = Q(w[k] * gr[k * inner], fm);
                    p1[t] = Q(p1[t] + ng, fa);
                    p2[t] = Q(p2[t] + Q(xhat * ng, fm), fa);
                }
            }
            gs = tree64_combine(p1, op_qadd, &fa);
            gsx = tree64_combine(p2, op_qadd, &fa);
        }
        gs = Q(gs / channel, fd);
        gsx = Q(gsx / channel, fd);
        for (int k = 0; k < channel; ++k) {
            float xhat = Q(Q(x[k * inner] - m, fa) * r, fm);
            float xg = Q(xhat * gr[k * inner], fm);
            float ng = Q(w[k] * gr[k * inner], fm);
            gbeta[k] = Q(gbeta[k] + gr[k * inner], fa);
            ggamma[k] = Q(ggamma[k] + xg, fa);
            float wg = Q(xhat * gsx, fm);
            float gi = Q(ng - gs, fa);
            gi = Q(gi - wg, fa);
            o[k * inner] = Q(gi * r, fm);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* MX and NVFP4 block quantizers -- NO reference counterpart, parity unpinned */
/* ------------------------------------------------------------------------- */

/* Round v to the OCP element format (exp_e exponent bits, man_e mantissa bits,
 * bias 2^(exp_e-1)-1, maximum finite `emax_val`) with round-to-nearest-even,
 * subnormals kept and saturation to +-emax_val.  E4M3: (4,3,448), E2M1: (2,1,6). */
static float ocp_elem_rne(float v, int exp_e, int man_e, float emax_val)
{
    if (v != v) return v;
    uint32_t t = f2u(v);
    uint32_t sign = t & 0x80000000u;
    float a = fabsf(v);
    if (a >= emax_val) return u2f(sign | f2u(emax_val));   /* also +-inf */
    int min_exp = 2 - (1 << (exp_e - 1));                   /* smallest normal exponent */
    int E = (int)((t << 1) >> 24) - 127;
    int qexp = (E < min_exp ? min_exp : E) - man_e;        /* exponent of the quantum */
    float quantum = ldexpf(1.0f, qexp);
    float r = nearbyintf(a / quantum) * quantum;           /* exact: power-of-two scaling, RNE mode */
    if (r > emax_val) r = emax_val;
    return u2f(sign | f2u(r));
}

/* Bit code of a value that is exactly representable in the OCP element format (sign, exp_e exponent bits with bias
 * 2^(exp_e-1)-1, man_e mantissa bits; subnormals below the smallest normal).  NaN: 0x7F for E4M3 (S.1111.111), 0 for
 * E2M1, which has no NaN. */
static uint8_t ocp_elem_code(float q, int exp_e, int man_e)
{
    if (q != q) return exp_e == 4 ? 0x7F : 0;
    uint32_t t = f2u(q);
    uint8_t sign = (uint8_t)((t >> 31) << (exp_e + man_e));
    float a = fabsf(q);
    int bias = (1 << (exp_e - 1)) - 1;
    int min_exp = 1 - bias;
    if (a < ldexpf(1.0f, min_exp)) return sign | (uint8_t)(a * ldexpf(1.0f, man_e - min_exp));   /* subnormal: a / 2^(min_exp-man) */
    int E = (int)((t << 1) >> 24) - 127;
    uint32_t man = (t & 0x7FFFFFu) >> (23 - man_e);
    return sign | (uint8_t)(((E + bias) << man_e) | man);
}

/* MX block quantize along the last (contiguous) dimension.
 * Shared scale: e = floor(log2(amax)) - emax_elem, clamped to [-127,127],
 * stored as E8M0 code e+127.  amax == 0 -> code 0 (scale 2^-127), block all 0.
 * A block holding NaN or inf gets code 0xFF and every output NaN.
 * Elements: RNE(v * 2^-e) in the element format, saturating; out = elem * 2^e.
 * elem_kind: 0 = E4M3 (emax_elem 8, max 448), 1 = E2M1 (emax_elem 2, max 6).
 * codes (optional): the element codes, one byte per element for E4M3, two elements per byte for E2M1 (element 2i
 * in the low nibble; a row occupies ceil(cols / 2) bytes).  A poisoned block writes 0x7F (E4M3) or 0 (E2M1). */
ORC_API void orc_mx_quantize_codes(const float *in, float *out, uint8_t *scales, uint8_t *codes, int64_t rows, int64_t cols,
                                   int block, int elem_kind);
ORC_API void orc_mx_quantize(const float *in, float *out, uint8_t *scales, int64_t rows, int64_t cols,
                             int block, int elem_kind)
{
    orc_mx_quantize_codes(in, out, scales, NULL, rows, cols, block, elem_kind);
}
static void put_code(uint8_t *codes, int64_t r, int64_t c, int64_t cols, int fp4, uint8_t code)
{
    if (!codes) return;
    if (!fp4) { codes[r * cols + c] = code; return; }
    uint8_t *b = codes + r * ((cols + 1) / 2) + c / 2;
    if (c & 1) *b = (uint8_t)((*b & 0x0F) | (code << 4));
    else *b = (uint8_t)((*b & 0xF0) | (code & 0x0F));
}
ORC_API void orc_mx_quantize_codes(const float *in, float *out, uint8_t *scales, uint8_t *codes, int64_t rows, int64_t cols,
                                   int block, int elem_kind)
{
    int exp_e = elem_kind == 0 ? 4 : 2, man_e = elem_kind == 0 ? 3 : 1;
    int emax_elem = elem_kind == 0 ? 8 : 2;
    float emax_val = elem_kind == 0 ? 448.0f : 6.0f;
    int64_t nblk = (cols + block - 1) / block;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t bidx = 0; bidx < nblk; ++bidx) {
            int64_t c0 = bidx * block, c1 = c0 + block < cols ? c0 + block : cols;
            uint32_t amax_bits = 0;
            for (int64_t c = c0; c < c1; ++c) {
                uint32_t ab = f2u(in[r * cols + c]) & 0x7FFFFFFFu;
                if (ab > amax_bits) amax_bits = ab;
            }
            uint8_t code;
            if (amax_bits >= 0x7F800000u) {
                code = 0xFF;
                for (int64_t c = c0; c < c1; ++c) {
                    out[r * cols + c] = NAN;
                    put_code(codes, r, c, cols, elem_kind == 1, elem_kind == 0 ? 0x7F : 0);
                }
            } else {
                int e;
                if (amax_bits == 0) e = -127;
                else {
                    int fl = (int)(amax_bits >> 23) - 127;            /* floor(log2) of a normal */
                    if ((amax_bits >> 23) == 0) {                      /* fp32 denormal */
                        fl = -127;
                        for (uint32_t mbits = amax_bits; mbits < 0x800000u; mbits <<= 1) fl--;
                        fl += 1;
                    }
                    e = fl - emax_elem;
                    if (e < -127) e = -127;
                    if (e > 127) e = 127;
                }
                code = (uint8_t)(e + 127);
                for (int64_t c = c0; c < c1; ++c) {
                    /* two exact power-of-two steps keep ldexp out of the denormal range */
                    float v = ldexpf(ldexpf(in[r * cols + c], -e / 2), -(e - e / 2));
                    float q = ocp_elem_rne(v, exp_e, man_e, emax_val);
                    out[r * cols + c] = ldexpf(ldexpf(q, e / 2), e - e / 2);
                    put_code(codes, r, c, cols, elem_kind == 1, ocp_elem_code(q, exp_e, man_e));
                }
            }
            if (scales) scales[r * nblk + bidx] = code;
        }
}

/* NVFP4: blocks of 16 along the last dimension, E2M1 elements, one E4M3 (OCP
 * "fn", max 448) scale per block and one fp32 global scale s_g.
 *   s_b  = RNE_E4M3(amax_block / (6 * s_g))        (true fp32 divisions)
 *   elem = RNE_E2M1(v / (s_b * s_g)), saturating at +-6;   out = elem * (s_b * s_g)
 * s_b == 0 -> block outputs 0, except that a NaN element stays NaN.  If
 * global_scale <= 0 it is computed as amax_tensor / (448 * 6) over the FINITE
 * entries (1.0 when there is none above zero): infinities and NaN do not
 * take part.  Within a block NaN entries are skipped by the maximum, an
 * infinite one saturates its block scale at 448 and itself at +-6.
 * codes (optional): E2M1 element codes, two per byte (element 2i in the low
 * nibble, ceil(cols / 2) bytes per row; a NaN element is coded as 0, E2M1
 * has no NaN); scale_codes (optional): the block scales as E4M3 bytes.    */
ORC_API float orc_nvfp4_quantize_codes(const float *in, float *out, float *block_scales, uint8_t *codes, uint8_t *scale_codes,
                                       int64_t rows, int64_t cols, float global_scale);
ORC_API float orc_nvfp4_quantize(const float *in, float *out, float *block_scales, int64_t rows, int64_t cols,
                                 float global_scale)
{
    return orc_nvfp4_quantize_codes(in, out, block_scales, NULL, NULL, rows, cols, global_scale);
}
ORC_API float orc_nvfp4_quantize_codes(const float *in, float *out, float *block_scales, uint8_t *codes, uint8_t *scale_codes,
                                       int64_t rows, int64_t cols, float global_scale)
{
    const int block = 16;
    float sg = global_scale;
    if (!(sg > 0.f)) {
        float amax = 0.f;
        for (int64_t i = 0; i < rows * cols; ++i) { float a = fabsf(in[i]); if (a > amax && a < INFINITY) amax = a; }
        sg = amax > 0.f ? amax / (448.0f * 6.0f) : 1.0f;
    }
    int64_t nblk = (cols + block - 1) / block;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t bidx = 0; bidx < nblk; ++bidx) {
            int64_t c0 = bidx * block, c1 = c0 + block < cols ? c0 + block : cols;
            float amax = 0.f;
            for (int64_t c = c0; c < c1; ++c) { float a = fabsf(in[r * cols + c]); if (a > amax) amax = a; }
            volatile float denom = 6.0f * sg;
            volatile float ratio = amax / denom;
            float sb = ocp_elem_rne(ratio, 4, 3, 448.0f);
            volatile float sc = sb * sg;
            if (block_scales) block_scales[r * nblk + bidx] = sb;
            if (scale_codes) scale_codes[r * nblk + bidx] = ocp_elem_code(sb, 4, 3);
            for (int64_t c = c0; c < c1; ++c) {
                float x = in[r * cols + c];
                if (sc == 0.f) { out[r * cols + c] = (x != x) ? x : 0.f; put_code(codes, r, c, cols, 1, 0); continue; }
                volatile float v = x / sc;
                volatile float q = ocp_elem_rne(v, 2, 1, 6.0f);
                out[r * cols + c] = q * sc;
                put_code(codes, r, c, cols, 1, ocp_elem_code(q, 2, 1));
            }
        }
    return sg;
}

/* Sequential quantized sum over dim 0 of a [rows, cols] matrix: for each column
 * acc = 0; acc = Q(acc + x[r, col]) for r = 0..rows-1.
 * reference: mptorch/quant/functional.py:736-748 (qsum_1d: starts from a zero
 * tensor, one quantize per slice, the first slice included).               */
ORC_API void orc_qsum_rows(const float *in, float *out, int64_t rows, int64_t cols,
                           int man, int exp, int sub, int sat)
{
    fmt_t f = {man, exp, sub, sat};
    for (int64_t c = 0; c < cols; ++c) {
        float acc = 0.f;
        for (int64_t r = 0; r < rows; ++r) acc = Q(acc + in[r * cols + c], f);
        out[c] = acc;
    }
}
