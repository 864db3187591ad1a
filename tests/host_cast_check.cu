// Host-side harness around mptorch_b200/csrc/cast.cuh (test infrastructure).
// The casters are __host__ __device__; compiling them for the CPU lets the CPU test suite
// sweep the very source the kernels use against the oracle, without a GPU.
#include <cstdint>
#include <cstring>

#include "../mptorch_b200/csrc/cast.cuh"

using namespace mpt;

#define HC_API extern "C" __attribute__((visibility("default")))

HC_API void hc_float_quantize(const float* in, float* out, int64_t n, int man, int exp, int sub, int sat,
                              int mode, const int32_t* rnd, int rbits) {
    const FpFmt f = make_fmt(man, exp, sub, sat);
    for (int64_t i = 0; i < n; ++i) {
        if (mode == 0) out[i] = cast_fp_nearest(in[i], f);
        else if (mode == 2) out[i] = cast_fp_truncate(in[i], f);
        else out[i] = cast_fp_stochastic(in[i], (uint32_t)rnd[i], rbits, f);
    }
}

HC_API void hc_binary8(const float* in, float* out, int64_t n, int P, int is_signed, int policy, int sub,
                       int mode, const int32_t* rnd, int prng_bits) {
    for (int64_t i = 0; i < n; ++i)
        out[i] = cast_binary8(in[i], P, is_signed != 0, policy, sub != 0, mode, rnd ? (uint32_t)rnd[i] : 0u, prng_bits);
}

HC_API void hc_superfp(const float* in, float* out, int64_t n, int man, int exp, int bl, int bu, int sat) {
    for (int64_t i = 0; i < n; ++i) out[i] = cast_superfp(in[i], man, exp, bl, bu, sat != 0);
}

// Sweep fp32 patterns first, first+stride, ... (count of them) and compare the fast FP-pipe rounding
// with the exact caster wherever the fast path's precondition holds (finite, exponent within
// fast_rn_exp_limit, and -- for exp == 8 formats -- not an fp32 denormal).  Returns the number of
// mismatches; the first mismatching pattern is written to *first_bad.
HC_API int64_t hc_sweep_fast_rn(int man, int exp, uint64_t first, uint64_t count, uint64_t stride,
                                uint32_t* first_bad) {
    const FpFmt f = make_fmt(man, exp, 1, 0);
    const FastRn fast = FastRn::make(f);
    const int lim = fast_rn_exp_limit(f);
    int64_t bad = 0;
    uint32_t firstbad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const uint32_t t = (uint32_t)(first + (uint64_t)i * stride);
        const int E = (int)((t << 1) >> 24) - 127;
        if (E > lim) continue;
        if (exp == 8 && E == -127 && (t & 0x7FFFFFu) != 0u) continue;
        const float x = u2f(t);
        const uint32_t want = f2u(cast_fp_nearest(x, f));
        const uint32_t got = f2u(fast(x));
        if (want != got) {
            ++bad;
#pragma omp critical
            if (firstbad == 0) firstbad = t;
        }
    }
    if (first_bad) *first_bad = firstbad;
    return bad;
}

// Same sweep for the whole-domain variant used by the elementwise quantizer: every pattern is
// compared, no precondition.
HC_API int64_t hc_sweep_full_rn(int man, int exp, int sat, uint64_t first, uint64_t count, uint64_t stride,
                                uint32_t* first_bad) {
    const FpFmt f = make_fmt(man, exp, 1, sat);
    const FullRn full = FullRn::make(f);
    int64_t bad = 0;
    uint32_t firstbad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const uint32_t t = (uint32_t)(first + (uint64_t)i * stride);
        const float x = u2f(t);
        const uint32_t want = f2u(cast_fp_nearest(x, f));
        const uint32_t got = f2u(full(x));
        const bool both_nan = (want & 0x7FFFFFFFu) > 0x7F800000u && (got & 0x7FFFFFFFu) > 0x7F800000u;
        if (want != got && !both_nan) {
            ++bad;
#pragma omp critical
            if (firstbad == 0) firstbad = t;
        }
    }
    if (first_bad) *first_bad = firstbad;
    return bad;
}

template <class Got, class Want>
static int64_t sweep_all(uint64_t first, uint64_t count, uint64_t stride, uint32_t* first_bad, Got got_fn, Want want_fn) {
    int64_t bad = 0;
    uint32_t firstbad = 0;
    bool have = false;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const uint32_t t = (uint32_t)(first + (uint64_t)i * stride);
        const float x = u2f(t);
        const uint32_t want = f2u(want_fn(x));
        const uint32_t got = f2u(got_fn(x));
        const bool both_nan = (want & 0x7FFFFFFFu) > 0x7F800000u && (got & 0x7FFFFFFFu) > 0x7F800000u;
        if (want != got && !both_nan) {
            ++bad;
#pragma omp critical
            if (!have) { firstbad = t; have = true; }
        }
    }
    if (first_bad) *first_bad = firstbad;
    return bad;
}

// fast_rn_nosub vs the exact caster of the same format without subnormals, over the domain the range-checked GEMM
// path guarantees: zero or a normal fp32 number, exponent at most fast_rn_exp_limit
HC_API int64_t hc_sweep_fast_rn_nosub(int man, int exp, uint64_t first, uint64_t count, uint64_t stride, uint32_t* first_bad) {
    const FpFmt f = make_fmt(man, exp, 0, 0);
    const FastRn fast = FastRn::make(f);
    const int lim = fast_rn_exp_limit(f);
    int64_t bad = 0;
    uint32_t worst = 0xFFFFFFFFu;
#pragma omp parallel for reduction(+ : bad) reduction(min : worst)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const uint32_t bits = (uint32_t)(first + (uint64_t)i * stride);
        const uint32_t a = bits & 0x7FFFFFFFu;
        const int e = (int)(a >> 23) - 127;
        if (a != 0u && (a < 0x00800000u || e > lim)) continue;
        const float x = u2f(bits);
        const uint32_t want = f2u(cast_fp_nearest(x, f));
        uint32_t rare = 0u;
        const uint32_t flagged = f2u(fast_rn_nosub_flag(fast, x, rare));
        // the flagged form promises the exact result whenever it does not raise its flag, and must raise it exactly
        // when the plain rounding lands on a nonzero value below the smallest normal one
        const bool flag_ok = rare ? true : flagged == want;
        if (f2u(fast_rn_nosub(fast, x)) != want || f2u(fast_rn_nosub_rare(fast, x)) != want || !flag_ok) { ++bad; if (bits < worst) worst = bits; }
    }
    if (first_bad) *first_bad = worst;
    return bad;
}

// whole-domain truncation (FullRz) vs the exact truncating caster
HC_API int64_t hc_sweep_full_rz(int man, int exp, int sat, uint64_t first, uint64_t count, uint64_t stride, uint32_t* first_bad) {
    const FpFmt f = make_fmt(man, exp, 1, sat);
    const FullRz full = FullRz::make(f);
    return sweep_all(first, count, stride, first_bad, [&](float x) { return full(x); }, [&](float x) { return cast_fp_truncate(x, f); });
}

// whole-domain binary8 nearest (FullRnB8) vs the exact binary8 caster
HC_API int64_t hc_sweep_full_b8(int P, int is_signed, int policy, uint64_t first, uint64_t count, uint64_t stride, uint32_t* first_bad) {
    const FullRnB8 full = FullRnB8::make(P, is_signed != 0, policy);
    return sweep_all(first, count, stride, first_bad, [&](float x) { return full(x); },
                     [&](float x) { return cast_binary8(x, P, is_signed != 0, policy, true, RND_NEAREST, 0u, 0); });
}

// whole-domain stochastic rounding (FullSr) vs the exact caster, random word derived from the pattern
HC_API int64_t hc_sweep_full_sr(int man, int exp, int sat, int rbits, uint64_t first, uint64_t count, uint64_t stride, uint32_t* first_bad) {
    const FpFmt f = make_fmt(man, exp, 1, sat);
    const FullSr full = FullSr::make(f, rbits);
    auto word = [](float x) { uint32_t h = f2u(x) * 2654435761u; h ^= h >> 15; h *= 2246822519u; h ^= h >> 13; return h & 0x7FFFFFFFu; };
    return sweep_all(first, count, stride, first_bad, [&](float x) { return full(x, word(x)); },
                     [&](float x) { return cast_fp_stochastic(x, word(x), rbits, f); });
}

// Random (a, b) pairs in the range the row kernels use div_with_rcp on: b = +-2^[-20, 20] * [1, 2), a zero or
// +-2^[lo_exp, hi_exp] * [1, 2) with a mantissa cut to `man_a` bits (the dividends are rounded values) or full.
// Compares with the host's IEEE division.  Returns the number of mismatches.
HC_API int64_t hc_sweep_div_with_rcp(uint64_t seed, uint64_t count, int lo_exp, int hi_exp, int man_a, uint32_t* first_bad) {
    int64_t bad = 0;
    uint32_t firstbad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        uint64_t z = seed + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1);      // splitmix64
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
        uint64_t w = z * 0xD6E8FEB86659FD93ull; w ^= w >> 32;
        const int eb = (int)(z % 41) - 20;
        const uint32_t tb = ((uint32_t)(eb + 127) << 23) | (uint32_t)((z >> 8) & 0x7FFFFFu) | ((uint32_t)((z >> 40) & 1u) << 31);
        const int ea = lo_exp + (int)(w % (uint64_t)(hi_exp - lo_exp + 1));
        uint32_t ma = (uint32_t)((w >> 8) & 0x7FFFFFu);
        if (man_a < 23) ma &= ~((1u << (23 - man_a)) - 1u);
        const uint32_t ta = ((uint32_t)(ea + 127) << 23) | ma | ((uint32_t)((w >> 41) & 1u) << 31);
        const float a = ((w >> 50) % 64 == 0) ? 0.0f : u2f(ta), b = u2f(tb);
        volatile float r = 1.0f / b;
        volatile float want = a / b;
        const float got = div_with_rcp(a, b, r);
        if (f2u(want) != f2u(got)) {
            ++bad;
#pragma omp critical
            if (firstbad == 0) firstbad = ta;
        }
    }
    if (first_bad) *first_bad = firstbad;
    return bad;
}
