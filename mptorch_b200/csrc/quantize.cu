// Elementwise quantizers: one streaming kernel family, 128-bit accesses, HBM-bound.
//
// Algorithmic traffic is 8 B per element (4 read + 4 written); the stochastic cast with caller
// supplied random words reads 4 B more.  The reference launches one thread per element over a
// pre-zeroed output (12 or 20 B per element); here the output is written once.
#include "cast.cuh"
#include "common.cuh"

namespace mpt {
namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;   // float4 loads in flight per thread

// F: float4 -> float4 functor given the linear index of the first element.
template <class F>
__global__ void __launch_bounds__(kThreads) map_f4_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                          int64_t n, F f) {
    const int64_t nvec = n >> 2;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; v + (kVecPerThread - 1) * stride < nvec; v += kVecPerThread * stride) {
        float4 x[kVecPerThread];
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) x[u] = __ldcs(in4 + v + u * stride);
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) __stcs(out4 + v + u * stride, f.vec(x[u], (v + u * stride) << 2));
    }
    for (; v < nvec; v += stride) __stcs(out4 + v, f.vec(__ldcs(in4 + v), v << 2));
    // ragged tail (n % 4 elements)
    const int64_t tail = (nvec << 2) + (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (tail < n) out[tail] = f.one(in[tail], tail);
}

// Fallback for pointers that are not 16-byte aligned.
template <class F>
__global__ void __launch_bounds__(kThreads) map_scalar_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                              int64_t n, F f) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = f.one(in[i], i);
}

template <class F>
int launch_map(const float* in, float* out, int64_t n, F f, cudaStream_t st, const char* what) {
    if (n == 0) return MPT_OK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const int sms = sm_count();
    if (aligned) {
        const int64_t nvec = n >> 2;
        int64_t blocks = (nvec + (int64_t)kThreads * kVecPerThread - 1) / ((int64_t)kThreads * kVecPerThread);
        const int64_t cap = (int64_t)sms * 8 * 4;      // 8 resident CTAs per SM, 4 waves
        if (blocks > cap) blocks = cap - cap % sms;
        if (blocks < 1) blocks = 1;
        map_f4_kernel<F><<<(unsigned)blocks, kThreads, 0, st>>>(in, out, n, f);
    } else {
        int64_t blocks = (n + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sms * 32;
        if (blocks > cap) blocks = cap;
        map_scalar_kernel<F><<<(unsigned)blocks, kThreads, 0, st>>>(in, out, n, f);
    }
    return check_launch(what);
}

#define MPT_VEC_FROM_ONE                                                                     \
    __device__ __forceinline__ float4 vec(float4 x, int64_t i) const {                       \
        return make_float4(one(x.x, i), one(x.y, i + 1), one(x.z, i + 2), one(x.w, i + 3));  \
    }

struct FpNearest {
    FpFmt f;
    __device__ __forceinline__ float one(float x, int64_t) const { return cast_fp_nearest(x, f); }
    MPT_VEC_FROM_ONE
};
// Same result as FpNearest on every input (swept on the host against the exact caster), about a
// quarter of the instructions: what keeps the kernel at the HBM roofline instead of the issue one.
struct FpNearestFast {
    FullRn r;
    __device__ __forceinline__ float one(float x, int64_t) const { return r(x); }
    MPT_VEC_FROM_ONE
};
// Formats without subnormals (the reference's FloatingPoint default): the settling FP-pipe rounding for zero and for
// normal fp32 inputs below the overflow threshold, which is nearly every input; fp32 denormals, overflow, infinities
// and NaN take the exact caster behind one compare.
struct FpNearestFastNoSub {
    FpFmt f;
    FastRn r;
    uint32_t span;        // as bit patterns: |x| in [2^-126, min(overflow threshold, largest magnitude the magic constant of an
                          // 8-bit-exponent format can serve)) is the fast domain
    __host__ static FpNearestFastNoSub make(const FpFmt& f) {
        const FullRn full = FullRn::make(f);
        const uint32_t top = full.ovf_from < full.exact_from ? full.ovf_from : full.exact_from;
        return FpNearestFastNoSub{f, full.fast, top - 0x00800000u};
    }
    __device__ __forceinline__ float one(float x, int64_t) const {
        const uint32_t a = __float_as_uint(x) & 0x7FFFFFFFu;
        if (a == 0u) return x;
        if (a - 0x00800000u >= span) return cast_fp_nearest(x, f);
        return fast_rn_nosub(r, x);
    }
    MPT_VEC_FROM_ONE
};
struct FpTruncateFast {
    FullRz r;
    __device__ __forceinline__ float one(float x, int64_t) const { return r(x); }
    MPT_VEC_FROM_ONE
};
struct Binary8NearestFast {
    FullRnB8 r;
    __device__ __forceinline__ float one(float x, int64_t) const { return r(x); }
    MPT_VEC_FROM_ONE
};
struct FpTruncate {
    FpFmt f;
    __device__ __forceinline__ float one(float x, int64_t) const { return cast_fp_truncate(x, f); }
    MPT_VEC_FROM_ONE
};
// SR casters with a common call shape: exact (every format) and the straight-line FullSr (formats with subnormals)
struct SrExact {
    FpFmt f;
    int rbits;
    __device__ __forceinline__ float operator()(float x, uint32_t r) const { return cast_fp_stochastic(x, r, rbits, f); }
};

template <class SR>
struct FpStochastic {
    SR sr;
    const int32_t* __restrict__ rnd;
    __device__ __forceinline__ float one(float x, int64_t i) const { return sr(x, (uint32_t)__ldcs(rnd + i)); }
    __device__ __forceinline__ float4 vec(float4 x, int64_t i) const {
        // the random words are as aligned as the data when the caller allocates both the same way
        int4 r;
        if ((reinterpret_cast<uintptr_t>(rnd) & 15u) == 0) r = __ldcs(reinterpret_cast<const int4*>(rnd + i));
        else r = make_int4(rnd[i], rnd[i + 1], rnd[i + 2], rnd[i + 3]);
        return make_float4(sr(x.x, (uint32_t)r.x), sr(x.y, (uint32_t)r.y), sr(x.z, (uint32_t)r.z), sr(x.w, (uint32_t)r.w));
    }
};
// Random words from Philox4x32-10: counter = (i / 4, i / 4 >> 32, 0, 0), key = seed; element i
// takes word i % 4.  31 bits are used, like the reference's randint_like(a, INT_MAX).
template <class SR>
struct FpStochasticPhilox {
    SR sr;
    uint32_t k0, k1;
    __device__ __forceinline__ float one(float x, int64_t i) const {
        const uint64_t blk = (uint64_t)i >> 2;
        Philox p((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u);
        p.run(k0, k1);
        return sr(x, p.c[i & 3] & 0x7FFFFFFFu);
    }
    __device__ __forceinline__ float4 vec(float4 x, int64_t i) const {
        const uint64_t blk = (uint64_t)i >> 2;
        Philox p((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u);
        p.run(k0, k1);
        return make_float4(sr(x.x, p.c[0] & 0x7FFFFFFFu), sr(x.y, p.c[1] & 0x7FFFFFFFu), sr(x.z, p.c[2] & 0x7FFFFFFFu),
                           sr(x.w, p.c[3] & 0x7FFFFFFFu));
    }
};
struct Binary8 {
    int P, is_signed, policy, sub, mode, prng_bits;
    const int32_t* __restrict__ rnd;
    __device__ __forceinline__ float one(float x, int64_t i) const {
        const uint32_t r = (mode == RND_STOCHASTIC) ? (uint32_t)rnd[i] : 0u;
        return cast_binary8(x, P, is_signed != 0, policy, sub != 0, mode, r, prng_bits);
    }
    MPT_VEC_FROM_ONE
};
struct SuperFp {
    int man, exp, bl, bu, sat;
    __device__ __forceinline__ float one(float x, int64_t) const { return cast_superfp(x, man, exp, bl, bu, sat != 0); }
    MPT_VEC_FROM_ONE
};

// ---------------------------------------------------------------------------------- many tensors, one launch
// The optimizer wrappers quantize every parameter, gradient and moment tensor of a model each step: hundreds of
// small tensors, one launch each in the reference (optim_low.py:65-113).  Here a launch carries a table of up to
// kMultiMax tensors in its kernel parameters (no device-side table, so nothing is allocated); a CTA looks up the
// tensor its block index falls into and processes one contiguous chunk of it.
constexpr int kMultiMax = 48;
constexpr int kMultiChunk = kThreads * 4 * kVecPerThread;     // elements per CTA

struct MultiTable {
    const float* in[kMultiMax];
    float* out[kMultiMax];
    int64_t n[kMultiMax];
    int first_block[kMultiMax + 1];
    int first_tensor;     // index of in[0] in the caller's list (decorrelates the stochastic streams)
    int count;
};

template <class F>
__global__ void __launch_bounds__(kThreads) multi_map_kernel(const __grid_constant__ MultiTable t, F f0) {
    int lo = 0, hi = t.count;
    const int b = blockIdx.x;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (t.first_block[mid] <= b) lo = mid; else hi = mid;
    }
    const F f = f0.for_tensor(t.first_tensor + lo);
    const float* __restrict__ in = t.in[lo];
    float* __restrict__ out = t.out[lo];
    const int64_t n = t.n[lo];
    const int64_t begin = (int64_t)(b - t.first_block[lo]) * kMultiChunk;
    const int64_t end = begin + kMultiChunk < n ? begin + kMultiChunk : n;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (aligned) {
        const int64_t vend = begin + ((end - begin) & ~(int64_t)3);       // begin is a multiple of 4
        for (int64_t i = begin + 4 * threadIdx.x; i < vend; i += 4 * kThreads)
            *reinterpret_cast<float4*>(out + i) = f.vec(*reinterpret_cast<const float4*>(in + i), i);
        const int64_t tail = vend + threadIdx.x;
        if (tail < end) out[tail] = f.one(in[tail], tail);
    } else {
        for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) out[i] = f.one(in[i], i);
    }
}

template <class F>
int launch_multi(const float* const* in, float* const* out, const int64_t* n, int count, F f, cudaStream_t st, const char* what) {
    int i = 0;
    while (i < count) {
        MultiTable t{};
        t.first_tensor = i;
        int blocks = 0, k = 0;
        for (; i < count && k < kMultiMax; ++i) {
            if (n[i] == 0) continue;
            const int64_t nb = (n[i] + kMultiChunk - 1) / kMultiChunk;
            if (nb > 0x3FFFFFFF - blocks) break;                 // keep the block prefix inside an int: start a new launch
            t.in[k] = in[i]; t.out[k] = out[i]; t.n[k] = n[i];
            t.first_block[k] = blocks;
            blocks += (int)nb;
            ++k;
        }
        if (k == 0) {
            if (i < count) { set_error("%s: tensor %d is too large for the multi-tensor path", what, i); return MPT_ERR_INVALID_ARGUMENT; }
            break;
        }
        // stochastic streams are keyed by the position of the tensor in the caller's list: entries skipped as empty
        // shift later keys, which is harmless (any key gives an independent stream)
        t.first_block[k] = blocks;
        t.count = k;
        multi_map_kernel<F><<<(unsigned)blocks, kThreads, 0, st>>>(t, f);
        const int rc = check_launch(what);
        if (rc) return rc;
    }
    return MPT_OK;
}

template <class F>
struct SameForAll : F {
    __device__ __forceinline__ SameForAll for_tensor(int) const { return *this; }
};
template <class SR>
struct PhiloxPerTensor : FpStochasticPhilox<SR> {
    __device__ __forceinline__ PhiloxPerTensor for_tensor(int idx) const {
        PhiloxPerTensor p = *this;
        p.k1 ^= 0x9E3779B9u * (uint32_t)(idx + 1);
        return p;
    }
};

}  // namespace
}  // namespace mpt

using namespace mpt;

extern "C" {

int mpt_float_quantize_nearest(const float* in, float* out, int64_t n, int man, int exp, int subnormals,
                               int saturate, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out)), "float_quantize_nearest: null pointer or negative size");
    MPT_REQUIRE(valid_format(man, exp), "float_quantize_nearest: unsupported format man=%d exp=%d", man, exp);
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    if (fast_rn_supported(f)) return launch_map(in, out, n, FpNearestFast{FullRn::make(f)}, as_stream(stream), "float_quantize_nearest");
    if (!f.sub && f.man <= 21 && f.exp >= 2) return launch_map(in, out, n, FpNearestFastNoSub::make(f), as_stream(stream), "float_quantize_nearest");
    return launch_map(in, out, n, FpNearest{f}, as_stream(stream), "float_quantize_nearest");
}

int mpt_float_quantize_truncate(const float* in, float* out, int64_t n, int man, int exp, int subnormals,
                                int saturate, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out)), "float_quantize_truncate: null pointer or negative size");
    MPT_REQUIRE(valid_format(man, exp), "float_quantize_truncate: unsupported format man=%d exp=%d", man, exp);
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    if (fast_rn_supported(f)) return launch_map(in, out, n, FpTruncateFast{FullRz::make(f)}, as_stream(stream), "float_quantize_truncate");
    return launch_map(in, out, n, FpTruncate{f}, as_stream(stream), "float_quantize_truncate");
}

int mpt_float_quantize_stochastic(const float* in, const int32_t* rand, float* out, int64_t n, int man, int exp,
                                  int prng_bits, int subnormals, int saturate, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out && rand)), "float_quantize_stochastic: null pointer or negative size");
    MPT_REQUIRE(valid_format(man, exp), "float_quantize_stochastic: unsupported format man=%d exp=%d", man, exp);
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    if (FullSr::supported(f))
        return launch_map(in, out, n, FpStochastic<FullSr>{FullSr::make(f, prng_bits), rand}, as_stream(stream), "float_quantize_stochastic");
    return launch_map(in, out, n, FpStochastic<SrExact>{SrExact{f, prng_bits}, rand}, as_stream(stream), "float_quantize_stochastic");
}

int mpt_float_quantize_stochastic_philox(const float* in, float* out, int64_t n, int man, int exp, int prng_bits,
                                         int subnormals, int saturate, uint64_t seed, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out)), "float_quantize_stochastic_philox: null pointer or negative size");
    MPT_REQUIRE(valid_format(man, exp), "float_quantize_stochastic_philox: unsupported format man=%d exp=%d", man, exp);
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    if (FullSr::supported(f))
        return launch_map(in, out, n, FpStochasticPhilox<FullSr>{FullSr::make(f, prng_bits), k0, k1}, as_stream(stream),
                          "float_quantize_stochastic_philox");
    return launch_map(in, out, n, FpStochasticPhilox<SrExact>{SrExact{f, prng_bits}, k0, k1}, as_stream(stream),
                      "float_quantize_stochastic_philox");
}

int mpt_float_quantize_multi(const float* const* in, float* const* out, const int64_t* n, int count, int man, int exp,
                             int subnormals, int saturate, int rounding, int prng_bits, uint64_t seed, void* stream) {
    MPT_REQUIRE(count >= 0, "float_quantize_multi: negative tensor count");
    if (count == 0) return MPT_OK;
    MPT_REQUIRE(in && out && n, "float_quantize_multi: null table");
    MPT_REQUIRE(valid_format(man, exp), "float_quantize_multi: unsupported format man=%d exp=%d", man, exp);
    MPT_REQUIRE(rounding >= 0 && rounding <= 2, "float_quantize_multi: unknown rounding mode %d", rounding);
    for (int i = 0; i < count; ++i)
        MPT_REQUIRE(n[i] >= 0 && (n[i] == 0 || (in[i] && out[i])), "float_quantize_multi: tensor %d has a null pointer or a negative size", i);
    const FpFmt f = make_fmt(man, exp, subnormals, saturate);
    cudaStream_t st = as_stream(stream);
    const char* who = "float_quantize_multi";
    if (rounding == MPT_RND_NEAREST) {
        if (fast_rn_supported(f)) return launch_multi(in, out, n, count, SameForAll<FpNearestFast>{{FullRn::make(f)}}, st, who);
        if (!f.sub && f.man <= 21 && f.exp >= 2) return launch_multi(in, out, n, count, SameForAll<FpNearestFastNoSub>{FpNearestFastNoSub::make(f)}, st, who);
        return launch_multi(in, out, n, count, SameForAll<FpNearest>{{f}}, st, who);
    }
    if (rounding == MPT_RND_TRUNCATE) {
        if (fast_rn_supported(f)) return launch_multi(in, out, n, count, SameForAll<FpTruncateFast>{{FullRz::make(f)}}, st, who);
        return launch_multi(in, out, n, count, SameForAll<FpTruncate>{{f}}, st, who);
    }
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    if (FullSr::supported(f)) return launch_multi(in, out, n, count, PhiloxPerTensor<FullSr>{{FullSr::make(f, prng_bits), k0, k1}}, st, who);
    return launch_multi(in, out, n, count, PhiloxPerTensor<SrExact>{{SrExact{f, prng_bits}, k0, k1}}, st, who);
}

int mpt_binary8_quantize(const float* in, const int32_t* rand, float* out, int64_t n, int P, int is_signed,
                         int overflow_policy, int subnormals, int rounding, int prng_bits, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out)), "binary8_quantize: null pointer or negative size");
    MPT_REQUIRE(P >= 1 && P <= 7, "binary8_quantize: P=%d outside 1..7", P);
    MPT_REQUIRE(overflow_policy >= 0 && overflow_policy <= 2, "binary8_quantize: unknown overflow policy %d", overflow_policy);
    MPT_REQUIRE(rounding >= 0 && rounding <= 2, "binary8_quantize: unknown rounding mode %d", rounding);
    MPT_REQUIRE(rounding != MPT_RND_STOCHASTIC || n == 0 || rand, "binary8_quantize: stochastic rounding needs random words");
    if (rounding == MPT_RND_NEAREST && FullRnB8::supported(P, subnormals != 0))
        return launch_map(in, out, n, Binary8NearestFast{FullRnB8::make(P, is_signed != 0, overflow_policy)}, as_stream(stream),
                          "binary8_quantize");
    return launch_map(in, out, n, Binary8{P, is_signed, overflow_policy, subnormals, rounding, prng_bits, rand},
                      as_stream(stream), "binary8_quantize");
}

int mpt_superfp_quantize_nearest(const float* in, float* out, int64_t n, int man, int exp, int binades_l,
                                 int binades_u, int saturate, void* stream) {
    MPT_REQUIRE(n >= 0 && (n == 0 || (in && out)), "superfp_quantize_nearest: null pointer or negative size");
    MPT_REQUIRE(valid_format(man, exp), "superfp_quantize_nearest: unsupported format man=%d exp=%d", man, exp);
    return launch_map(in, out, n, SuperFp{man, exp, binades_l, binades_u, saturate}, as_stream(stream),
                      "superfp_quantize_nearest");
}

}
