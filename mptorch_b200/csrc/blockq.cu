// Block-scaled quantizers along the last (contiguous) dimension: OCP MX (MXFP8-E4M3, MXFP4-E2M1 over
// 32-element blocks with E8M0 power-of-two scales) and NVFP4 (E2M1 over 16-element blocks with an E4M3
// scale per block and one fp32 scale per tensor).  Output convention of the library: an fp32 tensor of
// the input's shape holding the dequantized values; the scales and the packed element codes (one byte per E4M3
// element, two E2M1 elements per byte with the even element in the low nibble) can be written out as well.
//
// The reference has no such kernels (its block_quantize is a whole-tensor shared-exponent format), so
// the definitions are the ones frozen in the CPU oracle; they follow the OCP Microscaling and NVFP4
// descriptions: power-of-two scale 2^(floor(log2 amax) - emax_elem) for MX, amax / 6 rounded to E4M3
// for NVFP4, elements rounded to nearest even with saturation.
//
// HBM-bound: 8 B per element (plus 1/32 or 1/4 B per element of scales when requested).  Each thread
// owns four consecutive elements (one 128-bit load and store); the 8 (MX) or 4 (NVFP4) lanes that share
// a block find its maximum with warp shuffles.  The NVFP4 tensor scale, when not supplied, costs one
// extra read pass (a separate amax kernel into a 4-byte scratch word).
#include "cast.cuh"
#include "common.cuh"

namespace mpt {
namespace {

constexpr int kThreads = 256;

// Round |a| (finite, below `top`) to an OCP element format: quantum 2^(max(E, min_exp) - man), nearest even.
struct ElemFmt {
    int min_e_bits;   // (min normal exponent + 127) << 23
    float k;          // 1.5 * 2^(23 - man)
    float top;        // largest finite value
    // bit code of a rounded value: sign | ((|v| bits >> code_shift) - code_sub) for normals, (int)(|v| * sub_scale) below
    int code_shift, sign_shift;
    uint32_t code_sub, nan_code;
    float min_norm, sub_scale;
    __host__ __device__ static ElemFmt make(int exp_e, int man_e, float top) {
        ElemFmt f;
        f.min_e_bits = (2 - (1 << (exp_e - 1)) + 127) << 23;
        union { uint32_t u; float v; } c;
        c.u = ((uint32_t)(127 + 23 - man_e) << 23) | 0x400000u;
        f.k = c.v;
        f.top = top;
        const int bias = (1 << (exp_e - 1)) - 1;
        f.code_shift = 23 - man_e;
        f.sign_shift = 31 - (exp_e + man_e);
        f.code_sub = (uint32_t)(127 - bias) << man_e;
        f.nan_code = exp_e == 4 ? 0x7Fu : 0u;                 // E2M1 has no NaN
        c.u = (uint32_t)(127 + 1 - bias) << 23; f.min_norm = c.v;
        c.u = (uint32_t)(127 + man_e - (1 - bias)) << 23; f.sub_scale = c.v;
        return f;
    }
    // v: a value this format represents exactly (an output of round), or NaN
    __device__ __forceinline__ uint32_t code(float v) const {
        if (v != v) return nan_code;
        const uint32_t t = __float_as_uint(v), a = t & 0x7FFFFFFFu;
        const uint32_t mag = __uint_as_float(a) >= min_norm ? (a >> code_shift) - code_sub : (uint32_t)(__uint_as_float(a) * sub_scale);
        return ((t & 0x80000000u) >> sign_shift) | mag;
    }
    __device__ __forceinline__ float round(float v) const {
        if (v != v) return v;
        const uint32_t t = __float_as_uint(v);
        const uint32_t sign = t & 0x80000000u;
        const float a = __uint_as_float(t & 0x7FFFFFFFu);
        float r;
        if (a >= top) r = top;
        else {
            const int e = (int)(t & 0x7F800000u);
            const float m = __uint_as_float((uint32_t)max(e, min_e_bits));
            const float y = __fmaf_rn(m, k, a);
            r = fminf(__fmaf_rn(m, -k, y), top);
        }
        return __uint_as_float(sign | __float_as_uint(r));
    }
};

__device__ __forceinline__ float pow2f(int e) {   // 2^e for e in [-127, 127]
    return e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(0x00400000u);
}

// ---- MX -------------------------------------------------------------------------------------
// LANES lanes (each with 4 consecutive elements) share one block of 4 * LANES elements.
// CODES: the packed element codes are wanted too (a launch without them carries none of that arithmetic).
template <int LANES, bool CODES>
__global__ void __launch_bounds__(kThreads) mx_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                                      uint8_t* __restrict__ scales, uint8_t* __restrict__ codes, int fp4,
                                                      int64_t nvec, ElemFmt ef, int emax_elem) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    // the loop bound is rounded up to a whole warp so that shuffles always see 32 participating lanes
    const int64_t nvec_up = (nvec + 31) & ~(int64_t)31;
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec_up; v += stride) {
        const bool live = v < nvec;
        const float4 x = live ? __ldcs(in + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t amax = max(max(__float_as_uint(x.x) & 0x7FFFFFFFu, __float_as_uint(x.y) & 0x7FFFFFFFu),
                            max(__float_as_uint(x.z) & 0x7FFFFFFFu, __float_as_uint(x.w) & 0x7FFFFFFFu));
#pragma unroll
        for (int off = LANES / 2; off > 0; off >>= 1) amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        float4 y;
        uint8_t code;
        uint32_t packed = 0u;                 // the four element codes: a byte each (E4M3) or a nibble each (E2M1)
        if (amax >= 0x7F800000u) {            // a NaN or an infinity poisons the block
            code = 0xFF;
            const float nanv = __uint_as_float(0x7FC00000u);
            y = make_float4(nanv, nanv, nanv, nanv);
            if (CODES) packed = fp4 ? 0u : 0x7F7F7F7Fu;
        } else {
            int e = -127;
            if (amax != 0u) {
                const int fl = (amax >> 23) ? (int)(amax >> 23) - 127 : (31 - __clz((int)amax)) - 149;
                e = min(max(fl - emax_elem, -127), 127);
            }
            code = (uint8_t)(e + 127);
            const float down = pow2f(-e), up = pow2f(e);
            const float q0 = ef.round(__fmul_rn(x.x, down)), q1 = ef.round(__fmul_rn(x.y, down));
            const float q2 = ef.round(__fmul_rn(x.z, down)), q3 = ef.round(__fmul_rn(x.w, down));
            y.x = __fmul_rn(q0, up);
            y.y = __fmul_rn(q1, up);
            y.z = __fmul_rn(q2, up);
            y.w = __fmul_rn(q3, up);
            if (CODES) {
                const int w = fp4 ? 4 : 8;
                packed = ef.code(q0) | (ef.code(q1) << w) | (ef.code(q2) << (2 * w)) | (ef.code(q3) << (3 * w));
            }
        }
        if (live) {
            __stcs(out + v, y);
            if (scales != nullptr && (v % LANES) == 0) scales[v / LANES] = code;
            if (CODES) {
                if (fp4) reinterpret_cast<uint16_t*>(codes)[v] = (uint16_t)packed;
                else reinterpret_cast<uint32_t*>(codes)[v] = packed;
            }
        }
    }
}

// Any block size and any column count: one thread per block (slow path, same arithmetic).
// One thread writes all code bytes of its block: the caller guarantees an even block size when nibbles are packed.
__device__ __forceinline__ void put_code(uint8_t* codes, int64_t r, int64_t c, int64_t cols, int fp4, uint32_t code) {
    if (!fp4) { codes[r * cols + c] = (uint8_t)code; return; }
    uint8_t* b = codes + r * ((cols + 1) / 2) + c / 2;
    *b = (c & 1) ? (uint8_t)((*b & 0x0F) | (code << 4)) : (uint8_t)code;     // the even element writes the byte first
}

__global__ void __launch_bounds__(kThreads) mx_generic_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                              uint8_t* __restrict__ scales, uint8_t* __restrict__ codes, int fp4,
                                                              int64_t rows, int64_t cols, int block, ElemFmt ef, int emax_elem) {
    const int64_t nblk = (cols + block - 1) / block;
    const int64_t total = rows * nblk;
    for (int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x; b < total; b += (int64_t)gridDim.x * kThreads) {
        const int64_t r = b / nblk, c0 = (b % nblk) * block;
        const int64_t c1 = min(c0 + (int64_t)block, cols);
        const float* x = in + r * cols;
        float* y = out + r * cols;
        uint32_t amax = 0u;
        for (int64_t c = c0; c < c1; ++c) amax = max(amax, __float_as_uint(x[c]) & 0x7FFFFFFFu);
        uint8_t code;
        if (amax >= 0x7F800000u) {
            code = 0xFF;
            for (int64_t c = c0; c < c1; ++c) {
                y[c] = __uint_as_float(0x7FC00000u);
                if (codes != nullptr) put_code(codes, r, c, cols, fp4, ef.nan_code);
            }
        } else {
            int e = -127;
            if (amax != 0u) {
                const int fl = (amax >> 23) ? (int)(amax >> 23) - 127 : (31 - __clz((int)amax)) - 149;
                e = min(max(fl - emax_elem, -127), 127);
            }
            code = (uint8_t)(e + 127);
            const float down = pow2f(-e), up = pow2f(e);
            for (int64_t c = c0; c < c1; ++c) {
                const float q = ef.round(__fmul_rn(x[c], down));
                y[c] = __fmul_rn(q, up);
                if (codes != nullptr) put_code(codes, r, c, cols, fp4, ef.code(q));
            }
        }
        if (scales != nullptr) scales[b] = code;
    }
}

// ---- NVFP4 ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) amax_kernel(const float* __restrict__ x, int64_t n, uint32_t* amax_bits) {
    float m = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
        const float a = fabsf(x[i]);
        if (a < INFINITY) m = fmaxf(m, a);    // the tensor scale is taken over the finite entries: NaN and infinities are skipped
    }
    uint32_t b = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(m));   // non-negative floats order like their bits
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, b);
}

__global__ void amax_init_kernel(uint32_t* amax_bits) { *amax_bits = 0u; }

struct Nvfp4Fmt { ElemFmt e4m3, e2m1; };

__device__ __forceinline__ float nvfp4_global_scale(float given, const uint32_t* amax_bits) {
    if (given > 0.f) return given;
    const float amax = __uint_as_float(*amax_bits);
    return amax > 0.f ? __fdiv_rn(amax, 448.0f * 6.0f) : 1.0f;
}

// Dequantized value of one element; with CODES, `code` receives its E2M1 bits.  A zero block scale yields zeros, but a
// NaN stays NaN.
template <bool CODES>
__device__ __forceinline__ float nvfp4_elem(float x, float sc, const ElemFmt& e2m1, uint32_t& code) {
    if (sc == 0.f) { code = 0u; return (x != x) ? x : 0.f; }
    const float q = e2m1.round(__fdiv_rn(x, sc));
    if (CODES) code = e2m1.code(q);
    return __fmul_rn(q, sc);
}

template <bool CODES>
__global__ void __launch_bounds__(kThreads) nvfp4_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                                         float* __restrict__ block_scales, uint8_t* __restrict__ codes,
                                                         uint8_t* __restrict__ scale_codes, int64_t nvec, float given_scale,
                                                         const uint32_t* amax_bits, float* scale_out, Nvfp4Fmt f) {
    const float sg = nvfp4_global_scale(given_scale, amax_bits);
    if (scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = sg;
    const float denom = __fmul_rn(6.0f, sg);
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t nvec_up = (nvec + 31) & ~(int64_t)31;
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec_up; v += stride) {
        const bool live = v < nvec;
        const float4 x = live ? __ldcs(in + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        float amax = fmaxf(fmaxf(fmaxf(fmaxf(0.f, fabsf(x.x)), fabsf(x.y)), fabsf(x.z)), fabsf(x.w));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        const float sb = f.e4m3.round(__fdiv_rn(amax, denom));
        const float sc = __fmul_rn(sb, sg);
        if (live) {
            uint32_t c0 = 0u, c1 = 0u, c2 = 0u, c3 = 0u;
            const float4 y = make_float4(nvfp4_elem<CODES>(x.x, sc, f.e2m1, c0), nvfp4_elem<CODES>(x.y, sc, f.e2m1, c1),
                                         nvfp4_elem<CODES>(x.z, sc, f.e2m1, c2), nvfp4_elem<CODES>(x.w, sc, f.e2m1, c3));
            __stcs(out + v, y);
            if (CODES && codes != nullptr) reinterpret_cast<uint16_t*>(codes)[v] = (uint16_t)(c0 | (c1 << 4) | (c2 << 8) | (c3 << 12));
            if ((v & 3) == 0) {
                if (block_scales != nullptr) block_scales[v >> 2] = sb;
                if (CODES && scale_codes != nullptr) scale_codes[v >> 2] = (uint8_t)f.e4m3.code(sb);
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads) nvfp4_generic_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                 float* __restrict__ block_scales, uint8_t* __restrict__ codes,
                                                                 uint8_t* __restrict__ scale_codes, int64_t rows, int64_t cols,
                                                                 float given_scale, const uint32_t* amax_bits, float* scale_out, Nvfp4Fmt f) {
    const float sg = nvfp4_global_scale(given_scale, amax_bits);
    if (scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = sg;
    const float denom = __fmul_rn(6.0f, sg);
    const int64_t nblk = (cols + 15) / 16, total = rows * nblk;
    for (int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x; b < total; b += (int64_t)gridDim.x * kThreads) {
        const int64_t r = b / nblk, c0 = (b % nblk) * 16;
        const int64_t c1 = min(c0 + (int64_t)16, cols);
        const float* x = in + r * cols;
        float* y = out + r * cols;
        float amax = 0.f;
        for (int64_t c = c0; c < c1; ++c) amax = fmaxf(amax, fabsf(x[c]));
        const float sb = f.e4m3.round(__fdiv_rn(amax, denom));
        const float sc = __fmul_rn(sb, sg);
        if (block_scales != nullptr) block_scales[b] = sb;
        if (scale_codes != nullptr) scale_codes[b] = (uint8_t)f.e4m3.code(sb);
        for (int64_t c = c0; c < c1; ++c) {
            uint32_t code;
            y[c] = nvfp4_elem<true>(x[c], sc, f.e2m1, code);
            if (codes != nullptr) put_code(codes, r, c, cols, 1, code);
        }
    }
}

unsigned stream_blocks(int64_t items) {
    int64_t blocks = (items + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 8 * 4;
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace mpt

using namespace mpt;

extern "C" {

int mpt_mx_quantize(const float* in, float* out, uint8_t* scales, uint8_t* codes, int64_t rows, int64_t cols, int block,
                    int elem_format, void* stream) {
    MPT_REQUIRE(rows >= 0 && cols >= 0 && block >= 1, "mx_quantize: bad extents");
    MPT_REQUIRE(codes == nullptr || elem_format != MPT_ELEM_E2M1 || block % 2 == 0,
                "mx_quantize: packed E2M1 codes need an even block size");
    MPT_REQUIRE(elem_format == MPT_ELEM_E4M3 || elem_format == MPT_ELEM_E2M1, "mx_quantize: unknown element format %d", elem_format);
    if (rows == 0 || cols == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "mx_quantize: null pointer");
    const ElemFmt ef = elem_format == MPT_ELEM_E4M3 ? ElemFmt::make(4, 3, 448.0f) : ElemFmt::make(2, 1, 6.0f);
    const int emax_elem = elem_format == MPT_ELEM_E4M3 ? 8 : 2;
    const int fp4 = elem_format == MPT_ELEM_E2M1;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(codes) & 3u) == 0;
    cudaStream_t st = as_stream(stream);
    if (aligned && cols % block == 0 && (block == 32 || block == 16)) {
        const int64_t nvec = rows * cols / 4;
        auto kern = block == 32 ? (codes ? mx_kernel<8, true> : mx_kernel<8, false>) : (codes ? mx_kernel<4, true> : mx_kernel<4, false>);
        kern<<<stream_blocks(nvec), kThreads, 0, st>>>(reinterpret_cast<const float4*>(in), reinterpret_cast<float4*>(out), scales, codes, fp4, nvec, ef, emax_elem);
    } else {
        const int64_t nblk = rows * ((cols + block - 1) / block);
        mx_generic_kernel<<<stream_blocks(nblk), kThreads, 0, st>>>(in, out, scales, codes, fp4, rows, cols, block, ef, emax_elem);
    }
    return check_launch("mx_quantize");
}

int mpt_nvfp4_quantize(const float* in, float* out, float* block_scales, uint8_t* codes, uint8_t* scale_codes, int64_t rows,
                       int64_t cols, float global_scale, void* workspace, float* global_scale_out, void* stream) {
    MPT_REQUIRE(rows >= 0 && cols >= 0, "nvfp4_quantize: bad extents");
    if (rows == 0 || cols == 0) return MPT_OK;
    MPT_REQUIRE(in && out, "nvfp4_quantize: null pointer");
    MPT_REQUIRE(global_scale > 0.f || workspace != nullptr,
                "nvfp4_quantize: pass a positive global_scale, or 4 bytes of device workspace to compute it");
    cudaStream_t st = as_stream(stream);
    uint32_t* amax_bits = static_cast<uint32_t*>(workspace);
    if (!(global_scale > 0.f)) {
        amax_init_kernel<<<1, 1, 0, st>>>(amax_bits);
        amax_kernel<<<stream_blocks(rows * cols / 4 + 1), kThreads, 0, st>>>(in, rows * cols, amax_bits);
    }
    const Nvfp4Fmt f{ElemFmt::make(4, 3, 448.0f), ElemFmt::make(2, 1, 6.0f)};
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(codes) & 1u) == 0;
    if (aligned && cols % 16 == 0) {
        const int64_t nvec = rows * cols / 4;
        auto kern = (codes != nullptr || scale_codes != nullptr) ? nvfp4_kernel<true> : nvfp4_kernel<false>;
        kern<<<stream_blocks(nvec), kThreads, 0, st>>>(reinterpret_cast<const float4*>(in), reinterpret_cast<float4*>(out),
                                                      block_scales, codes, scale_codes, nvec, global_scale, amax_bits, global_scale_out, f);
    } else {
        nvfp4_generic_kernel<<<stream_blocks(rows * ((cols + 15) / 16)), kThreads, 0, st>>>(in, out, block_scales, codes, scale_codes, rows, cols,
                                                                                     global_scale, amax_bits, global_scale_out, f);
    }
    return check_launch("nvfp4_quantize");
}

}
