// Register-resident layer-normalisation forward rows (see reduce.cuh for the scheme).
// Compiled with nvcc's default floating-point flags like reduce.cu: expf must match the reference's CUDA build.
#include "reduce.cuh"

namespace mpt {
namespace {

template <int JMAX, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_fwd_rows_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                                                const float* __restrict__ bias, float* __restrict__ out,
                                                                                float* __restrict__ mean, float* __restrict__ rstd, float eps,
                                                                                int64_t rows, int C, const __grid_constant__ LnFmt f,
                                                                                RowLimits lim) {
    constexpr bool TRUSTED = MODE != 0;
    // Pairs of roundings as packed fp32x2 operations: 5 % faster where every format has fewer than 8 exponent bits;
    // with the bookkeeping of the 8-bit-exponent mode the packed form is slower (more register moves), so that mode
    // keeps the scalar form.
    constexpr bool PAIRS = MODE == 1;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    float* y = out + row * C;
    const float fC = (float)C;
    bool odd = false;
    const RAdd<MODE> qacc{f.acc, odd};
    float v[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        v[j] = x[lane + 32 * j];
    float s0 = 0.f, s1 = 0.f, xm = 0.f, xa = 0.f;
    if (PAIRS) {
        // the two partial sums of a lane advance as one packed pair
        float2 s = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < JMAX; j += 2) {
            xm = fmaxf(xm, fmaxf(fabsf(v[j]), fabsf(v[j + 1])));
            xa = __fadd_rn(xa, __fadd_rn(fabsf(v[j]), fabsf(v[j + 1])));
            s = rr2<MODE>(f.acc, __fadd2_rn(s, make_float2(v[j], v[j + 1])), odd);
        }
        s0 = s.x; s1 = s.y;
    } else {
#pragma unroll
        for (int j = 0; j < JMAX; j += 2) {
            if (TRUSTED) {
                xm = fmaxf(xm, fmaxf(fabsf(v[j]), fabsf(v[j + 1])));
                xa = __fadd_rn(xa, __fadd_rn(fabsf(v[j]), fabsf(v[j + 1])));
            }
            s0 = qacc(s0, v[j]); s1 = qacc(s1, v[j + 1]);
        }
    }
    const float sum = tree64(s0, s1, qacc);
    const float m = __fdiv_rn(sum, fC);
    bool ok = true;
    float dm = 0.f;
    if (TRUSTED) {
        xm = warp_max_nonneg(xm);
        const float sb = warp_sum_bound(xa) * lim.growth;        // bound of every partial sum of the row
        dm = (xm + fabsf(m)) * lim.slack;                        // bound of |Q(x - mean)|
        ok = sb < lim.top[0] && fabsf(sum) <= sb && dm < lim.top[0] && dm * dm * lim.slack < lim.top[1];
    }
    if (ok) {
        s0 = 0.f; s1 = 0.f;
        if (PAIRS) {
            float2 s = make_float2(0.f, 0.f);
            const float2 nm = make_float2(-m, -m);                     // x - m is x + (-m)
#pragma unroll
            for (int j = 0; j < JMAX; j += 2) {
                const float2 d = rr2<MODE>(f.acc, __fadd2_rn(make_float2(v[j], v[j + 1]), nm), odd);
                v[j] = d.x; v[j + 1] = d.y;
                s = rr2<MODE>(f.acc, __fadd2_rn(s, rr2<MODE>(f.mul, __fmul2_rn(d, d), odd)), odd);
            }
            s0 = s.x; s1 = s.y;
        } else {
#pragma unroll
            for (int j = 0; j < JMAX; j += 2) {
                const float d0 = rr<MODE>(f.acc, __fsub_rn(v[j], m), odd), d1 = rr<MODE>(f.acc, __fsub_rn(v[j + 1], m), odd);
                v[j] = d0; v[j + 1] = d1;
                s0 = qacc(s0, rr<MODE>(f.mul, __fmul_rn(d0, d0), odd));
                s1 = qacc(s1, rr<MODE>(f.mul, __fmul_rn(d1, d1), odd));
            }
        }
        const float vsum = tree64(s0, s1, qacc);
        const float var = __fdiv_rn(vsum, fC);
        // per-row scalars take the whole-domain rounding
        const float sd = cast_fp_nearest(__fsqrt_rn(cast_fp_nearest(__fadd_rn(var, eps), f.acc)), f.sqrt);
        float rs = 0.f;
        if (TRUSTED) {
            // the squares are non-negative, so their total bounds every partial sum of theirs
            ok = vsum < lim.top[0] && sd >= 0x1p-20f && sd <= 0x1p20f;
            rs = __frcp_rn(sd);
            ok = ok && dm * rs * 1.001f < lim.top[2];
        }
        if (ok) {
            float pm = 0.f;
            if (PAIRS) {
#pragma unroll
                for (int j = 0; j < JMAX; j += 2) {
                    const float2 q = row_div2<MODE>(make_float2(v[j], v[j + 1]), sd, rs, odd);
                    const float2 p = __fmul2_rn(make_float2(w[lane + 32 * j], w[lane + 32 * (j + 1)]), rr2<MODE>(f.div, q, odd));
                    pm = fmaxf(pm, fmaxf(fabsf(p.x), fabsf(p.y)));
                    const float2 o = __fadd2_rn(rr2<MODE>(f.mul, p, odd), make_float2(bias[lane + 32 * j], bias[lane + 32 * (j + 1)]));
                    v[j] = o.x; v[j + 1] = o.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < JMAX; ++j) {
                    const float q = TRUSTED ? row_div<MODE>(v[j], sd, rs, odd) : __fdiv_rn(v[j], sd);
                    const float p = __fmul_rn(w[lane + 32 * j], rr<MODE>(f.div, q, odd));
                    if (TRUSTED) pm = fmaxf(pm, fabsf(p));
                    v[j] = __fadd_rn(rr<MODE>(f.mul, p, odd), bias[lane + 32 * j]);
                }
            }
            if (TRUSTED) {
                pm = warp_max_nonneg(pm);
                // fmaxf skips a NaN product (a NaN weight); the trusted rounding turns it into NaN as the exact one does
                ok = pm < lim.top[1];
                if (MODE >= 2) ok = ok && !__any_sync(0xFFFFFFFFu, odd);
            }
            if (ok) {
#pragma unroll
                for (int j = 0; j < JMAX; ++j)
                    y[lane + 32 * j] = v[j];
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

}  // namespace

void launch_layernorm_fwd_rows(const float* in, const float* weight, const float* bias, float* out, float* mean, float* rstd, float eps,
                               const RowGeom& g, const LnFmt& f, int mode, const RowLimits& lim, void* stream) {
    MPT_ROWS_DISPATCH_WIDE(layernorm_fwd_rows_kernel, mode, in, weight, bias, out, mean, rstd, eps, g.rows, g.channel, f, lim);
}

}  // namespace mpt
