// Register-resident softmax forward rows (see reduce.cuh for the scheme).
// Compiled with nvcc's default floating-point flags like reduce.cu: expf must match the reference's CUDA build.
#include "reduce.cuh"

namespace mpt {
namespace {

template <int JMAX, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_fwd_rows_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                              int64_t rows, int C, const __grid_constant__ Caster fexp,
                                                                              const __grid_constant__ Caster foff,
                                                                              const __grid_constant__ Caster facc, RowLimits lim) {
    constexpr bool TRUSTED = MODE != 0;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    float* y = out + row * C;
    float v[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        v[j] = x[lane + 32 * j];
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2)
        { m0 = fmaxf(m0, v[j]); m1 = fmaxf(m1, v[j + 1]); }
    const float mx = tree64(m0, m1, FMax{});
    bool ok = true, odd = false;
    {
        const RAdd<MODE> qadd{facc, odd};
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < JMAX; j += 2)
            {
                const float d0 = __fsub_rn(v[j], mx), d1 = __fsub_rn(v[j + 1], mx);
                float e0 = rr<MODE>(fexp, expf(rr<MODE>(foff, d0, odd)), odd);
                float e1 = rr<MODE>(fexp, expf(rr<MODE>(foff, d1, odd)), odd);
                if (TRUSTED) {
                    // x - max <= -128 (masked entries, -inf included) rounds to a value <= -128 in any format that reaches
                    // 128, whose exponential is exactly zero; everything else lies in (-128, 0], inside the fast range.
                    // A NaN difference fails the comparison and poisons the sum, which sends the row to the fallback.
                    e0 = d0 <= -128.0f ? 0.0f : e0;
                    e1 = d1 <= -128.0f ? 0.0f : e1;
                }
                v[j] = e0; v[j + 1] = e1;
                s0 = qadd(s0, e0); s1 = qadd(s1, e1);
            }
        const float sum = tree64(s0, s1, qadd);
        if (TRUSTED) {
            // the addends are non-negative, so the total bounds every partial sum; a NaN element ends up here as well
            ok = sum >= 1.0f && sum < lim.top[2] && sum <= 0x1p20f && fabsf(mx) < 3.0e38f;
            if (ok) {
                const float r = __frcp_rn(sum);
#pragma unroll
                for (int j = 0; j < JMAX; ++j) v[j] = row_div<MODE>(v[j], sum, r, odd);
                if (MODE >= 2) ok = !__any_sync(0xFFFFFFFFu, odd);
                if (ok) {
#pragma unroll
                    for (int j = 0; j < JMAX; ++j) y[lane + 32 * j] = v[j];
                    return;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < JMAX; ++j)
                y[lane + 32 * j] = __fdiv_rn(v[j], sum);
            return;
        }
    }
    softmax_fwd_row_cold(x, y, C, lane, &fexp, &foff, &facc);
}

}  // namespace

void launch_softmax_fwd_rows(const float* in, float* out, const RowGeom& g, const Caster& fe, const Caster& fo, const Caster& fa,
                             int mode, const RowLimits& lim, void* stream) {
    MPT_ROWS_DISPATCH_WIDE(softmax_fwd_rows_kernel, mode, in, out, g.rows, g.channel, fe, fo, fa, lim);
}

}  // namespace mpt
