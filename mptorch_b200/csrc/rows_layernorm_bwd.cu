// Register-resident layer-normalisation input-gradient rows (see reduce.cuh for the scheme).
// Compiled with nvcc's default floating-point flags like reduce.cu: expf must match the reference's CUDA build.
#include "reduce.cuh"

namespace mpt {
namespace {

template <int JMAX, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_bwd_rows_kernel(const float* __restrict__ in, const float* __restrict__ gout,
                                                                                const float* __restrict__ w, const float* __restrict__ mean,
                                                                                const float* __restrict__ rstd, float* __restrict__ gin,
                                                                                int64_t rows, int C, const __grid_constant__ LnFmt f,
                                                                                RowLimits lim) {
    constexpr bool TRUSTED = MODE != 0;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    const float* gr = gout + row * C;
    float* o = gin + row * C;
    const float fC = (float)C;
    const float m = mean[row], r = rstd[row];
    bool odd = false;
    const RAdd<MODE> qacc{f.acc, odd};
    float xh[JMAX], ng[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        { xh[j] = x[lane + 32 * j]; ng[j] = __fmul_rn(w[lane + 32 * j], gr[lane + 32 * j]); }
    float xm = 0.f, gm = 0.f, ga = 0.f;
    if (TRUSTED) {
#pragma unroll
        for (int j = 0; j < JMAX; ++j)
            { xm = fmaxf(xm, fabsf(xh[j])); gm = fmaxf(gm, fabsf(ng[j])); ga = __fadd_rn(ga, fabsf(ng[j])); }
        xm = warp_max_nonneg(xm); gm = warp_max_nonneg(gm);
        ga = warp_sum_bound(ga);
    }
    bool ok = true;
    float hb = 0.f, sa = 0.f, sb = 0.f;
    if (TRUSTED) {
        const float dm = (xm + fabsf(m)) * lim.slack;            // bound of |Q(x - mean)|
        hb = dm * fabsf(r) * lim.slack;                          // bound of |x-hat|
        sa = ga * lim.slack * lim.growth;                        // bound of the partial sums of w * dy
        sb = hb * sa * lim.slack;                                // bound of the partial sums of x-hat * w * dy
        ok = dm < lim.top[0] && hb < lim.top[1] && gm < lim.top[1] && hb * gm * lim.slack < lim.top[1] && sa < lim.top[0] &&
             sb < lim.top[0];
    }
    if (ok) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int j = 0; j < JMAX; j += 2)
            {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float h = rr<MODE>(f.mul, __fmul_rn(rr<MODE>(f.acc, __fsub_rn(xh[j + u], m), odd), r), odd);
                    const float n = rr<MODE>(f.mul, ng[j + u], odd);
                    xh[j + u] = h; ng[j + u] = n;
                    const float dot = rr<MODE>(f.mul, __fmul_rn(h, n), odd);
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
            for (int j = 0; j < JMAX; ++j) {
                const float wg = rr<MODE>(f.mul, __fmul_rn(xh[j], gsx), odd);
                float gi = rr<MODE>(f.acc, __fsub_rn(ng[j], gs), odd);
                gi = rr<MODE>(f.acc, __fsub_rn(gi, wg), odd);
                xh[j] = rr<MODE>(f.mul, __fmul_rn(gi, r), odd);
            }
            if (MODE >= 2) ok = !__any_sync(0xFFFFFFFFu, odd);
            if (ok) {
#pragma unroll
                for (int j = 0; j < JMAX; ++j) o[lane + 32 * j] = xh[j];
                return;
            }
        }
    }
    layernorm_bwd_row_cold(x, gr, w, m, r, o, C, lane, &f);
}

}  // namespace

void launch_layernorm_bwd_rows(const float* in, const float* grad_out, const float* weight, const float* mean, const float* rstd,
                               float* grad_in, const RowGeom& g, const LnFmt& f, int mode, const RowLimits& lim, void* stream) {
    MPT_ROWS_DISPATCH(layernorm_bwd_rows_kernel, mode, in, grad_out, weight, mean, rstd, grad_in, g.rows, g.channel, f, lim);
}

}  // namespace mpt
