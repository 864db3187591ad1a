// Register-resident softmax backward rows (see reduce.cuh for the scheme).
// Compiled with nvcc's default floating-point flags like reduce.cu: expf must match the reference's CUDA build.
#include "reduce.cuh"

namespace mpt {
namespace {

template <int JMAX, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_bwd_rows_kernel(const float* __restrict__ yv, const float* __restrict__ gv,
                                                                              float* __restrict__ out, int64_t rows, int C,
                                                                              const __grid_constant__ Caster fadd,
                                                                              const __grid_constant__ Caster fmul, RowLimits lim) {
    constexpr bool TRUSTED = MODE != 0;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* y = yv + row * C;
    const float* gr = gv + row * C;
    float* o = out + row * C;
    float a[JMAX], b[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j)
        { a[j] = y[lane + 32 * j]; b[j] = gr[lane + 32 * j]; }
    bool odd = false;
    const RAdd<MODE> qadd{fadd, odd};
    float s0 = 0.f, s1 = 0.f, pm = 0.f, gm = 0.f, pa = 0.f;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2)
        {
            const float p0 = __fmul_rn(a[j], b[j]), p1 = __fmul_rn(a[j + 1], b[j + 1]);
            if (TRUSTED) {
                pm = fmaxf(pm, fmaxf(fabsf(p0), fabsf(p1)));
                pa = __fadd_rn(pa, __fadd_rn(fabsf(p0), fabsf(p1)));
                gm = fmaxf(gm, fmaxf(fabsf(b[j]), fabsf(b[j + 1])));
            }
            s0 = qadd(s0, rr<MODE>(fmul, p0, odd));
            s1 = qadd(s1, rr<MODE>(fmul, p1, odd));
        }
    const float s = tree64(s0, s1, qadd);
    bool ok = true;
    if (TRUSTED) {
        pm = warp_max_nonneg(pm); gm = warp_max_nonneg(gm);
        pa = warp_sum_bound(pa);
        // fmaxf skips NaN, so the inputs' finiteness is established through the sums below: a NaN or infinite input
        // makes s NaN or infinite (inf * 0 and inf - inf included)
        const float sb = pa * lim.slack * lim.growth;                            // bound of every partial sum
        ok = pm < lim.top[1] && sb < lim.top[0] && (gm + sb) * lim.slack < lim.top[0] && fabsf(s) <= sb;
    }
    if (ok) {
#pragma unroll
        for (int j = 0; j < JMAX; ++j) b[j] = __fmul_rn(rr<MODE>(fadd, __fsub_rn(b[j], s), odd), a[j]);
        if (MODE >= 2) ok = !__any_sync(0xFFFFFFFFu, odd);
        if (ok) {
#pragma unroll
            for (int j = 0; j < JMAX; ++j) o[lane + 32 * j] = b[j];
            return;
        }
    }
    softmax_bwd_row_cold(y, gr, o, C, lane, &fadd, &fmul);
}

}  // namespace

void launch_softmax_bwd_rows(const float* y, const float* grad, float* out, const RowGeom& g, const Caster& fa, const Caster& fm,
                             int mode, const RowLimits& lim, void* stream) {
    MPT_ROWS_DISPATCH(softmax_bwd_rows_kernel, mode, y, grad, out, g.rows, g.channel, fa, fm, lim);
}

}  // namespace mpt
