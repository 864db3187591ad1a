// Register-resident softmax forward rows, log-sum-exp form (see reduce.cuh for the scheme).
// Compiled with nvcc's default floating-point flags like reduce.cu: expf / logf must match the reference's CUDA build.
#include "reduce.cuh"

namespace mpt {
namespace {

// l (op) v = Q(log(exp(l) + exp(v))).  An all-masked prefix gives log(0) = -inf, which the exact rounding passes
// through and the bare FP-pipe rounding would not.
template <int MODE>
struct RLse {
    const Caster& c;
    bool& odd;
    __device__ __forceinline__ float operator()(float a, float b) const {
        const float t = logf(__fadd_rn(expf(a), expf(b)));
        const float r = rr<MODE>(c, t, odd);
        return (MODE != 0 && t == -INFINITY) ? t : r;
    }
};

template <int JMAX, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) softmax_lse_rows_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                              int64_t rows, int C, const __grid_constant__ Caster foff,
                                                                              const __grid_constant__ Caster flse) {
    constexpr bool TRUSTED = MODE != 0;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* x = in + row * C;
    float* y = out + row * C;
    float v[JMAX];
#pragma unroll
    for (int j = 0; j < JMAX; ++j) v[j] = x[lane + 32 * j];
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2) { m0 = fmaxf(m0, v[j]); m1 = fmaxf(m1, v[j + 1]); }
    const float mx = tree64(m0, m1, FMax{});
    bool odd = false;
    const RLse<MODE> qlse{flse, odd};
    float l0 = -INFINITY, l1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < JMAX; j += 2) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const float d = __fsub_rn(v[j + u], mx);
            float q = rr<MODE>(foff, d, odd);
            // x - max <= -128 (masked entries, -inf included): its rounded value is <= -128 in a format that reaches 256,
            // so its exponential is an exact zero and so is the final output; -128 stands in for it on the fast path.
            // A NaN difference fails the comparison and poisons the log-sum, which sends the row to the fallback.
            if (TRUSTED) q = d <= -128.0f ? -128.0f : q;
            v[j + u] = q;
            if (u == 0) l0 = qlse(l0, q); else l1 = qlse(l1, q);
        }
    }
    const float lgs = tree64(l0, l1, qlse);
    bool ok = true;
    if (TRUSTED) ok = fabsf(lgs) < 128.0f && fabsf(mx) < 3.0e38f;      // false for NaN and infinities
    if (ok) {
#pragma unroll
        for (int j = 0; j < JMAX; ++j) v[j] = expf(rr<MODE>(foff, __fsub_rn(v[j], lgs), odd));
        if (MODE >= 2) ok = !__any_sync(0xFFFFFFFFu, odd);
        if (ok) {
#pragma unroll
            for (int j = 0; j < JMAX; ++j) y[lane + 32 * j] = v[j];
            return;
        }
    }
    softmax_lse_row_cold(x, y, C, lane, &foff, &flse);
}

}  // namespace

void launch_softmax_lse_rows(const float* in, float* out, const RowGeom& g, const Caster& fo, const Caster& fl, int mode, void* stream) {
    MPT_ROWS_DISPATCH(softmax_lse_rows_kernel, mode, in, out, g.rows, g.channel, fo, fl);
}

}  // namespace mpt
