// GEMM for rounding formats the FP-pipe rounding does not cover (supernormal float, binary8, float formats without
// subnormals or with 22-23 mantissa bits below 8 exponent bits): every rounding is the exact caster, 60-200
// instructions with data-dependent branches, so the kernel is bound by those and shaped for them rather than for
// operand reuse: one warp-wide row of 32 outputs per warp step, four outputs per thread as independent chains, many
// resident warps (about 40 registers per thread), the casters inlined once per format kind.  The accumulation
// orders, the zero padding of the CUDA order and the continuation from the sums held in C are those of mm_kernel.
#include "gemm_kernel.cuh"

namespace mpt {
namespace {

constexpr int XT = 32;        // tile edge: 32 x 32 outputs, K slabs of 32
constexpr int XPER = 4;       // outputs per thread: rows ty, ty + 8, ty + 16, ty + 24 of column tx

// One format as this kernel rounds to it.  KIND 0: a float format, exact caster; 2: supernormal; 3: binary8 (that caster
// alone is inlined); 1: any mixture (cast_any); 4: float formats the FP-pipe rounding covers, through its whole-domain
// form (FullRn: what reaches this kernel with such formats are products whose operands ruled the range-checked path
// out, and compensated sums of fp32-accumulating formats); 5: float formats without subnormals, the settling rounding
// with the exact caster behind one compare for fp32 denormals, overflow, infinities and NaN.
struct Rounding {
    AnyFmt any;
    FullRn full;
    uint32_t span;
    __device__ __forceinline__ static Rounding make(const AnyFmt& f) {
        Rounding r;
        r.any = f;
        r.full = FullRn::make(f.fp);
        const uint32_t top = r.full.ovf_from < r.full.exact_from ? r.full.ovf_from : r.full.exact_from;
        r.span = top - 0x00800000u;
        return r;
    }
};
template <int KIND>
__device__ __forceinline__ float round_to(float x, const Rounding& r) {
    const AnyFmt& f = r.any;
    if (KIND == 0) return cast_fp_nearest(x, f.fp);
    if (KIND == 2) return cast_superfp(x, f.fp.man, f.fp.exp, f.bl, f.bu, f.fp.sat != 0);
    if (KIND == 3) return cast_binary8(x, f.P, f.is_signed != 0, f.policy, f.fp.sub != 0, RND_NEAREST, 0u, 0);
    if (KIND == 4) return fmt_identity(f.fp) ? x : r.full(x);
    if (KIND == 5) {
        const uint32_t a = __float_as_uint(x) & 0x7FFFFFFFu;
        if (a == 0u) return x;
        if (a - 0x00800000u >= r.span) return cast_fp_nearest(x, f.fp);
        return fast_rn_nosub(r.full.fast, x);
    }
    return cast_any(x, f);
}

template <int ALGO, bool FMA, int KIND>
__global__ void __launch_bounds__(256) exact_mm_kernel(const __grid_constant__ MmParams p, int64_t nbatch) {
    __shared__ float As[XT][XT + 1];
    __shared__ float Bs[XT][XT];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int tiles_n = (p.N + XT - 1) / XT, tiles_m = (p.M + XT - 1) / XT;
    const int64_t per_entry = (int64_t)tiles_n * tiles_m, total = per_entry * nbatch;
    const int ksteps = (ALGO == ALGO_SEQ || (p.resume & MM_MORE)) ? p.K : p.K + 8 - p.K % 8;
    // a CTA walks tiles (a grid of a few CTAs per SM): launched behind mm_kernel for the same product it usually has
    // nothing to do, and finding that out must cost microseconds whatever the size of the product
    int64_t planned = -1;       // batch entry the verdict below belongs to (reading the statistics costs a trip to L2)
    bool taken = false;         // mm_kernel computed that entry
    for (int64_t tile = blockIdx.x; tile < total; tile += gridDim.x) {
    const int64_t batch = tile / per_entry;
    const int in_entry = (int)(tile - batch * per_entry);
    // only the batch entries mm_kernel left alone
    if (p.defer_exact && batch != planned) { planned = batch; taken = make_plan<ALGO, FMA>(p, batch).ok; }
    if (p.defer_exact && taken) continue;
    const int m0 = (in_entry / tiles_n) * XT, n0 = (in_entry % tiles_n) * XT;
    const float* A = p.a + batch * p.stride_a;
    const float* B = p.b + batch * p.stride_b;
    float* C = p.c + batch * p.stride_c;
    const int gn = n0 + tx;

    const Rounding qa = Rounding::make(p.gadd), qm = Rounding::make(p.gmul);
    float run[XPER], outer[XPER];       // the running (inner) sum; the outer sum of the CUDA order / the compensation term
#pragma unroll
    for (int i = 0; i < XPER; ++i) {
        run[i] = 0.0f; outer[i] = 0.0f;
        if (p.resume & MM_FROM_C) {
            const int gm = m0 + ty + 8 * i;
            const float v = (gm < p.M && gn < p.N) ? C[(int64_t)gm * p.N + gn] : 0.0f;
            if (ALGO == ALGO_TILE8) outer[i] = v; else run[i] = v;
        }
    }
    for (int k0 = 0; k0 < ksteps; k0 += XT) {
#pragma unroll
        for (int i = 0; i < XPER; ++i) {
            const int r = ty + 8 * i;
            const int gm = m0 + r, gk = k0 + tx;
            As[r][tx] = (gm < p.M && gk < p.K) ? A[(int64_t)gm * p.K + gk] : 0.0f;
            const int bk = k0 + r;
            Bs[r][tx] = (bk < p.K && gn < p.N) ? B[(int64_t)bk * p.N + gn] : 0.0f;
        }
        __syncthreads();
        const int nk = min(XT, ksteps - k0);
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const float b = Bs[k][tx];
#pragma unroll
            for (int i = 0; i < XPER; ++i) {
                const float a = As[ty + 8 * i][k];
                if (ALGO == ALGO_KAHAN) {
                    // y = Q(product - comp); t = Q(sum + y); comp = Q(Q(t - sum) - y); sum = t   (mm_kernel.h:457-520)
                    const float y = FMA ? round_to<KIND>(fma_rn(a, b, -outer[i]), qa)
                                        : round_to<KIND>(add_rn(round_to<KIND>(mul_rn(a, b), qm), -outer[i]), qa);
                    const float t = round_to<KIND>(add_rn(run[i], y), qa);
                    outer[i] = round_to<KIND>(add_rn(round_to<KIND>(add_rn(t, -run[i]), qa), -y), qa);
                    run[i] = t;
                } else {
                    run[i] = FMA ? round_to<KIND>(fma_rn(a, b, run[i]), qa)
                                 : round_to<KIND>(add_rn(run[i], round_to<KIND>(mul_rn(a, b), qm)), qa);
                }
            }
            if (ALGO == ALGO_TILE8 && ((k0 + k) & 7) == 7) {
#pragma unroll
                for (int i = 0; i < XPER; ++i) { outer[i] = round_to<KIND>(add_rn(outer[i], run[i]), qa); run[i] = 0.0f; }
            }
        }
        __syncthreads();
    }
    if (gn < p.N) {
#pragma unroll
        for (int i = 0; i < XPER; ++i) {
            const int gm = m0 + ty + 8 * i;
            if (gm < p.M) C[(int64_t)gm * p.N + gn] = ALGO == ALGO_TILE8 ? outer[i] : run[i];
        }
    }
    }   // tiles
}

template <int ALGO, bool FMA>
int launch_exact(const MmParams& p, int64_t batch, cudaStream_t st) {
    const int64_t tiles = (((int64_t)p.M + XT - 1) / XT) * (((int64_t)p.N + XT - 1) / XT) * batch;
    const int64_t cap = (int64_t)sm_count() * 8;
    const dim3 grid((unsigned)(tiles < cap ? tiles : cap));
    const int ka = p.gadd.kind, km = p.gmul.kind;          // run_mm sets gmul = gadd for the fused form
    const auto covered = [](const FpFmt& f) { return fast_rn_supported(f) || fmt_identity(f); };
    if (ka == FMT_FLOAT && km == FMT_FLOAT && covered(p.gadd.fp) && covered(p.gmul.fp)) exact_mm_kernel<ALGO, FMA, 4><<<grid, 256, 0, st>>>(p, batch);
    else if (ka == FMT_FLOAT && km == FMT_FLOAT && mm_fast_format_nosub(p.gadd.fp) && mm_fast_format_nosub(p.gmul.fp))
        exact_mm_kernel<ALGO, FMA, 5><<<grid, 256, 0, st>>>(p, batch);
    else if (ka == FMT_FLOAT && km == FMT_FLOAT) exact_mm_kernel<ALGO, FMA, 0><<<grid, 256, 0, st>>>(p, batch);
    else if (ka == FMT_SUPERFP && km == FMT_SUPERFP) exact_mm_kernel<ALGO, FMA, 2><<<grid, 256, 0, st>>>(p, batch);
    else if (ka == FMT_BINARY8 && km == FMT_BINARY8) exact_mm_kernel<ALGO, FMA, 3><<<grid, 256, 0, st>>>(p, batch);
    else exact_mm_kernel<ALGO, FMA, 1><<<grid, 256, 0, st>>>(p, batch);
    return check_launch("float_mm");
}

}  // namespace

int launch_mm_exact(int algo, bool fma, const MmParams& p, int64_t batch, cudaStream_t st) {
    if (algo == ALGO_SEQ) return fma ? launch_exact<ALGO_SEQ, true>(p, batch, st) : launch_exact<ALGO_SEQ, false>(p, batch, st);
    if (algo == ALGO_KAHAN) return fma ? launch_exact<ALGO_KAHAN, true>(p, batch, st) : launch_exact<ALGO_KAHAN, false>(p, batch, st);
    return fma ? launch_exact<ALGO_TILE8, true>(p, batch, st) : launch_exact<ALGO_TILE8, false>(p, batch, st);
}

}  // namespace mpt
