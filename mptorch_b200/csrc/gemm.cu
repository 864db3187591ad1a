// C entry points of the per-MAC rounded GEMM and of the implicit-GEMM convolution: argument checks, operand
// statistics, problem set-up.  The kernel lives in gemm_kernel.cuh, its instantiations in gemm_*.cu.
#include <cmath>

#include "gemm_kernel.cuh"

namespace mpt {
namespace {

double growth8_bound(int man) {
    double g = 1.0, f = 1.0 + ldexp(1.0, -(man + 1));
    for (int i = 0; i < 8; ++i) g *= f;
    return g * 1.0001;
}

// Bounds for the Kahan fast path.  One step maps the magnitudes S = |sum|, C = |comp| and the product bound P to
//     Y  <= g (P + C) + d            y = Q(update - comp)
//     T  <= g (S + Y) + d            t = Q(sum + y),  |t - (sum + y)| <= E = u (S + Y) + d
//     C1 <= g (Y + E) + d            c1 = Q(t - sum), t - sum = y + e with |e| <= E (the fp32 subtraction adds 2^-24)
//     C' <= g (E + u (Y + E) + d) + d
// with u = 2^-(man+1) the relative rounding error of the add format, g = 1 + u, and d = 2^min_exp covering the absolute
// error of roundings that land in the subnormal range.  Every bound is linear with non-negative coefficients in
// (S, C, P, d), so the largest intermediate of eight steps is at most sc * max(S, C) + cp * P + cd * d, where each
// coefficient is the largest one seen for its variable; the kernel keeps a group on the fast path while that stays
// below the add format's fast-rounding limit.
struct KahanBounds { double sc, p, d; };
KahanBounds kahan_bounds(int man) {
    const double u = ldexp(1.0, -(man + 1)), g = (1.0 + u) * (1.0 + ldexp(1.0, -23));
    // vectors of coefficients over (S0, C0, P, d)
    struct V { double v[4]; };
    auto add = [](V a, V b) { V r; for (int i = 0; i < 4; ++i) r.v[i] = a.v[i] + b.v[i]; return r; };
    auto mul = [](V a, double k) { V r; for (int i = 0; i < 4; ++i) r.v[i] = a.v[i] * k; return r; };
    V S{{1, 0, 0, 0}}, C{{0, 1, 0, 0}}, P{{0, 0, 1, 0}}, D{{0, 0, 0, 1}}, top{{0, 0, 0, 0}};
    auto see = [&](V x) { for (int i = 0; i < 4; ++i) top.v[i] = x.v[i] > top.v[i] ? x.v[i] : top.v[i]; };
    see(S); see(C);
    for (int step = 0; step < 8; ++step) {
        V Y = add(mul(add(P, C), g), D);
        V T = add(mul(add(S, Y), g), D);
        V E = add(mul(add(S, Y), u), D);
        V C1 = add(mul(add(Y, E), g), D);
        V Cn = add(mul(add(add(E, mul(add(Y, E), u)), D), g), D);
        see(Y); see(T); see(C1); see(Cn);
        S = T; C = Cn;
    }
    return KahanBounds{(top.v[0] + top.v[1]) * 1.001, top.v[2] * 1.001, top.v[3] * 1.001};
}

int run_mm(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, const AnyFmt& gadd, const AnyFmt& gmul_in,
           int rbits_add, int rbits_mul, bool fma_in, int algo, uint64_t seed, void* workspace, size_t workspace_bytes,
           cudaStream_t st, int resume = 0) {
    // A multiply format that rounds nothing leaves `sum + a * b` in the reference's CUDA kernel (mm_kernel.h:53), and
    // its build contracts that into one fused multiply-add (measured: its results equal the fused variant with the
    // add format, not the separately rounded product).  The CUDA order follows the CUDA build; the sequential order
    // follows the CPU build, which multiplies and adds separately.
    const bool contracted = !fma_in && algo == ALGO_TILE8 && gadd.kind == FMT_FLOAT && gmul_in.kind == FMT_FLOAT && fmt_identity(gmul_in.fp);
    const bool fma = fma_in || contracted;
    const AnyFmt gmul = contracted ? gadd : gmul_in;
    const FpFmt fadd = gadd.fp, fmul = gmul.fp;
    const bool all_float = gadd.kind == FMT_FLOAT && (fma || gmul.kind == FMT_FLOAT);
    if (batch == 0 || M == 0 || N == 0) return MPT_OK;
    if (K == 0 && (resume & MM_FROM_C)) return MPT_OK;      // nothing to add to the sums C holds
    if (K == 0) {   // an empty sum: every order yields +0
        cudaError_t e = cudaMemsetAsync(c, 0, sizeof(float) * (size_t)batch * M * N, st);
        if (e != cudaSuccess) { set_error("float_mm: cudaMemsetAsync: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
        return MPT_OK;
    }
    MmParams p;
    p.a = a; p.b = b; p.c = c;
    p.M = M; p.N = N; p.K = K;
    p.resume = resume;
    p.stride_a = (int64_t)M * K; p.stride_b = (int64_t)K * N; p.stride_c = (int64_t)M * N;
    p.fadd = fadd; p.fmul = fmul;
    p.gadd = gadd; p.gmul = fma ? gadd : gmul;
    p.radd = mm_fast_rn(fadd); p.rmul = mm_fast_rn(fmul);
    p.rbits_add = rbits_add; p.rbits_mul = rbits_mul;
    p.seed_lo = (uint32_t)seed; p.seed_hi = (uint32_t)(seed >> 32);
    p.growth8 = (float)growth8_bound(fadd.man);
    {
        const KahanBounds kb = kahan_bounds(fadd.man);
        p.kah_sc = (float)kb.sc; p.kah_p = (float)kb.p; p.kah_const = (float)(kb.d * ldexp(1.0, fadd.min_exp));
        p.growth8_sr = (float)(pow(1.0 + ldexp(1.0, -fadd.man), 8.0) * 1.0001);
    }
    p.stats = nullptr;
    p.whole_ok = all_float && fast_rn_supported(fadd) && (fma || fast_rn_supported(fmul));
    p.wadd = FullRn::make(fadd); p.wmul = FullRn::make(fma ? fadd : fmul);
    p.sr_ok = all_float && FullSr::supported(fadd) && (fma || FullSr::supported(fmul));
    p.sadd = FullSr::make(fadd, rbits_add); p.smul = FullSr::make(fma ? fadd : fmul, fma ? rbits_add : rbits_mul);
    p.sr_nosub = all_float && !fadd.sub && fadd.exp >= 2 && (fma || (!fmul.sub && fmul.exp >= 2));

    // formats without subnormals: their own instantiation of the range-checked kernel (plain and sequential sums)
    const bool nosub = (algo == ALGO_SEQ || algo == ALGO_TILE8) && mm_fast_format_nosub(fadd) && (fma || mm_fast_format_nosub(fmul));
    p.nosub = nosub ? 1 : 0;
    const bool fmt_fast = algo == ALGO_SR ? (p.sr_ok != 0 || p.sr_nosub != 0) : (nosub || (mm_fast_format(fadd) && (fma || mm_fast_format(fmul))));
    const bool fast_candidate = all_float && fmt_fast && workspace != nullptr &&
                                workspace_bytes >= sizeof(MmStats) * (size_t)batch &&
                                (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0 && K > 0;
    if (fast_candidate) {
        MmStats* s = static_cast<MmStats*>(workspace);
        stats_init_kernel<<<(unsigned)((batch + 255) / 256), 256, 0, st>>>(s, batch);
        const int64_t na = (int64_t)M * K, nb = (int64_t)K * N;
        const int sms = sm_count();
        auto grid = [&](int64_t n) {
            int64_t g = (n + 255) / 256;
            const int64_t cap = ((int64_t)sms * 8 + batch - 1) / batch;
            return dim3((unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), (unsigned)batch);
        };
        stats_kernel<<<grid(na), 256, 0, st>>>(a, na, s, 0);
        stats_kernel<<<grid(nb), 256, 0, st>>>(b, nb, s, 1);
        int rc = check_launch("float_mm statistics");
        if (rc) return rc;
        p.stats = s;
    }
    const bool vec = (K % 4 == 0) && (N % 4 == 0) && (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0);
    // formats without the FP-pipe rounding: the kernel built around the exact casters
    if (algo != ALGO_SR && !(all_float && fmt_fast)) return launch_mm_exact(algo, fma, p, batch, st);
    // fewer 128-row tiles than SMs: the 16-row instantiation spreads the same outputs over eight times the CTAs
    const int64_t big_tiles = (((int64_t)M + BM - 1) / BM) * (((int64_t)N + BN - 1) / BN) * batch;
    const bool small = (algo == ALGO_SEQ || algo == ALGO_TILE8) && big_tiles < sm_count() &&
                       ((int64_t)M + kSmallTileRows - 1) / kSmallTileRows <= 65535;
    // Range-checked launch, then the exact kernel for the batch entries whose statistics rule that path out.  The
    // second launch costs a few microseconds when it has nothing to do, so only products long enough not to notice
    // (2^33 MACs, about 2 ms) get it; shorter ones keep the exact path inside mm_kernel for such entries.
    const bool defer = algo != ALGO_SR && p.stats != nullptr && (double)batch * M * N * K >= 8589934592.0;
    p.defer_exact = defer ? 1 : 0;
    if (nosub && p.stats != nullptr) {
        const int rc = launch_mm_nosub(algo, fma, p, batch, vec, st);
        return (rc || !defer) ? rc : launch_mm_exact(algo, fma, p, batch, st);
    }
    if (small || defer) {
        const int rc = small ? launch_mm_small(algo, fma, p, batch, vec, st)
                     : algo == ALGO_SEQ ? launch_mm_seq(fma, p, batch, vec, st)
                     : algo == ALGO_TILE8 ? launch_mm_tile8(fma, p, batch, vec, st) : launch_mm_kahan(fma, p, batch, vec, st);
        return (rc || !defer) ? rc : launch_mm_exact(algo, fma, p, batch, st);
    }
    switch (algo) {
        case ALGO_SEQ: return launch_mm_seq(fma, p, batch, vec, st);
        case ALGO_TILE8: return launch_mm_tile8(fma, p, batch, vec, st);
        case ALGO_KAHAN: return launch_mm_kahan(fma, p, batch, vec, st);
        default: return launch_mm_sr(fma, p, batch, vec, st);
    }
}

int run_conv(const float* x, const float* wt, float* y, int n_img, int c_in, int H, int W, int c_out, int groups, int KH, int KW,
             int sh, int sw, int ph, int pw, int dh, int dw, const FpFmt& fadd, const FpFmt& fmul, bool fma, int algo,
             void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const int OH = (H + 2 * ph - dh * (KH - 1) - 1) / sh + 1, OW = (W + 2 * pw - dw * (KW - 1) - 1) / sw + 1;
    if (n_img == 0 || c_out == 0 || OH <= 0 || OW <= 0) return MPT_OK;
    const int cg = c_in / groups, og = c_out / groups;
    const int64_t M64 = (int64_t)n_img * OH * OW, K64 = (int64_t)cg * KH * KW;
    MPT_REQUIRE(M64 <= 0x7FFFFFFF && K64 <= 0x7FFFFFFF, "float_conv2d: problem too large");
    MPT_REQUIRE((M64 + BM - 1) / BM <= 65535, "float_conv2d: more than 65535 row tiles (images x output positions too large)");
    MmParams p;
    p.cv = ConvGeom{H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, (int64_t)c_in * H * W, (int64_t)c_out * OH * OW};
    p.M = (int)M64; p.N = og; p.K = (int)K64;
    p.stride_a = p.stride_b = p.stride_c = 0;
    p.fadd = fadd; p.fmul = fma ? fadd : fmul;
    p.gadd = any_float(fadd); p.gmul = any_float(fma ? fadd : fmul);
    p.radd = FastRn::make(fadd); p.rmul = FastRn::make(p.fmul);
    p.rbits_add = p.rbits_mul = 0; p.seed_lo = p.seed_hi = 0;
    p.growth8 = (float)growth8_bound(fadd.man);
    p.stats = nullptr;
    p.whole_ok = 0; p.sr_ok = 0;
    p.kah_sc = p.kah_p = p.kah_const = 0.0f; p.growth8_sr = 1.0f;
    p.wadd = p.wmul = FullRn::make(fadd);
    p.sadd = p.smul = FullSr::make(fadd, 0);
    const bool nosub = mm_fast_format_nosub(fadd) && (fma || mm_fast_format_nosub(fmul));
    const bool fast_candidate = (nosub || (fast_rn_supported(fadd) && (fma || fast_rn_supported(fmul)))) && workspace != nullptr &&
                                workspace_bytes >= sizeof(MmStats) && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0 && K64 > 0;
    p.nosub = (nosub && fast_candidate) ? 1 : 0;
    if (K64 == 0) {
        cudaError_t e = cudaMemsetAsync(y, 0, sizeof(float) * (size_t)n_img * c_out * OH * OW, st);
        if (e != cudaSuccess) { set_error("float_conv2d: cudaMemsetAsync: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
        return MPT_OK;
    }
    if (fast_candidate) {
        // one record for all groups: the maxima over the whole input and the whole weight bound every group's products
        MmStats* s = static_cast<MmStats*>(workspace);
        stats_init_kernel<<<1, 256, 0, st>>>(s, 1);
        const int64_t nx = (int64_t)n_img * c_in * H * W, nw = (int64_t)c_out * K64;
        const int sms = sm_count();
        auto grid = [&](int64_t n) { int64_t g = (n + 255) / 256; const int64_t cap = (int64_t)sms * 8; return dim3((unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 1); };
        stats_kernel<<<grid(nx), 256, 0, st>>>(x, nx, s, 0);
        stats_kernel<<<grid(nw), 256, 0, st>>>(wt, nw, s, 1);
        int rc = check_launch("float_conv2d statistics");
        if (rc) return rc;
        p.stats = s;
    }
    for (int g = 0; g < groups; ++g) {
        p.a = x + (int64_t)g * cg * H * W;
        p.b = wt + (int64_t)g * K64 * og;
        p.c = y + (int64_t)g * og * OH * OW;
        const int rc = launch_conv_any(algo, fma, p, st);
        if (rc) return rc;
    }
    return MPT_OK;
}

// Weight gradient of the convolution as an implicit GEMM per group: M = output channels of the group, K = images x
// output positions, N = input channels of the group x KH x KW.
int run_conv_wgrad(const float* gout, const float* x, float* gw, int n_img, int c_in, int H, int W, int c_out, int groups, int KH,
                   int KW, int sh, int sw, int ph, int pw, int dh, int dw, const FpFmt& fadd, const FpFmt& fmul, bool fma, int algo,
                   void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const int OH = (H + 2 * ph - dh * (KH - 1) - 1) / sh + 1, OW = (W + 2 * pw - dw * (KW - 1) - 1) / sw + 1;
    const int cg = c_in / groups, og = c_out / groups;
    const int64_t Kw = (int64_t)cg * KH * KW;
    if (c_out == 0 || Kw == 0) return MPT_OK;
    const int64_t L = (OH > 0 && OW > 0) ? (int64_t)OH * OW : 0, K64 = (int64_t)n_img * L;
    MPT_REQUIRE(K64 <= 0x7FFFFFF0 && Kw <= 0x7FFFFFFF, "float_conv2d_wgrad: problem too large");
    if (K64 == 0) {   // no output positions: an empty sum
        cudaError_t e = cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)c_out * Kw, st);
        if (e != cudaSuccess) { set_error("float_conv2d_wgrad: cudaMemsetAsync: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
        return MPT_OK;
    }
    MmParams p;
    p.cv = ConvGeom{H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, (int64_t)c_in * H * W, (int64_t)c_out * L};
    p.M = og; p.N = (int)Kw; p.K = (int)K64;
    p.stride_a = p.stride_b = p.stride_c = 0;
    p.fadd = fadd; p.fmul = fma ? fadd : fmul;
    p.gadd = any_float(fadd); p.gmul = any_float(fma ? fadd : fmul);
    p.radd = FastRn::make(fadd); p.rmul = FastRn::make(p.fmul);
    p.rbits_add = p.rbits_mul = 0; p.seed_lo = p.seed_hi = 0;
    p.growth8 = (float)growth8_bound(fadd.man);
    p.stats = nullptr;
    p.whole_ok = 0; p.sr_ok = 0;
    p.kah_sc = p.kah_p = p.kah_const = 0.0f; p.growth8_sr = 1.0f;
    p.wadd = p.wmul = FullRn::make(fadd);
    p.sadd = p.smul = FullSr::make(fadd, 0);
    const bool nosub = mm_fast_format_nosub(fadd) && (fma || mm_fast_format_nosub(fmul));
    const bool fast_candidate = (nosub || (fast_rn_supported(fadd) && (fma || fast_rn_supported(fmul)))) && workspace != nullptr &&
                                workspace_bytes >= sizeof(MmStats) && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0;
    p.nosub = (nosub && fast_candidate) ? 1 : 0;
    if (fast_candidate) {
        MmStats* s = static_cast<MmStats*>(workspace);
        stats_init_kernel<<<1, 256, 0, st>>>(s, 1);
        const int64_t ng = (int64_t)n_img * c_out * L, nx = (int64_t)n_img * c_in * H * W;
        const int sms = sm_count();
        auto grid = [&](int64_t n) { int64_t g = (n + 255) / 256; const int64_t cap = (int64_t)sms * 8; return dim3((unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 1); };
        stats_kernel<<<grid(ng), 256, 0, st>>>(gout, ng, s, 0);
        stats_kernel<<<grid(nx), 256, 0, st>>>(x, nx, s, 1);
        int rc = check_launch("float_conv2d_wgrad statistics");
        if (rc) return rc;
        p.stats = s;
    }
    for (int g = 0; g < groups; ++g) {
        p.a = gout + (int64_t)g * og * L;
        p.b = x + (int64_t)g * cg * H * W;
        p.c = gw + (int64_t)g * og * Kw;
        // fewer 128-row tiles than SMs: the 16-row instantiation spreads the same outputs over eight times the CTAs
        const int64_t big_tiles = (((int64_t)p.M + BM - 1) / BM) * (((int64_t)p.N + BN - 1) / BN);
        const bool small = big_tiles < sm_count() && ((int64_t)p.M + kSmallTileRows - 1) / kSmallTileRows <= 65535;
        const int rc = small ? launch_conv_wgrad_small_any(algo, fma, p, st) : launch_conv_wgrad_any(algo, fma, p, st);
        if (rc) return rc;
    }
    return MPT_OK;
}

int check_mm_args(const char* who, const float* a, const float* b, float* c, int64_t batch, int M, int N, int K) {
    MPT_REQUIRE(batch >= 0 && M >= 0 && N >= 0 && K >= 0, "%s: negative dimension", who);
    MPT_REQUIRE(batch <= 65535, "%s: batch %lld exceeds 65535", who, (long long)batch);
    MPT_REQUIRE(((int64_t)M + BM - 1) / BM <= 65535, "%s: M=%d too large", who, M);
    const bool empty = batch == 0 || M == 0 || N == 0;
    MPT_REQUIRE(empty || (c && (K == 0 || (a && b))), "%s: null pointer", who);
    return MPT_OK;
}

// ---- scratch for the entry point that allocates nothing -------------------------------------------
// Some callers cannot hand the GEMM a workspace because they cannot allocate device memory at all: a host
// application that has already given every byte of the GPU to its own pool, a plugin interface that
// passes nothing but input and output buffers, or a latency-critical loop in which cudaMalloc (and the
// device-wide synchronisation it implies) is forbidden.  For them the operand statistics live in this
// fixed array instead.  It is part of the library image: every GPU that loads the library holds these
// 64 KiB until the process exits.
constexpr int kStaticScratchMaxBatch = 4096;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchMaxBatch * sizeof(MmStats)];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the address on
// the current device comes from cudaGetSymbolAddress, asked once per device and cached.
int static_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("float_mm_nearest_static: cudaGetDevice: %s", cudaGetErrorString(e)); return MPT_ERR_CUDA; }
    if (dev < 0 || dev >= 64) { set_error("float_mm_nearest_static: device ordinal %d not supported", dev); return MPT_ERR_INVALID_ARGUMENT; }
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("float_mm_nearest_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return MPT_ERR_CUDA;
        }
        cached[dev] = p;
    }
    *out = cached[dev];
    return MPT_OK;
}

}  // namespace
}  // namespace mpt

using namespace mpt;

extern "C" {

size_t mpt_mm_workspace_bytes(int64_t batch) {
    const size_t need = sizeof(MmStats) * (size_t)(batch < 1 ? 1 : batch);
    return (need + 255) & ~(size_t)255;
}

int mpt_float_mm_nearest(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, int man_add,
                         int exp_add, int man_mul, int exp_mul, int subnormals, int saturate, int compensated,
                         int order, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_mm_args("float_mm_nearest", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_add, exp_add) && valid_format(man_mul, exp_mul), "float_mm_nearest: unsupported format");
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "float_mm_nearest: unknown order %d", order);
    const int algo = compensated ? ALGO_KAHAN : (order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8);
    return run_mm(a, b, c, batch, M, N, K, any_float(make_fmt(man_add, exp_add, subnormals, saturate)),
                  any_float(make_fmt(man_mul, exp_mul, subnormals, saturate)), 0, 0, false, algo, 0, workspace, workspace_bytes,
                  as_stream(stream));
}

int mpt_float_mm_nearest_piece(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, int man_add,
                               int exp_add, int man_mul, int exp_mul, int subnormals, int saturate, int fma, int order,
                               int flags, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_mm_args("float_mm_nearest_piece", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_add, exp_add) && (fma || valid_format(man_mul, exp_mul)), "float_mm_nearest_piece: unsupported format");
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "float_mm_nearest_piece: unknown order %d", order);
    MPT_REQUIRE((flags & ~(MPT_MM_PIECE_FROM_C | MPT_MM_PIECE_MORE)) == 0, "float_mm_nearest_piece: unknown flags %d", flags);
    MPT_REQUIRE(!(flags & MPT_MM_PIECE_MORE) || K % 8 == 0,
                "float_mm_nearest_piece: a piece that another follows must cover a multiple of 8 steps (K=%d)", K);
    const AnyFmt fa = any_float(make_fmt(man_add, exp_add, subnormals, saturate));
    const AnyFmt fm = fma ? fa : any_float(make_fmt(man_mul, exp_mul, subnormals, saturate));
    const int resume = ((flags & MPT_MM_PIECE_FROM_C) ? MM_FROM_C : 0) | ((flags & MPT_MM_PIECE_MORE) ? MM_MORE : 0);
    return run_mm(a, b, c, batch, M, N, K, fa, fm, 0, 0, fma != 0, order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8, 0, workspace,
                  workspace_bytes, as_stream(stream), resume);
}

int mpt_float_mm_nearest_static(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, int man_add,
                                int exp_add, int man_mul, int exp_mul, int subnormals, int saturate, int compensated,
                                int order, void* stream) {
    int rc = check_mm_args("float_mm_nearest_static", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_add, exp_add) && valid_format(man_mul, exp_mul), "float_mm_nearest_static: unsupported format");
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "float_mm_nearest_static: unknown order %d", order);
    MPT_REQUIRE(batch <= kStaticScratchMaxBatch,
                "float_mm_nearest_static: batch %lld exceeds the %d entries of the built-in scratch; use "
                "mpt_float_mm_nearest with a caller-provided workspace", (long long)batch, kStaticScratchMaxBatch);
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    const int algo = compensated ? ALGO_KAHAN : (order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8);
    // run_mm re-initialises the statistics records it uses before reading them, so whatever the previous
    // call left in the array is never seen
    return run_mm(a, b, c, batch, M, N, K, any_float(make_fmt(man_add, exp_add, subnormals, saturate)),
                  any_float(make_fmt(man_mul, exp_mul, subnormals, saturate)), 0, 0, false, algo, 0, scratch,
                  sizeof(MmStats) * (size_t)kStaticScratchMaxBatch, as_stream(stream));
}

int mpt_mm_nearest_fmt(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, const mpt_format* add,
                       const mpt_format* mul, int fma, int order, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_mm_args("mm_nearest_fmt", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "mm_nearest_fmt: unknown order %d", order);
    AnyFmt ga, gm;
    if (!convert_format("mm_nearest_fmt", add, &ga)) return MPT_ERR_INVALID_ARGUMENT;
    if (fma) gm = ga;
    else if (!convert_format("mm_nearest_fmt", mul, &gm)) return MPT_ERR_INVALID_ARGUMENT;
    return run_mm(a, b, c, batch, M, N, K, ga, gm, 0, 0, fma != 0, order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8, 0, workspace,
                  workspace_bytes, as_stream(stream));
}

int mpt_float_conv2d_nearest(const float* x, const float* wt, float* y, int n_img, int c_in, int H, int W, int c_out, int groups,
                             int KH, int KW, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int man_add,
                             int exp_add, int man_mul, int exp_mul, int subnormals, int saturate, int fma, int order,
                             void* workspace, size_t workspace_bytes, void* stream) {
    MPT_REQUIRE(n_img >= 0 && c_in >= 0 && H >= 0 && W >= 0 && c_out >= 0, "float_conv2d_nearest: negative extent");
    MPT_REQUIRE(groups >= 1 && c_in % groups == 0 && c_out % groups == 0, "float_conv2d_nearest: channels not divisible by groups=%d", groups);
    MPT_REQUIRE(KH >= 1 && KW >= 1 && stride_h >= 1 && stride_w >= 1 && dil_h >= 1 && dil_w >= 1 && pad_h >= 0 && pad_w >= 0,
                "float_conv2d_nearest: invalid kernel / stride / padding / dilation");
    MPT_REQUIRE(valid_format(man_add, exp_add) && (fma || valid_format(man_mul, exp_mul)), "float_conv2d_nearest: unsupported format");
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "float_conv2d_nearest: unknown order %d", order);
    MPT_REQUIRE((int64_t)c_in * H * W <= 0x7FFFFFFF, "float_conv2d_nearest: one input image exceeds 2^31 elements");
    const bool empty = n_img == 0 || c_out == 0;
    MPT_REQUIRE(empty || (x && wt && y), "float_conv2d_nearest: null pointer");
    return run_conv(x, wt, y, n_img, c_in, H, W, c_out, groups, KH, KW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w,
                    make_fmt(man_add, exp_add, subnormals, saturate), make_fmt(fma ? man_add : man_mul, fma ? exp_add : exp_mul, subnormals, saturate),
                    fma != 0, order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8, workspace, workspace_bytes, as_stream(stream));
}

int mpt_float_conv2d_wgrad_nearest(const float* grad_out, const float* x, float* grad_w, int n_img, int c_in, int H, int W, int c_out,
                                   int groups, int KH, int KW, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                   int man_add, int exp_add, int man_mul, int exp_mul, int subnormals, int saturate, int fma, int order,
                                   void* workspace, size_t workspace_bytes, void* stream) {
    const char* who = "float_conv2d_wgrad_nearest";
    MPT_REQUIRE(n_img >= 0 && c_in >= 0 && H >= 0 && W >= 0 && c_out >= 0, "%s: negative extent", who);
    MPT_REQUIRE(groups >= 1 && c_in % groups == 0 && c_out % groups == 0, "%s: channels not divisible by groups=%d", who, groups);
    MPT_REQUIRE(KH >= 1 && KW >= 1 && stride_h >= 1 && stride_w >= 1 && dil_h >= 1 && dil_w >= 1 && pad_h >= 0 && pad_w >= 0,
                "%s: invalid kernel / stride / padding / dilation", who);
    MPT_REQUIRE(valid_format(man_add, exp_add) && (fma || valid_format(man_mul, exp_mul)), "%s: unsupported format", who);
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "%s: unknown order %d", who, order);
    MPT_REQUIRE((int64_t)c_in * H * W <= 0x7FFFFFFF, "%s: one input image exceeds 2^31 elements", who);
    MPT_REQUIRE(c_out / groups <= 65535 * BM, "%s: too many output channels per group", who);
    const bool empty = c_out == 0 || c_in == 0;
    MPT_REQUIRE(empty || grad_w, "%s: null pointer", who);
    MPT_REQUIRE(empty || n_img == 0 || (grad_out && x), "%s: null pointer", who);
    return run_conv_wgrad(grad_out, x, grad_w, n_img, c_in, H, W, c_out, groups, KH, KW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w,
                          make_fmt(man_add, exp_add, subnormals, saturate), make_fmt(fma ? man_add : man_mul, fma ? exp_add : exp_mul, subnormals, saturate),
                          fma != 0, order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8, workspace, workspace_bytes, as_stream(stream));
}

int mpt_float_mm_nearest_fma(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, int man_fma,
                             int exp_fma, int subnormals, int saturate, int compensated, int order, void* workspace,
                             size_t workspace_bytes, void* stream) {
    int rc = check_mm_args("float_mm_nearest_fma", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_fma, exp_fma), "float_mm_nearest_fma: unsupported format");
    MPT_REQUIRE(order == MPT_ORDER_SEQ || order == MPT_ORDER_CUDA, "float_mm_nearest_fma: unknown order %d", order);
    const int algo = compensated ? ALGO_KAHAN : (order == MPT_ORDER_SEQ ? ALGO_SEQ : ALGO_TILE8);
    const AnyFmt f = any_float(make_fmt(man_fma, exp_fma, subnormals, saturate));
    return run_mm(a, b, c, batch, M, N, K, f, f, 0, 0, true, algo, 0, workspace, workspace_bytes, as_stream(stream));
}

int mpt_float_mm_stochastic(const float* a, const float* b, float* c, int64_t batch, int M, int N, int K, int man_add,
                            int exp_add, int rbits_add, int man_mul, int exp_mul, int rbits_mul, int subnormals,
                            int saturate, int fma, uint64_t seed, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_mm_args("float_mm_stochastic", a, b, c, batch, M, N, K);
    if (rc) return rc;
    MPT_REQUIRE(valid_format(man_add, exp_add) && (fma || valid_format(man_mul, exp_mul)), "float_mm_stochastic: unsupported format");
    const AnyFmt fa = any_float(make_fmt(man_add, exp_add, subnormals, saturate));
    const AnyFmt fm = fma ? fa : any_float(make_fmt(man_mul, exp_mul, subnormals, saturate));
    return run_mm(a, b, c, batch, M, N, K, fa, fm, rbits_add, rbits_mul, fma != 0, ALGO_SR, seed, workspace, workspace_bytes,
                  as_stream(stream));
}

}
