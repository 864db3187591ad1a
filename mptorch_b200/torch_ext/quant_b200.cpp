// PyTorch C++ extension `quant_b200`: the reference's `quant_cuda` pybind11 module re-expressed over the
// C ABI of libmptorch_b200.so.  Same function names, argument order and tensor checks as the
// registrations in the reference's mptorch/quant/quant_cuda/pybind_cuda.cpp (lines cited per function),
// so `quant_function.py` can use this module in place of `quant_cuda`.  The extension holds no kernels:
// it checks tensors, selects the device and the current stream, allocates outputs and a small GEMM
// workspace through the caching allocator, and forwards.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <vector>

#include "mptorch_b200.h"

namespace {

#define CHECK_CUDA(x) TORCH_CHECK(x.is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
    CHECK_CUDA(x);     \
    CHECK_CONTIGUOUS(x); \
    TORCH_CHECK(x.scalar_type() == at::kFloat, #x " must be float32")

void check(int rc) { TORCH_CHECK(rc == MPT_OK, mpt_last_error()); }
void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int g_accum_order = MPT_ORDER_CUDA, g_reduce_order = MPT_ORDER_CUDA;

struct Geom { int64_t outer; int channel; int64_t inner; };

// reference: quant_cuda/quant.cu:678-726 (partition_tensor for one dim and for a list of trailing dims)
Geom partition(const at::Tensor& t, const std::vector<int>& dims) {
    const int nd = (int)t.dim();
    std::vector<int> real;
    for (int d : dims) real.push_back((nd + (d % nd)) % nd);
    Geom g{1, 1, 1};
    for (int d : real) g.channel *= (int)t.size(d);
    for (int i = 0; i < real.back(); ++i) g.outer *= t.size(i);
    for (int i = real.front() + 1; i < nd; ++i) g.inner *= t.size(i);
    return g;
}

at::Tensor float_quantize_nearest(at::Tensor a, int man_bits, int exp_bits, bool subnormals, bool saturate) {   // :44
    CHECK_INPUT(a);
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty_like(a);
    check(mpt_float_quantize_nearest(a.data_ptr<float>(), o.data_ptr<float>(), a.numel(), man_bits, exp_bits, subnormals, saturate, stream()));
    return o;
}

at::Tensor float_quantize_stochastic(at::Tensor a, int man_bits, int exp_bits, int prng_bits, bool subnormals, bool saturate) {   // :98
    CHECK_INPUT(a);
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty_like(a);
    auto r = at::randint_like(a, INT_MAX, a.options().dtype(at::kInt));   // the reference's draw (quant.cu:132)
    check(mpt_float_quantize_stochastic(a.data_ptr<float>(), r.data_ptr<int>(), o.data_ptr<float>(), a.numel(), man_bits, exp_bits, prng_bits,
                                        subnormals, saturate, stream()));
    return o;
}

at::Tensor float_quantize_truncate(at::Tensor a, int man_bits, int exp_bits, bool subnormals, bool saturate) {   // new
    CHECK_INPUT(a);
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty_like(a);
    check(mpt_float_quantize_truncate(a.data_ptr<float>(), o.data_ptr<float>(), a.numel(), man_bits, exp_bits, subnormals, saturate, stream()));
    return o;
}

at::Tensor binary8(at::Tensor a, int P, int prng_bits, bool is_signed, int policy, bool subnormals, int rounding) {
    CHECK_INPUT(a);
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty_like(a);
    at::Tensor r;
    const int* rp = nullptr;
    if (rounding == MPT_RND_STOCHASTIC) {
        r = at::randint_like(a, INT_MAX, a.options().dtype(at::kInt));    // quant.cu:202
        rp = r.data_ptr<int>();
    }
    check(mpt_binary8_quantize(a.data_ptr<float>(), rp, o.data_ptr<float>(), a.numel(), P, is_signed, policy, subnormals, rounding, prng_bits, stream()));
    return o;
}
at::Tensor binary8_quantize_nearest(at::Tensor a, int P, bool is_signed, int policy, bool subnormals) {   // :61
    return binary8(a, P, 0, is_signed, policy, subnormals, MPT_RND_NEAREST);
}
at::Tensor binary8_quantize_stochastic(at::Tensor a, int P, int prng_bits, bool is_signed, int policy, bool subnormals) {   // :107
    return binary8(a, P, prng_bits, is_signed, policy, subnormals, MPT_RND_STOCHASTIC);
}
at::Tensor binary8_quantize_truncate(at::Tensor a, int P, bool is_signed, int policy, bool subnormals) {   // :115
    return binary8(a, P, 0, is_signed, policy, subnormals, MPT_RND_TRUNCATE);
}

at::Tensor superfp_quantize_nearest(at::Tensor a, int man_bits, int exp_bits, int binades_l, int binades_u, bool saturate) {   // :53
    CHECK_INPUT(a);
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty_like(a);
    check(mpt_superfp_quantize_nearest(a.data_ptr<float>(), o.data_ptr<float>(), a.numel(), man_bits, exp_bits, binades_l, binades_u, saturate, stream()));
    return o;
}

void mm_nearest(at::Tensor a, at::Tensor b, at::Tensor c, int64_t batch, int M, int N, int K, int man_add, int exp_add, int man_mul, int exp_mul,
                bool subnormals, bool saturate, bool compensated, bool fma) {
    CHECK_INPUT(a); CHECK_INPUT(b); CHECK_INPUT(c);
    c10::cuda::CUDAGuard guard(a.device());
    auto ws = at::empty({(int64_t)mpt_mm_workspace_bytes(batch)}, a.options().dtype(at::kByte));
    if (fma)
        check(mpt_float_mm_nearest_fma(a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), batch, M, N, K, man_add, exp_add, subnormals,
                                       saturate, compensated, g_accum_order, ws.data_ptr(), (size_t)ws.numel(), stream()));
    else
        check(mpt_float_mm_nearest(a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), batch, M, N, K, man_add, exp_add, man_mul, exp_mul,
                                   subnormals, saturate, compensated, g_accum_order, ws.data_ptr(), (size_t)ws.numel(), stream()));
}
int64_t batch_of(const at::Tensor& a) { return a.dim() > 2 ? a.size(0) : 1; }   // quant.cu:370-379

void float_quantize_nearest_mm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int man_mul, int exp_mul,
                               bool subnormals, bool saturate, bool compensated) {   // :123
    mm_nearest(a, b, c, 1, M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, compensated, false);
}
void float_quantize_nearest_bmm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int man_mul, int exp_mul,
                                bool subnormals, bool saturate, bool compensated) {   // :140
    mm_nearest(a, b, c, batch_of(a), M, N, K, man_add, exp_add, man_mul, exp_mul, subnormals, saturate, compensated, false);
}
void float_quantize_nearest_mm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, bool subnormals,
                                   bool saturate, bool compensated) {   // :157
    mm_nearest(a, b, c, 1, M, N, K, man_fma, exp_fma, man_fma, exp_fma, subnormals, saturate, compensated, true);
}
void float_quantize_nearest_bmm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, bool subnormals,
                                    bool saturate, bool compensated) {   // :173
    mm_nearest(a, b, c, batch_of(a), M, N, K, man_fma, exp_fma, man_fma, exp_fma, subnormals, saturate, compensated, true);
}

void mm_sr(at::Tensor a, at::Tensor b, at::Tensor c, int64_t batch, int M, int N, int K, int man_add, int exp_add, int rbits_add, int man_mul,
           int exp_mul, int rbits_mul, bool subnormals, bool saturate, bool fma) {
    CHECK_INPUT(a); CHECK_INPUT(b); CHECK_INPUT(c);
    c10::cuda::CUDAGuard guard(a.device());
    const uint64_t seed = (uint64_t)at::randint(0, INT64_MAX >> 1, {1}, at::kLong).item<int64_t>();   // reproducible under torch.manual_seed
    auto ws = at::empty({(int64_t)mpt_mm_workspace_bytes(batch)}, a.options().dtype(at::kByte));
    check(mpt_float_mm_stochastic(a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), batch, M, N, K, man_add, exp_add, rbits_add, man_mul,
                                  exp_mul, rbits_mul, subnormals, saturate, fma, seed, ws.data_ptr(), (size_t)ws.numel(), stream()));
}
void float_quantize_stochastic_mm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int rbits_add,
                                  int man_mul, int exp_mul, int rbits_mul, bool subnormals, bool saturate) {   // :254
    mm_sr(a, b, c, 1, M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals, saturate, false);
}
void float_quantize_stochastic_bmm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int rbits_add,
                                   int man_mul, int exp_mul, int rbits_mul, bool subnormals, bool saturate) {   // :270
    mm_sr(a, b, c, batch_of(a), M, N, K, man_add, exp_add, rbits_add, man_mul, exp_mul, rbits_mul, subnormals, saturate, false);
}
void float_quantize_stochastic_mm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, int rbits_fma,
                                      bool subnormals, bool saturate) {   // :286
    mm_sr(a, b, c, 1, M, N, K, man_fma, exp_fma, rbits_fma, man_fma, exp_fma, rbits_fma, subnormals, saturate, true);
}
void float_quantize_stochastic_bmm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, int rbits_fma,
                                       bool subnormals, bool saturate) {   // :300
    mm_sr(a, b, c, batch_of(a), M, N, K, man_fma, exp_fma, rbits_fma, man_fma, exp_fma, rbits_fma, subnormals, saturate, true);
}

void float_quantize_nearest_softmax_forward(at::Tensor a, at::Tensor o, int dim, int man_exp, int exp_exp, int man_off, int exp_off, int man_acc,
                                            int exp_acc, bool subnormals, bool saturate) {   // :599
    CHECK_INPUT(a); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_float_softmax_forward(a.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, man_exp, exp_exp, man_off, exp_off,
                                    man_acc, exp_acc, subnormals, saturate, g_reduce_order, stream()));
}
void float_quantize_nearest_softmax_lse_forward(at::Tensor a, at::Tensor o, int dim, int man_off, int exp_off, int man_lse, int exp_lse,
                                                bool subnormals, bool saturate) {   // :615
    CHECK_INPUT(a); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_float_softmax_lse_forward(a.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, man_off, exp_off, man_lse, exp_lse,
                                        subnormals, saturate, g_reduce_order, stream()));
}
void float_quantize_nearest_softmax_backward(at::Tensor a, at::Tensor grad, at::Tensor o, int dim, int man_add, int exp_add, int man_mul,
                                             int exp_mul, bool subnormals, bool saturate) {   // :629
    CHECK_INPUT(a); CHECK_INPUT(grad); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_float_softmax_backward(a.data_ptr<float>(), grad.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, man_add,
                                     exp_add, man_mul, exp_mul, subnormals, saturate, g_reduce_order, stream()));
}

void float_quantize_layernorm_forward(at::Tensor input, at::Tensor weight, at::Tensor bias, at::Tensor output, at::Tensor mean, at::Tensor rstd,
                                      float eps, std::vector<int> dims, int man_acc, int exp_acc, int man_mul, int exp_mul, int man_div,
                                      int exp_div, int man_sqrt, int exp_sqrt, bool subnormals, bool saturate) {   // :434
    CHECK_INPUT(input); CHECK_INPUT(weight); CHECK_INPUT(bias); CHECK_INPUT(output); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    c10::cuda::CUDAGuard guard(input.device());
    const Geom g = partition(input, dims);
    check(mpt_float_layernorm_forward(input.data_ptr<float>(), weight.data_ptr<float>(), bias.data_ptr<float>(), output.data_ptr<float>(),
                                      mean.data_ptr<float>(), rstd.data_ptr<float>(), eps, g.outer, g.channel, g.inner, man_acc, exp_acc, man_mul,
                                      exp_mul, man_div, exp_div, man_sqrt, exp_sqrt, subnormals, saturate, g_reduce_order, stream()));
}
void float_quantize_layernorm_backward(at::Tensor input, at::Tensor grad_output, at::Tensor weight, at::Tensor bias, at::Tensor mean,
                                       at::Tensor rstd, at::Tensor grad_input, at::Tensor grad_gamma, at::Tensor grad_beta,
                                       std::vector<int> dims, int man_acc, int exp_acc, int man_mul, int exp_mul, int man_div, int exp_div,
                                       bool subnormals, bool saturate) {   // :459
    CHECK_INPUT(input); CHECK_INPUT(grad_output); CHECK_INPUT(weight); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    CHECK_INPUT(grad_input); CHECK_INPUT(grad_gamma); CHECK_INPUT(grad_beta);
    (void)bias;
    c10::cuda::CUDAGuard guard(input.device());
    const Geom g = partition(input, dims);
    check(mpt_float_layernorm_backward(input.data_ptr<float>(), grad_output.data_ptr<float>(), weight.data_ptr<float>(), mean.data_ptr<float>(),
                                       rstd.data_ptr<float>(), grad_input.data_ptr<float>(), grad_gamma.data_ptr<float>(),
                                       grad_beta.data_ptr<float>(), g.outer, g.channel, g.inner, man_acc, exp_acc, man_mul, exp_mul, man_div,
                                       exp_div, subnormals, saturate, g_reduce_order, stream()));
}


// ---- the other nearest-rounding format families (pybind_cuda.cpp:815-824, :887-924) -------------------------------
enum class OverflowPolicy { SATURATE_INFTY = MPT_SATURATE_INFTY, SATURATE_MAXFLOAT = MPT_SATURATE_MAXFLOAT, SATURATE_MAXFLOAT2 = MPT_SATURATE_MAXFLOAT2 };

mpt_format superfp(int man, int exp, int bl, int bu, bool saturate) {
    mpt_format f{};
    f.kind = MPT_FMT_SUPERFP; f.man = man; f.exp = exp; f.subnormals = 1; f.saturate = saturate; f.binades_l = bl; f.binades_u = bu;
    f.P = 1; f.is_signed = 1;
    return f;
}
mpt_format binary8(int P, int policy, bool is_signed, bool subnormals) {
    mpt_format f{};
    f.kind = MPT_FMT_BINARY8; f.subnormals = subnormals; f.binades_l = f.binades_u = 1; f.P = P; f.is_signed = is_signed; f.overflow_policy = policy;
    return f;
}

void mm_fmt(at::Tensor a, at::Tensor b, at::Tensor c, int64_t batch, int M, int N, int K, const mpt_format& fa, const mpt_format& fm, bool fma) {
    CHECK_INPUT(a); CHECK_INPUT(b); CHECK_INPUT(c);
    c10::cuda::CUDAGuard guard(a.device());
    auto ws = at::empty({(int64_t)mpt_mm_workspace_bytes(batch)}, a.options().dtype(at::kByte));
    check(mpt_mm_nearest_fmt(a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), batch, M, N, K, &fa, &fm, fma, g_accum_order,
                             ws.data_ptr(), (size_t)ws.numel(), stream()));
}
void superfp_quantize_nearest_mm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int man_mul, int exp_mul,
                                 int bal, int bau, int bml, int bmu, bool saturate) {   // :815
    mm_fmt(a, b, c, 1, M, N, K, superfp(man_add, exp_add, bal, bau, saturate), superfp(man_mul, exp_mul, bml, bmu, saturate), false);
}
void superfp_quantize_nearest_bmm(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_add, int exp_add, int man_mul, int exp_mul,
                                  int bal, int bau, int bml, int bmu, bool saturate) {   // :818
    mm_fmt(a, b, c, batch_of(a), M, N, K, superfp(man_add, exp_add, bal, bau, saturate), superfp(man_mul, exp_mul, bml, bmu, saturate), false);
}
void superfp_quantize_nearest_mm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, int bl, int bu,
                                     bool saturate) {   // :821
    const mpt_format f = superfp(man_fma, exp_fma, bl, bu, saturate);
    mm_fmt(a, b, c, 1, M, N, K, f, f, true);
}
void superfp_quantize_nearest_bmm_fma(at::Tensor a, at::Tensor b, at::Tensor c, int M, int N, int K, int man_fma, int exp_fma, int bl, int bu,
                                      bool saturate) {   // :824
    const mpt_format f = superfp(man_fma, exp_fma, bl, bu, saturate);
    mm_fmt(a, b, c, batch_of(a), M, N, K, f, f, true);
}

void softmax_fwd_fmt(at::Tensor a, at::Tensor o, int dim, const mpt_format& fe, const mpt_format& fo, const mpt_format& fa) {
    CHECK_INPUT(a); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_softmax_forward_fmt(a.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, &fe, &fo, &fa, g_reduce_order, stream()));
}
void softmax_lse_fmt(at::Tensor a, at::Tensor o, int dim, const mpt_format& fo, const mpt_format& fl) {
    CHECK_INPUT(a); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_softmax_lse_forward_fmt(a.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, &fo, &fl, g_reduce_order, stream()));
}
void softmax_bwd_fmt(at::Tensor a, at::Tensor gr, at::Tensor o, int dim, const mpt_format& fa, const mpt_format& fm) {
    CHECK_INPUT(a); CHECK_INPUT(gr); CHECK_INPUT(o);
    c10::cuda::CUDAGuard guard(a.device());
    const Geom g = partition(a, {dim});
    check(mpt_softmax_backward_fmt(a.data_ptr<float>(), gr.data_ptr<float>(), o.data_ptr<float>(), g.outer, g.channel, g.inner, &fa, &fm,
                                   g_reduce_order, stream()));
}
void superfp_quantize_nearest_softmax_forward(at::Tensor a, at::Tensor o, int dim, int man_exp, int exp_exp, int bel, int beu, int man_off,
                                              int exp_off, int bol, int bou, int man_acc, int exp_acc, int bal, int bau, bool saturate) {   // :887
    softmax_fwd_fmt(a, o, dim, superfp(man_exp, exp_exp, bel, beu, saturate), superfp(man_off, exp_off, bol, bou, saturate),
                    superfp(man_acc, exp_acc, bal, bau, saturate));
}
void superfp_quantize_nearest_softmax_lse_forward(at::Tensor a, at::Tensor o, int dim, int man_off, int exp_off, int bol, int bou, int man_lse,
                                                  int exp_lse, int bll, int blu, bool saturate) {   // :890
    softmax_lse_fmt(a, o, dim, superfp(man_off, exp_off, bol, bou, saturate), superfp(man_lse, exp_lse, bll, blu, saturate));
}
void superfp_quantize_nearest_softmax_backward(at::Tensor a, at::Tensor g, at::Tensor o, int dim, int man_add, int exp_add, int bal, int bau,
                                               int man_mul, int exp_mul, int bml, int bmu, bool saturate) {   // :893
    softmax_bwd_fmt(a, g, o, dim, superfp(man_add, exp_add, bal, bau, saturate), superfp(man_mul, exp_mul, bml, bmu, saturate));
}
void binary8_quantize_nearest_softmax_forward(at::Tensor a, at::Tensor o, int dim, int P_exp, int op_exp, bool signed_exp, int P_off, int op_off,
                                              bool signed_off, int P_acc, int op_acc, bool signed_acc, bool subnormals) {   // :897
    softmax_fwd_fmt(a, o, dim, binary8(P_exp, op_exp, signed_exp, subnormals), binary8(P_off, op_off, signed_off, subnormals),
                    binary8(P_acc, op_acc, signed_acc, subnormals));
}
void binary8_quantize_nearest_softmax_lse_forward(at::Tensor a, at::Tensor o, int dim, int P_off, int op_off, bool signed_off, int P_lse,
                                                  int op_lse, bool signed_lse, bool subnormals) {   // :900
    softmax_lse_fmt(a, o, dim, binary8(P_off, op_off, signed_off, subnormals), binary8(P_lse, op_lse, signed_lse, subnormals));
}
void binary8_quantize_nearest_softmax_backward(at::Tensor a, at::Tensor g, at::Tensor o, int dim, int P_add, int op_add, bool signed_add,
                                               int P_mul, int op_mul, bool signed_mul, bool subnormals) {   // :903
    softmax_bwd_fmt(a, g, o, dim, binary8(P_add, op_add, signed_add, subnormals), binary8(P_mul, op_mul, signed_mul, subnormals));
}

void layernorm_fwd_fmt(at::Tensor input, at::Tensor weight, at::Tensor bias, at::Tensor output, at::Tensor mean, at::Tensor rstd, float eps,
                       const std::vector<int>& dims, const mpt_format& fa, const mpt_format& fm, const mpt_format& fd, const mpt_format& fs) {
    CHECK_INPUT(input); CHECK_INPUT(weight); CHECK_INPUT(bias); CHECK_INPUT(output); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    c10::cuda::CUDAGuard guard(input.device());
    const Geom g = partition(input, dims);
    check(mpt_layernorm_forward_fmt(input.data_ptr<float>(), weight.data_ptr<float>(), bias.data_ptr<float>(), output.data_ptr<float>(),
                                    mean.data_ptr<float>(), rstd.data_ptr<float>(), eps, g.outer, g.channel, g.inner, &fa, &fm, &fd, &fs,
                                    g_reduce_order, stream()));
}
void layernorm_bwd_fmt(at::Tensor input, at::Tensor grad_output, at::Tensor weight, at::Tensor mean, at::Tensor rstd, at::Tensor grad_input,
                       at::Tensor grad_gamma, at::Tensor grad_beta, const std::vector<int>& dims, const mpt_format& fa, const mpt_format& fm,
                       const mpt_format& fd) {
    CHECK_INPUT(input); CHECK_INPUT(grad_output); CHECK_INPUT(weight); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    CHECK_INPUT(grad_input); CHECK_INPUT(grad_gamma); CHECK_INPUT(grad_beta);
    c10::cuda::CUDAGuard guard(input.device());
    const Geom g = partition(input, dims);
    check(mpt_layernorm_backward_fmt(input.data_ptr<float>(), grad_output.data_ptr<float>(), weight.data_ptr<float>(), mean.data_ptr<float>(),
                                     rstd.data_ptr<float>(), grad_input.data_ptr<float>(), grad_gamma.data_ptr<float>(),
                                     grad_beta.data_ptr<float>(), g.outer, g.channel, g.inner, &fa, &fm, &fd, g_reduce_order, stream()));
}
void superfp_quantize_layernorm_forward(at::Tensor input, at::Tensor weight, at::Tensor bias, at::Tensor output, at::Tensor mean, at::Tensor rstd,
                                        float eps, std::vector<int> dims, int man_acc, int exp_acc, int bal, int bau, int man_mul, int exp_mul,
                                        int bml, int bmu, int man_div, int exp_div, int bdl, int bdu, int man_sqrt, int exp_sqrt, int bsl,
                                        int bsu, bool saturate) {   // :914
    layernorm_fwd_fmt(input, weight, bias, output, mean, rstd, eps, dims, superfp(man_acc, exp_acc, bal, bau, saturate),
                      superfp(man_mul, exp_mul, bml, bmu, saturate), superfp(man_div, exp_div, bdl, bdu, saturate),
                      superfp(man_sqrt, exp_sqrt, bsl, bsu, saturate));
}
void superfp_quantize_layernorm_backward(at::Tensor input, at::Tensor grad_output, at::Tensor weight, at::Tensor bias, at::Tensor mean,
                                         at::Tensor rstd, at::Tensor grad_input, at::Tensor grad_gamma, at::Tensor grad_beta,
                                         std::vector<int> dims, int man_acc, int exp_acc, int bal, int bau, int man_mul, int exp_mul, int bml,
                                         int bmu, int man_div, int exp_div, int bdl, int bdu, bool saturate) {   // :917
    (void)bias;
    layernorm_bwd_fmt(input, grad_output, weight, mean, rstd, grad_input, grad_gamma, grad_beta, dims, superfp(man_acc, exp_acc, bal, bau, saturate),
                      superfp(man_mul, exp_mul, bml, bmu, saturate), superfp(man_div, exp_div, bdl, bdu, saturate));
}
void binary8_quantize_layernorm_forward(at::Tensor input, at::Tensor weight, at::Tensor bias, at::Tensor output, at::Tensor mean, at::Tensor rstd,
                                        float eps, std::vector<int> dims, int P_acc, int op_acc, bool signed_acc, int P_mul, int op_mul,
                                        bool signed_mul, int P_div, int op_div, bool signed_div, int P_sqrt, int op_sqrt, bool signed_sqrt,
                                        bool subnormals) {   // :921
    layernorm_fwd_fmt(input, weight, bias, output, mean, rstd, eps, dims, binary8(P_acc, op_acc, signed_acc, subnormals),
                      binary8(P_mul, op_mul, signed_mul, subnormals), binary8(P_div, op_div, signed_div, subnormals),
                      binary8(P_sqrt, op_sqrt, signed_sqrt, subnormals));
}
void binary8_quantize_layernorm_backward(at::Tensor input, at::Tensor grad_output, at::Tensor weight, at::Tensor bias, at::Tensor mean,
                                         at::Tensor rstd, at::Tensor grad_input, at::Tensor grad_gamma, at::Tensor grad_beta,
                                         std::vector<int> dims, int P_acc, int op_acc, bool signed_acc, int P_mul, int op_mul, bool signed_mul,
                                         int P_div, int op_div, bool signed_div, bool subnormals) {   // :924
    (void)bias;
    layernorm_bwd_fmt(input, grad_output, weight, mean, rstd, grad_input, grad_gamma, grad_beta, dims, binary8(P_acc, op_acc, signed_acc, subnormals),
                      binary8(P_mul, op_mul, signed_mul, subnormals), binary8(P_div, op_div, signed_div, subnormals));
}

// ---- entry points without a quant_cuda counterpart ----------------------------------------------------------------
at::Tensor qsum_rows(at::Tensor a, int man_bits, int exp_bits, bool subnormals, bool saturate) {
    CHECK_INPUT(a);
    TORCH_CHECK(a.dim() == 2, "qsum_rows expects a 2-D tensor");
    c10::cuda::CUDAGuard guard(a.device());
    auto o = at::empty({a.size(1)}, a.options());
    check(mpt_qsum_rows(a.data_ptr<float>(), o.data_ptr<float>(), a.size(0), a.size(1), man_bits, exp_bits, subnormals, saturate, stream()));
    return o;
}
void float_conv2d_nearest(at::Tensor x, at::Tensor wt, at::Tensor y, int groups, std::vector<int> kernel, std::vector<int> stride,
                          std::vector<int> padding, std::vector<int> dilation, int man_add, int exp_add, int man_mul, int exp_mul,
                          bool subnormals, bool saturate, bool fma) {
    CHECK_INPUT(x); CHECK_INPUT(wt); CHECK_INPUT(y);
    TORCH_CHECK(x.dim() == 4 && y.dim() == 4 && kernel.size() == 2 && stride.size() == 2 && padding.size() == 2 && dilation.size() == 2,
                "float_conv2d_nearest: NCHW tensors and 2-element geometry lists expected");
    c10::cuda::CUDAGuard guard(x.device());
    auto ws = at::empty({(int64_t)mpt_mm_workspace_bytes(1)}, x.options().dtype(at::kByte));
    check(mpt_float_conv2d_nearest(x.data_ptr<float>(), wt.data_ptr<float>(), y.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (int)x.size(2),
                                   (int)x.size(3), (int)y.size(1), groups, kernel[0], kernel[1], stride[0], stride[1], padding[0], padding[1],
                                   dilation[0], dilation[1], man_add, exp_add, man_mul, exp_mul, subnormals, saturate, fma, g_accum_order,
                                   ws.data_ptr(), (size_t)ws.numel(), stream()));
}
std::vector<at::Tensor> mx_quantize(at::Tensor a, const std::string& elem, int block, bool return_scales, bool return_codes) {
    CHECK_INPUT(a);
    TORCH_CHECK(elem == "e4m3" || elem == "e2m1", "elem_format must be 'e4m3' or 'e2m1'");
    TORCH_CHECK(a.dim() >= 1 && block >= 1, "mx_quantize: at least one dimension and a positive block size");
    c10::cuda::CUDAGuard guard(a.device());
    const int64_t cols = a.size(-1), rows = cols ? a.numel() / cols : 0;
    auto o = at::empty_like(a);
    auto shape = a.sizes().vec();
    at::Tensor sc, codes;
    if (return_scales) { shape.back() = (cols + block - 1) / block; sc = at::empty(shape, a.options().dtype(at::kByte)); }
    if (return_codes) { shape.back() = elem == "e4m3" ? cols : (cols + 1) / 2; codes = at::zeros(shape, a.options().dtype(at::kByte)); }
    check(mpt_mx_quantize(a.data_ptr<float>(), o.data_ptr<float>(), return_scales ? sc.data_ptr<uint8_t>() : nullptr,
                          return_codes ? codes.data_ptr<uint8_t>() : nullptr, rows, cols, block, elem == "e4m3" ? MPT_ELEM_E4M3 : MPT_ELEM_E2M1,
                          stream()));
    std::vector<at::Tensor> out{o};
    if (return_scales) out.push_back(sc);
    if (return_codes) out.push_back(codes);
    return out;
}
std::vector<at::Tensor> nvfp4_quantize(at::Tensor a, double global_scale, bool return_scales, bool return_codes) {
    CHECK_INPUT(a);
    TORCH_CHECK(a.dim() >= 1, "nvfp4_quantize: at least one dimension");
    c10::cuda::CUDAGuard guard(a.device());
    const int64_t cols = a.size(-1), rows = cols ? a.numel() / cols : 0;
    auto o = at::empty_like(a);
    auto shape = a.sizes().vec();
    at::Tensor sc, gs, codes, scodes, ws;
    shape.back() = (cols + 15) / 16;
    if (return_scales) { sc = at::empty(shape, a.options()); gs = at::empty({1}, a.options()); }
    if (return_codes) {
        scodes = at::empty(shape, a.options().dtype(at::kByte));
        shape.back() = (cols + 1) / 2;
        codes = at::zeros(shape, a.options().dtype(at::kByte));
    }
    if (!(global_scale > 0.0)) ws = at::empty({1}, a.options().dtype(at::kInt));
    check(mpt_nvfp4_quantize(a.data_ptr<float>(), o.data_ptr<float>(), return_scales ? sc.data_ptr<float>() : nullptr,
                             return_codes ? codes.data_ptr<uint8_t>() : nullptr, return_codes ? scodes.data_ptr<uint8_t>() : nullptr, rows, cols,
                             global_scale > 0.0 ? (float)global_scale : 0.f, ws.defined() ? ws.data_ptr() : nullptr,
                             return_scales ? gs.data_ptr<float>() : nullptr, stream()));
    std::vector<at::Tensor> out{o};
    if (return_scales) { out.push_back(sc); out.push_back(gs); }
    if (return_codes) { out.push_back(codes); out.push_back(scodes); }
    return out;
}
void float_quantize_multi(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int man_bits, int exp_bits, bool subnormals, bool saturate,
                          int rounding, int prng_bits, uint64_t seed) {
    TORCH_CHECK(ins.size() == outs.size(), "float_quantize_multi: as many outputs as inputs");
    if (ins.empty()) return;
    std::vector<const float*> pi(ins.size());
    std::vector<float*> po(ins.size());
    std::vector<int64_t> n(ins.size());
    for (size_t i = 0; i < ins.size(); ++i) {
        CHECK_INPUT(ins[i]); CHECK_INPUT(outs[i]);
        TORCH_CHECK(ins[i].device() == ins[0].device() && outs[i].device() == ins[0].device() && ins[i].numel() == outs[i].numel(),
                    "float_quantize_multi: tensors must live on one device and outputs must match inputs in size");
        pi[i] = ins[i].data_ptr<float>(); po[i] = outs[i].data_ptr<float>(); n[i] = ins[i].numel();
    }
    c10::cuda::CUDAGuard guard(ins[0].device());
    check(mpt_float_quantize_multi(pi.data(), po.data(), n.data(), (int)ins.size(), man_bits, exp_bits, subnormals, saturate, rounding, prng_bits,
                                   seed, stream()));
}
std::vector<at::Tensor> scale_quantize(at::Tensor a, double normal_max, int margin, bool quantize, int man, int exp, bool subnormals, bool saturate) {
    CHECK_INPUT(a);
    TORCH_CHECK(a.dim() >= 2, "scale_quantize expects at least two dimensions");
    c10::cuda::CUDAGuard guard(a.device());
    const int64_t per = a.size(-1) * a.size(-2), mats = per ? a.numel() / per : 0;
    auto o = at::empty_like(a);
    auto shape = a.sizes().vec();
    shape[shape.size() - 1] = 1; shape[shape.size() - 2] = 1;
    auto sc = at::empty(shape, a.options());
    auto ws = at::empty({(int64_t)mpt_scale_quantize_workspace_bytes(mats)}, a.options().dtype(at::kByte));
    check(mpt_scale_quantize(a.data_ptr<float>(), o.data_ptr<float>(), mats, per, normal_max, margin, quantize, man, exp, subnormals, saturate,
                             sc.data_ptr<float>(), ws.data_ptr(), (size_t)ws.numel(), stream()));
    return {o, sc};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "quant_cuda-compatible front end of the B200 simulated-arithmetic kernels";
    // reference: pybind_cuda.cpp:784-787; the binary8 entry points take the policy as an int, which accepts this enum
    py::enum_<OverflowPolicy>(m, "OverflowPolicy", py::arithmetic(), py::module_local())
        .value("SATURATE_INFTY", OverflowPolicy::SATURATE_INFTY)
        .value("SATURATE_MAXFLOAT", OverflowPolicy::SATURATE_MAXFLOAT)
        .value("SATURATE_MAXFLOAT2", OverflowPolicy::SATURATE_MAXFLOAT2);
    m.def("set_accum_order", [](const std::string& o) { g_accum_order = (o == "seq") ? MPT_ORDER_SEQ : MPT_ORDER_CUDA; });
    m.def("set_reduce_order", [](const std::string& o) { g_reduce_order = (o == "seq") ? MPT_ORDER_SEQ : MPT_ORDER_CUDA; });
    m.def("float_quantize_nearest", &float_quantize_nearest);
    m.def("float_quantize_stochastic", &float_quantize_stochastic);
    m.def("float_quantize_truncate", &float_quantize_truncate);
    m.def("binary8_quantize_nearest", &binary8_quantize_nearest);
    m.def("binary8_quantize_stochastic", &binary8_quantize_stochastic);
    m.def("binary8_quantize_truncate", &binary8_quantize_truncate);
    m.def("superfp_quantize_nearest", &superfp_quantize_nearest);
    m.def("float_quantize_nearest_mm", &float_quantize_nearest_mm);
    m.def("float_quantize_nearest_bmm", &float_quantize_nearest_bmm);
    m.def("float_quantize_nearest_mm_fma", &float_quantize_nearest_mm_fma);
    m.def("float_quantize_nearest_bmm_fma", &float_quantize_nearest_bmm_fma);
    m.def("float_quantize_stochastic_mm", &float_quantize_stochastic_mm);
    m.def("float_quantize_stochastic_bmm", &float_quantize_stochastic_bmm);
    m.def("float_quantize_stochastic_mm_fma", &float_quantize_stochastic_mm_fma);
    m.def("float_quantize_stochastic_bmm_fma", &float_quantize_stochastic_bmm_fma);
    m.def("float_quantize_nearest_softmax_forward", &float_quantize_nearest_softmax_forward);
    m.def("float_quantize_nearest_softmax_lse_forward", &float_quantize_nearest_softmax_lse_forward);
    m.def("float_quantize_nearest_softmax_backward", &float_quantize_nearest_softmax_backward);
    m.def("float_quantize_layernorm_forward", &float_quantize_layernorm_forward);
    m.def("float_quantize_layernorm_backward", &float_quantize_layernorm_backward);
    m.def("superfp_quantize_nearest_mm", &superfp_quantize_nearest_mm);
    m.def("superfp_quantize_nearest_bmm", &superfp_quantize_nearest_bmm);
    m.def("superfp_quantize_nearest_mm_fma", &superfp_quantize_nearest_mm_fma);
    m.def("superfp_quantize_nearest_bmm_fma", &superfp_quantize_nearest_bmm_fma);
    m.def("superfp_quantize_nearest_softmax_forward", &superfp_quantize_nearest_softmax_forward);
    m.def("superfp_quantize_nearest_softmax_lse_forward", &superfp_quantize_nearest_softmax_lse_forward);
    m.def("superfp_quantize_nearest_softmax_backward", &superfp_quantize_nearest_softmax_backward);
    m.def("binary8_quantize_nearest_softmax_forward", &binary8_quantize_nearest_softmax_forward);
    m.def("binary8_quantize_nearest_softmax_lse_forward", &binary8_quantize_nearest_softmax_lse_forward);
    m.def("binary8_quantize_nearest_softmax_backward", &binary8_quantize_nearest_softmax_backward);
    m.def("superfp_quantize_layernorm_forward", &superfp_quantize_layernorm_forward);
    m.def("superfp_quantize_layernorm_backward", &superfp_quantize_layernorm_backward);
    m.def("binary8_quantize_layernorm_forward", &binary8_quantize_layernorm_forward);
    m.def("binary8_quantize_layernorm_backward", &binary8_quantize_layernorm_backward);
    m.def("qsum_rows", &qsum_rows);
    m.def("float_conv2d_nearest", &float_conv2d_nearest, py::arg("x"), py::arg("wt"), py::arg("y"), py::arg("groups"), py::arg("kernel_size"),
          py::arg("stride"), py::arg("padding"), py::arg("dilation"), py::arg("man_add"), py::arg("exp_add"), py::arg("man_mul"), py::arg("exp_mul"),
          py::arg("subnormals"), py::arg("saturate"), py::arg("fma") = false);
    m.def("mx_quantize", &mx_quantize, py::arg("a"), py::arg("elem_format") = "e4m3", py::arg("block") = 32, py::arg("return_scales") = false,
          py::arg("return_codes") = false);
    m.def("nvfp4_quantize", &nvfp4_quantize, py::arg("a"), py::arg("global_scale") = 0.0, py::arg("return_scales") = false,
          py::arg("return_codes") = false);
    m.def("float_quantize_multi", &float_quantize_multi, py::arg("ins"), py::arg("outs"), py::arg("man_bits"), py::arg("exp_bits"),
          py::arg("subnormals"), py::arg("saturate"), py::arg("rounding") = 0, py::arg("prng_bits") = 0, py::arg("seed") = 0);
    m.def("scale_quantize", &scale_quantize);
}
