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

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "quant_cuda-compatible front end of the B200 simulated-arithmetic kernels";
    m.attr("SATURATE_INFTY") = (int)MPT_SATURATE_INFTY;
    m.attr("SATURATE_MAXFLOAT") = (int)MPT_SATURATE_MAXFLOAT;
    m.attr("SATURATE_MAXFLOAT2") = (int)MPT_SATURATE_MAXFLOAT2;
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
}
