// PyTorch extension module `cuda`: the drop-in for microsoft/RepDL's `repdl.backend.cuda`.
//
// Exports the ten functions the reference's backend/cuda/bind.cpp:12-19 registers (same names,
// positional arguments and result shapes as backend/cuda/*.cu declare them), each implemented by
// one call into the C ABI of include/repdl_b200.h, plus exp2d / log1d (backend/cuda/math.h:14-15,
// which the reference never exports) and div / sqrt.  Differences from the reference, on purpose:
//   * results are allocated on the INPUT's device and kernels run on the CURRENT stream of that
//     device (the reference allocates on the current device and launches on the legacy stream);
//   * inputs are checked (device, dtype, rank, shape) and made contiguous when needed (the
//     reference reads raw pointers and silently assumes contiguity);
//   * a failing launch raises instead of being ignored.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "repdl_b200.h"

namespace {

void *cur_stream() { return (void *)at::cuda::getCurrentCUDAStream().stream(); }

void ok(int status, const char *what)
{
    TORCH_CHECK(status == 0, "repdl_b200 ", what, " failed: status ", status, " (",
                repdl_b200_strerror(status), ")");
}

const torch::Tensor &need(const torch::Tensor &t, const char *name, int64_t dim,
                          at::ScalarType dt = at::kFloat)
{
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == dt, name, " must be ", dt, ", got ", t.scalar_type());
    TORCH_CHECK(dim < 0 || t.dim() == dim, name, " must have ", dim, " dimensions, got ", t.dim());
    return t;
}

const float *fp(const torch::Tensor &t) { return t.const_data_ptr<float>(); }
float *fpw(torch::Tensor &t) { return t.mutable_data_ptr<float>(); }

torch::Tensor rowmajor(const torch::Tensor &t)
{
    if (t.stride(1) == 1 && t.stride(0) >= std::max<int64_t>(1, t.size(1))) return t;
    return t.contiguous();
}

// backend/cpu/summation.cpp:15: float factor = average ? 1.0 / count : 1.0
float mean_factor(bool average, int64_t count)
{
    return (average && count > 0) ? (float)(1.0 / (double)count) : 1.0f;
}

// ---- backend/cuda/matrix_multiplication.cu:234-260 ----
torch::Tensor mm(const torch::Tensor &input, const torch::Tensor &mat2, bool transA, bool transB)
{
    need(input, "input", 2);
    need(mat2, "mat2", 2);
    TORCH_CHECK(input.device() == mat2.device(), "mm: operands on different devices");
    const int64_t M = transA ? input.size(1) : input.size(0);
    const int64_t K = transA ? input.size(0) : input.size(1);
    const int64_t N = transB ? mat2.size(0) : mat2.size(1);
    TORCH_CHECK((transB ? mat2.size(1) : mat2.size(0)) == K, "mm: inner dimensions differ");
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor a = rowmajor(input), b = rowmajor(mat2);
    torch::Tensor out = torch::empty({M, N}, input.options());
    ok(repdl_b200_mm(fp(a), fp(b), fpw(out), M, N, K, transA, transB, a.stride(0), b.stride(0),
                     std::max<int64_t>(N, 1), cur_stream()),
       "mm");
    return out;
}

// ---- backend/cuda/convolution.cu:153-173 ----
torch::Tensor conv2d(const torch::Tensor &input, const torch::Tensor &kernel, unsigned strideH,
                     unsigned strideW, unsigned paddingH, unsigned paddingW, unsigned groups)
{
    need(input, "input", 4);
    need(kernel, "kernel", 4);
    TORCH_CHECK(groups > 0 && kernel.size(1) * groups == input.size(1),
                "conv2d: kernel.size(1) * groups != input channels");
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous(), k = kernel.contiguous();
    const int64_t N = x.size(0), IC = x.size(1), H = x.size(2), W = x.size(3);
    const int64_t OC = k.size(0), KH = k.size(2), KW = k.size(3);
    TORCH_CHECK(strideH > 0 && strideW > 0, "conv2d: stride must be positive");
    TORCH_CHECK(H + 2 * paddingH >= KH && W + 2 * paddingW >= KW, "conv2d: the kernel does not fit into the padded image");
    const int64_t OH = (H + 2 * paddingH - KH) / strideH + 1, OW = (W + 2 * paddingW - KW) / strideW + 1;
    torch::Tensor out = torch::empty({N, OC, OH, OW}, input.options());
    ok(repdl_b200_conv2d(fp(x), fp(k), fpw(out), N, IC, H, W, OC, KH, KW, strideH, strideW,
                         paddingH, paddingW, groups, cur_stream()),
       "conv2d");
    return out;
}

// ---- backend/cuda/convolution.cu:259-277 ----
torch::Tensor conv2d_grad_input(const torch::Tensor &grad_output, const torch::Tensor &kernel,
                                unsigned H, unsigned W, unsigned strideH, unsigned strideW,
                                unsigned paddingH, unsigned paddingW)
{
    need(grad_output, "grad_output", 4);
    need(kernel, "kernel", 4);
    c10::cuda::CUDAGuard guard(grad_output.device());
    torch::Tensor go = grad_output.contiguous(), k = kernel.contiguous();
    const int64_t N = go.size(0), OC = k.size(0), IC = k.size(1), KH = k.size(2), KW = k.size(3);
    // the kernels index grad_output with the extents they derive from H, W: it must have them
    TORCH_CHECK(strideH > 0 && strideW > 0, "conv2d_grad_input: stride must be positive");
    TORCH_CHECK((int64_t)H + 2 * paddingH >= KH && (int64_t)W + 2 * paddingW >= KW,
                "conv2d_grad_input: the kernel does not fit into the padded image");
    TORCH_CHECK(go.size(1) == OC && go.size(2) == ((int64_t)H + 2 * paddingH - KH) / strideH + 1 &&
                    go.size(3) == ((int64_t)W + 2 * paddingW - KW) / strideW + 1,
                "conv2d_grad_input: grad_output does not have the shape of this convolution's output");
    torch::Tensor out = torch::empty({N, IC, (int64_t)H, (int64_t)W}, grad_output.options());
    ok(repdl_b200_conv2d_grad_input(fp(go), fp(k), fpw(out), N, IC, H, W, OC, KH, KW, strideH,
                                    strideW, paddingH, paddingW, cur_stream()),
       "conv2d_grad_input");
    return out;
}

// ---- backend/cuda/convolution.cu:359-377 ----
torch::Tensor conv2d_grad_kernel(const torch::Tensor &grad_output, const torch::Tensor &input,
                                 unsigned KH, unsigned KW, unsigned strideH, unsigned strideW,
                                 unsigned paddingH, unsigned paddingW)
{
    need(grad_output, "grad_output", 4);
    need(input, "input", 4);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor go = grad_output.contiguous(), x = input.contiguous();
    const int64_t N = x.size(0), IC = x.size(1), H = x.size(2), W = x.size(3), OC = go.size(1);
    TORCH_CHECK(strideH > 0 && strideW > 0, "conv2d_grad_kernel: stride must be positive");
    TORCH_CHECK(H + 2 * paddingH >= (int64_t)KH && W + 2 * paddingW >= (int64_t)KW,
                "conv2d_grad_kernel: the kernel does not fit into the padded image");
    TORCH_CHECK(go.size(0) == N && go.size(2) == (H + 2 * paddingH - (int64_t)KH) / strideH + 1 &&
                    go.size(3) == (W + 2 * paddingW - (int64_t)KW) / strideW + 1,
                "conv2d_grad_kernel: grad_output does not have the shape of this convolution's output");
    torch::Tensor out = torch::empty({OC, IC, (int64_t)KH, (int64_t)KW}, input.options());
    ok(repdl_b200_conv2d_grad_kernel(fp(go), fp(x), fpw(out), N, IC, H, W, OC, KH, KW, strideH,
                                     strideW, paddingH, paddingW, cur_stream()),
       "conv2d_grad_kernel");
    return out;
}

// ---- backend/cuda/summation.cu:33-43, 59-71, 94-105, 132-144 ----
torch::Tensor sum1d(const torch::Tensor &input, bool average)
{
    need(input, "input", 1);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    const int64_t n = x.numel();
    torch::Tensor out = torch::empty({}, input.options());
    const size_t nbytes = repdl_b200_sum1d_scratch_bytes(n);
    torch::Tensor scratch = torch::empty({(int64_t)nbytes}, input.options().dtype(at::kByte));
    ok(repdl_b200_sum1d(fp(x), fpw(out), n, mean_factor(average, n), scratch.data_ptr(), nbytes,
                        cur_stream()),
       "sum1d");
    return out;
}

torch::Tensor sum2d_dim0(const torch::Tensor &input, bool keepdim, bool average)
{
    need(input, "input", 2);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor out = torch::empty({1, x.size(1)}, input.options());
    ok(repdl_b200_sum2d_dim0(fp(x), fpw(out), x.size(0), x.size(1), mean_factor(average, x.size(0)),
                             cur_stream()),
       "sum2d_dim0");
    return keepdim ? out : out.squeeze();
}

torch::Tensor sum2d_dim1(const torch::Tensor &input, bool keepdim, bool average)
{
    need(input, "input", 2);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor out = torch::empty({x.size(0), 1}, input.options());
    ok(repdl_b200_sum2d_dim1(fp(x), fpw(out), x.size(0), x.size(1), mean_factor(average, x.size(1)),
                             cur_stream()),
       "sum2d_dim1");
    return keepdim ? out : out.squeeze();
}

torch::Tensor sum4d_dim023(const torch::Tensor &input, bool keepdim, bool average)
{
    need(input, "input", 4);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    const int64_t N = x.size(0), C = x.size(1), HW = x.size(2) * x.size(3);
    torch::Tensor out = torch::empty({1, C, 1, 1}, input.options());
    ok(repdl_b200_sum4d_dim023(fp(x), fpw(out), N, C, HW, mean_factor(average, N * HW), cur_stream()),
       "sum4d_dim023");
    return keepdim ? out : out.squeeze();
}

// ---- elementwise ----
template <int (*FN)(const float *, float *, int64_t, void *)>
torch::Tensor unary(const torch::Tensor &input, int64_t dim, const char *what)
{
    need(input, "input", dim);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor out = torch::empty_like(x);
    ok(FN(fp(x), fpw(out), x.numel(), cur_stream()), what);
    return out;
}

torch::Tensor exp2d(const torch::Tensor &input) { return unary<repdl_b200_exp>(input, 2, "exp2d"); }
torch::Tensor log1d(const torch::Tensor &input) { return unary<repdl_b200_log>(input, 1, "log1d"); }
torch::Tensor exp_any(const torch::Tensor &input) { return unary<repdl_b200_exp>(input, -1, "exp"); }
torch::Tensor log_any(const torch::Tensor &input) { return unary<repdl_b200_log>(input, -1, "log"); }
torch::Tensor sqrt_any(const torch::Tensor &input) { return unary<repdl_b200_sqrt>(input, -1, "sqrt"); }

torch::Tensor div_scalar(const torch::Tensor &input, double divisor)
{
    need(input, "input", -1);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor out = torch::empty_like(x);
    ok(repdl_b200_div_scalar(fp(x), (float)divisor, fpw(out), x.numel(), cur_stream()), "div");
    return out;
}

torch::Tensor div_tensor(const torch::Tensor &input, const torch::Tensor &other)
{
    need(input, "input", -1);
    need(other, "other", -1);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor d = other.expand_as(x).contiguous();
    torch::Tensor out = torch::empty_like(x);
    ok(repdl_b200_div(fp(x), fp(d), fpw(out), x.numel(), cur_stream()), "div");
    return out;
}

// ---- backend/cuda/softmax.cpp:15-21, backend/cuda/cross_entropy.cpp:15-24 ----
torch::Tensor softmax(const torch::Tensor &input)
{
    need(input, "input", 2);
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous();
    torch::Tensor out = torch::empty_like(x);
    ok(repdl_b200_softmax(fp(x), fpw(out), x.size(0), x.size(1), cur_stream()), "softmax");
    return out;
}

torch::Tensor cross_entropy(const torch::Tensor &input, const torch::Tensor &target)
{
    need(input, "input", 2);
    need(target, "target", 1, at::kLong);
    TORCH_CHECK(target.size(0) == input.size(0), "cross_entropy: target length != rows");
    c10::cuda::CUDAGuard guard(input.device());
    torch::Tensor x = input.contiguous(), t = target.contiguous();
    torch::Tensor out = torch::empty({}, input.options());
    torch::Tensor rows = torch::empty({x.size(0)}, input.options());
    ok(repdl_b200_cross_entropy(fp(x), t.const_data_ptr<int64_t>(), fpw(out), x.size(0), x.size(1),
                                fpw(rows), cur_stream()),
       "cross_entropy");
    return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "repdl_b200: sm_100a drop-in for repdl.backend.cuda";
    // the reference's ten names (backend/cuda/bind.cpp:12-19)
    m.def("conv2d", &conv2d);
    m.def("conv2d_grad_input", &conv2d_grad_input);
    m.def("conv2d_grad_kernel", &conv2d_grad_kernel);
    m.def("cross_entropy", &cross_entropy);
    m.def("mm", &mm);
    m.def("softmax", &softmax);
    m.def("sum1d", &sum1d);
    m.def("sum2d_dim0", &sum2d_dim0);
    m.def("sum2d_dim1", &sum2d_dim1);
    m.def("sum4d_dim023", &sum4d_dim023);
    // additions
    m.def("exp2d", &exp2d);
    m.def("log1d", &log1d);
    m.def("exp", &exp_any);
    m.def("log", &log_any);
    m.def("sqrt", &sqrt_any);
    m.def("div_scalar", &div_scalar);
    m.def("div", &div_tensor);
}
