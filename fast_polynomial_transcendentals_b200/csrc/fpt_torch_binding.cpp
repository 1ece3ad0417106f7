// Compiled PyTorch binding of the element-wise hot operators: tensor checks, output allocation, device guard and the
// call into the C ABI in C++, so that an eager call costs a function call and a kernel launch, not an interpreter
// round trip per argument.
//
// Two doors into the same functions:
//   * a Python extension module (`_fpt_torch`), what `spline_ops.py` calls for its hot operators;
//   * dispatcher operators `fpt_b200::unary`, `fpt_b200::binary_bwd`, `fpt_b200::swish_mul`, `fpt_b200::swish_mul_bwd`,
//     `fpt_b200::swish_mul_packed`, `fpt_b200::swish_mul_packed_bwd` (TORCH_LIBRARY), for graphs and C++ callers.
// Checks and messages are the reference's (reference: autonumerics_zero/spline_ops/spline_ops.cpp:293-298 tensor
// checks, :1149-1185 unary / variant dispatch, :1647-1649 and :1781-1785 pair checks, :1671-1686 packed shape rules);
// unlike the reference the launch runs under a guard for the tensor's device and element counts stay 64-bit.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <tuple>

#include "../../include/fpt_b200.h"

namespace {

const char* const kFunctionNames[] = {"sigmoid", "tanh", "swish", "erf", "gelu"};

void check_input(const at::Tensor& x, const char* name) {
    TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, name, " must be float16 or bfloat16");
}

int dtype_id(const at::Tensor& x) { return x.scalar_type() == at::kBFloat16 ? FPT_BF16 : FPT_FP16; }

int64_t checked_source(int64_t source, const at::Tensor& x) {
    TORCH_CHECK(source == 0 || source == 1, "coeff_source_id must be 0 (current) or 1 (sollya)");
    TORCH_CHECK(source == 0 || x.scalar_type() == at::kBFloat16, "FP16 spline kernels only support coeff_source=current");
    return source;
}

void check_same(const at::Tensor& a, const at::Tensor& b, const char* an, const char* bn) {
    TORCH_CHECK(a.scalar_type() == b.scalar_type(), an, " and ", bn, " must have the same dtype");
    TORCH_CHECK(a.numel() == b.numel(), an, " and ", bn, " must have the same number of elements");
    TORCH_CHECK(a.device() == b.device(), an, " and ", bn, " must be on the same device");
}

void check_status(int status, const char* entry) {
    TORCH_CHECK(status == 0, entry, " failed with status ", status, ": ", fpt_status_string(status));
}

fpt_stream_t stream_of(const at::Tensor& x) {
    return reinterpret_cast<fpt_stream_t>(at::cuda::getCurrentCUDAStream(x.device().index()).stream());
}

at::Tensor unary(const at::Tensor& x, int64_t function, int64_t direction, int64_t degree, int64_t source) {
    check_input(x, "x");
    TORCH_CHECK(function >= 0 && function <= FPT_FN_GELU, "unknown function");
    source = checked_source(source, x);
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor out = at::empty_like(x);
    const int rc = fpt_unary(out.data_ptr(), x.data_ptr(), x.numel(), int(function), int(direction), int(degree), dtype_id(x),
                             int(source), stream_of(x));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported ", kFunctionNames[function],
                direction == FPT_FWD ? " forward degree: " : " backward degree: ", degree);
    check_status(rc, "fpt_unary");
    return out;
}

at::Tensor binary_bwd(const at::Tensor& grad_out, const at::Tensor& x, int64_t function, int64_t degree, int64_t source) {
    check_input(grad_out, "grad_out");
    check_input(x, "x");
    check_same(grad_out, x, "grad_out", "x");
    TORCH_CHECK(function >= 0 && function <= FPT_FN_GELU, "unknown function");
    source = checked_source(source, x);
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor grad_in = at::empty_like(x);
    const int rc = fpt_binary_bwd(grad_in.data_ptr(), grad_out.data_ptr(), x.data_ptr(), x.numel(), int(function), int(degree),
                                  dtype_id(x), int(source), stream_of(x));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported ", kFunctionNames[function], " backward degree: ", degree);
    check_status(rc, "fpt_binary_bwd");
    return grad_in;
}

at::Tensor swish_mul(const at::Tensor& gate, const at::Tensor& up, int64_t degree, int64_t source) {
    check_input(gate, "gate");
    check_input(up, "up");
    check_same(gate, up, "gate", "up");
    source = checked_source(source, gate);
    const c10::cuda::CUDAGuard guard(gate.device());
    at::Tensor out = at::empty_like(up);
    const int rc = fpt_swish_mul(out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.numel(), int(degree), dtype_id(gate),
                                 int(source), stream_of(gate));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported swish_mul forward degree: ", degree);
    check_status(rc, "fpt_swish_mul");
    return out;
}

std::tuple<at::Tensor, at::Tensor> swish_mul_bwd(const at::Tensor& grad_out, const at::Tensor& gate, const at::Tensor& up,
                                                 int64_t degree, int64_t source) {
    check_input(grad_out, "grad_out");
    check_input(gate, "gate");
    check_input(up, "up");
    TORCH_CHECK(grad_out.scalar_type() == gate.scalar_type() && gate.scalar_type() == up.scalar_type(),
                "grad_out, gate, and up must have the same dtype");
    TORCH_CHECK(grad_out.numel() == gate.numel() && gate.numel() == up.numel(),
                "grad_out, gate, and up must have the same number of elements");
    TORCH_CHECK(grad_out.device() == gate.device() && gate.device() == up.device(),
                "grad_out, gate, and up must be on the same device");
    source = checked_source(source, gate);
    const c10::cuda::CUDAGuard guard(gate.device());
    at::Tensor grad_gate = at::empty_like(gate), grad_up = at::empty_like(up);
    const int rc = fpt_swish_mul_bwd(grad_gate.data_ptr(), grad_up.data_ptr(), grad_out.data_ptr(), gate.data_ptr(),
                                     up.data_ptr(), gate.numel(), int(degree), dtype_id(gate), int(source), stream_of(gate));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported swish_mul backward degree: ", degree);
    check_status(rc, "fpt_swish_mul_bwd");
    return {grad_gate, grad_up};
}

int64_t packed_hidden(const at::Tensor& packed) {
    TORCH_CHECK(packed.dim() >= 1, "packed gate/up tensor must have at least one dimension");
    const int64_t width = packed.size(-1);
    TORCH_CHECK(width % 2 == 0, "packed gate/up last dimension must be even");
    TORCH_CHECK((width / 2) % 2 == 0, "packed SwiGLU hidden size must be even");
    return width / 2;
}

at::Tensor swish_mul_packed(const at::Tensor& packed, int64_t degree, int64_t source) {
    check_input(packed, "packed");
    const int64_t hidden = packed_hidden(packed);
    source = checked_source(source, packed);
    const c10::cuda::CUDAGuard guard(packed.device());
    auto shape = packed.sizes().vec();
    shape.back() = hidden;
    at::Tensor out = at::empty(shape, packed.options());
    if (packed.numel() == 0) return out;
    const int rc = fpt_swish_mul_packed(out.data_ptr(), packed.data_ptr(), packed.numel() / (2 * hidden), hidden, int(degree),
                                        dtype_id(packed), int(source), stream_of(packed));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported packed swish_mul forward degree: ", degree);
    check_status(rc, "fpt_swish_mul_packed");
    return out;
}

at::Tensor swish_mul_packed_bwd(const at::Tensor& grad_out, const at::Tensor& packed, int64_t degree, int64_t source) {
    check_input(grad_out, "grad_out");
    check_input(packed, "packed");
    const int64_t hidden = packed_hidden(packed);
    TORCH_CHECK(grad_out.scalar_type() == packed.scalar_type(), "grad_out and packed must have the same dtype");
    TORCH_CHECK(grad_out.device() == packed.device(), "grad_out and packed must be on the same device");
    TORCH_CHECK(grad_out.numel() * 2 == packed.numel() && (grad_out.dim() == 0 || grad_out.size(-1) == hidden),
                "grad_out must match the packed tensor with its last dimension halved");
    source = checked_source(source, packed);
    const c10::cuda::CUDAGuard guard(packed.device());
    at::Tensor grad_packed = at::empty_like(packed);
    if (packed.numel() == 0) return grad_packed;
    const int rc = fpt_swish_mul_packed_bwd(grad_packed.data_ptr(), grad_out.data_ptr(), packed.data_ptr(),
                                            packed.numel() / (2 * hidden), hidden, int(degree), dtype_id(packed), int(source),
                                            stream_of(packed));
    TORCH_CHECK(rc != FPT_ERR_UNKNOWN_PROGRAM, "Unsupported packed swish_mul backward degree: ", degree);
    check_status(rc, "fpt_swish_mul_packed_bwd");
    return grad_packed;
}

}  // namespace

TORCH_LIBRARY(fpt_b200, m) {
    m.def("unary(Tensor x, int function, int direction, int degree, int source) -> Tensor");
    m.def("binary_bwd(Tensor grad_out, Tensor x, int function, int degree, int source) -> Tensor");
    m.def("swish_mul(Tensor gate, Tensor up, int degree, int source) -> Tensor");
    m.def("swish_mul_bwd(Tensor grad_out, Tensor gate, Tensor up, int degree, int source) -> (Tensor, Tensor)");
    m.def("swish_mul_packed(Tensor packed, int degree, int source) -> Tensor");
    m.def("swish_mul_packed_bwd(Tensor grad_out, Tensor packed, int degree, int source) -> Tensor");
}

TORCH_LIBRARY_IMPL(fpt_b200, CUDA, m) {
    m.impl("unary", &unary);
    m.impl("binary_bwd", &binary_bwd);
    m.impl("swish_mul", &swish_mul);
    m.impl("swish_mul_bwd", &swish_mul_bwd);
    m.impl("swish_mul_packed", &swish_mul_packed);
    m.impl("swish_mul_packed_bwd", &swish_mul_packed_bwd);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "compiled binding of the element-wise hot operators over the fpt_* C ABI";
    m.def("unary", &unary);
    m.def("binary_bwd", &binary_bwd);
    m.def("swish_mul", &swish_mul);
    m.def("swish_mul_bwd", &swish_mul_bwd);
    m.def("swish_mul_packed", &swish_mul_packed);
    m.def("swish_mul_packed_bwd", &swish_mul_packed_bwd);
}
