// pybind11 / PyTorch binding of the C ABI (include/ldn_b200.h): the compiled counterpart of the reference's
// extension module (core/cuda/norm_dist.cpp:40-204).  Twelve functions with the reference's names, argument
// order and in-place semantics; every tensor must be a contiguous CUDA tensor (norm_dist.cpp:8-10), shapes are
// read from the tensors as the reference does (norm_dist.cpp:44,73,127).  Differences: launches go to the
// current stream of the tensors' device (with a device guard) and a non-zero status raises.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "ldn_b200.h"

namespace {

using torch::Tensor;

const float* fptr(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    return t.data_ptr<float>();  // raises for a wrong dtype, like the reference
}
float* fptr_mut(Tensor& t, const char* name) { return const_cast<float*>(fptr(t, name)); }
int* iptr(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    return t.data_ptr<int>();
}
float* opt_fptr(c10::optional<Tensor>& t, const char* name) { return t.has_value() ? fptr_mut(*t, name) : nullptr; }

ldn_stream_t stream() { return reinterpret_cast<ldn_stream_t>(at::cuda::getCurrentCUDAStream().stream()); }

void check(int status, const char* what) {
    TORCH_CHECK(status == 0, what, " failed with status ", status, ": ", ldn_status_string(status));
}

void norm_dist_forward(Tensor& input, Tensor& weight, Tensor& output, int G, float p) {
    const float *x = fptr(input, "input"), *w = fptr(weight, "weight");
    float* y = fptr_mut(output, "output");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_norm_dist_forward(x, w, input.size(0), output.size(1), input.size(1), G, input.size(2), y, p, stream()),
          "norm_dist_forward");
}

void norm_dist_forward_with_max(Tensor& input, Tensor& weight, Tensor& max_output, Tensor& output, int G, float p) {
    const float *x = fptr(input, "input"), *w = fptr(weight, "weight"), *m = fptr(max_output, "max_output");
    float* y = fptr_mut(output, "output");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_norm_dist_forward_with_max(x, w, m, input.size(0), output.size(1), input.size(1), G, input.size(2), y, p,
                                         stream()),
          "norm_dist_forward_with_max");
}

void norm_dist_backward_input(Tensor& grad_output, Tensor& input, Tensor& weight, Tensor& output, Tensor& grad_input,
                              int G, float p) {
    const float *g = fptr(grad_output, "grad_output"), *x = fptr(input, "input"), *w = fptr(weight, "weight"),
                *y = fptr(output, "output");
    float* gx = fptr_mut(grad_input, "grad_input");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_norm_dist_backward_input(g, x, w, y, grad_output.size(0), output.size(1), input.size(1), G, input.size(2),
                                       gx, p, stream()),
          "norm_dist_backward_input");
}

// grad_input may be None when the caller does not need it (an extension of the reference interface)
void norm_dist_backward_input_weight(Tensor& grad_output, Tensor& input, Tensor& weight, Tensor& output,
                                     c10::optional<Tensor> grad_input, Tensor& grad_weight, int G, float p) {
    const float *g = fptr(grad_output, "grad_output"), *x = fptr(input, "input"), *w = fptr(weight, "weight"),
                *y = fptr(output, "output");
    float* gx = opt_fptr(grad_input, "grad_input");
    float* gw = fptr_mut(grad_weight, "grad_weight");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_norm_dist_backward_input_weight(g, x, w, y, grad_output.size(0), output.size(1), input.size(1), G,
                                              input.size(2), gx, gw, p, stream()),
          "norm_dist_backward_input_weight");
}

void inf_dist_forward(Tensor& input, Tensor& weight, Tensor& output, Tensor& pos, int G) {
    const float *x = fptr(input, "input"), *w = fptr(weight, "weight");
    float* y = fptr_mut(output, "output");
    int* ps = iptr(pos, "pos");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_inf_dist_forward(x, w, input.size(0), output.size(1), input.size(1), G, input.size(2), y, ps, stream()),
          "inf_dist_forward");
}

void inf_dist_forward_nograd(Tensor& input, Tensor& weight, Tensor& output, int G) {
    const float *x = fptr(input, "input"), *w = fptr(weight, "weight");
    float* y = fptr_mut(output, "output");
    const c10::cuda::CUDAGuard guard(input.device());
    check(ldn_inf_dist_forward_nograd(x, w, input.size(0), output.size(1), input.size(1), G, input.size(2), y, stream()),
          "inf_dist_forward_nograd");
}

void inf_dist_backward_input(Tensor& grad_output, Tensor& pos, Tensor& grad_input, int G) {
    const float* g = fptr(grad_output, "grad_output");
    const int* ps = iptr(pos, "pos");
    float* gx = fptr_mut(grad_input, "grad_input");
    const c10::cuda::CUDAGuard guard(grad_output.device());
    check(ldn_inf_dist_backward_input(g, ps, grad_output.size(0), grad_output.size(1), grad_input.size(1), G,
                                      grad_input.size(2), gx, stream()),
          "inf_dist_backward_input");
}

void inf_dist_backward_input_weight(Tensor& grad_output, Tensor& pos, c10::optional<Tensor> grad_input,
                                    Tensor& grad_weight, int G) {
    const float* g = fptr(grad_output, "grad_output");
    const int* ps = iptr(pos, "pos");
    float* gx = opt_fptr(grad_input, "grad_input");
    float* gw = fptr_mut(grad_weight, "grad_weight");
    const c10::cuda::CUDAGuard guard(grad_output.device());
    check(ldn_inf_dist_backward_input_weight(g, ps, grad_output.size(0), grad_output.size(1), grad_weight.size(1) * G, G,
                                             grad_output.size(2), gx, gw, stream()),
          "inf_dist_backward_input_weight");
}

void bound_inf_dist_forward(Tensor& inputL, Tensor& inputU, Tensor& weight, Tensor& outputL, Tensor& outputU,
                            Tensor& posL, Tensor& posU, int G) {
    const float *xl = fptr(inputL, "inputL"), *xu = fptr(inputU, "inputU"), *w = fptr(weight, "weight");
    float *yl = fptr_mut(outputL, "outputL"), *yu = fptr_mut(outputU, "outputU");
    int *pl = iptr(posL, "posL"), *pu = iptr(posU, "posU");
    const c10::cuda::CUDAGuard guard(inputL.device());
    check(ldn_bound_inf_dist_forward(xl, xu, w, inputL.size(0), outputL.size(1), inputL.size(1), G, inputL.size(2), yl, yu,
                                     pl, pu, stream()),
          "bound_inf_dist_forward");
}

void bound_inf_dist_forward_nograd(Tensor& inputL, Tensor& inputU, Tensor& weight, Tensor& outputL, Tensor& outputU,
                                   int G) {
    const float *xl = fptr(inputL, "inputL"), *xu = fptr(inputU, "inputU"), *w = fptr(weight, "weight");
    float *yl = fptr_mut(outputL, "outputL"), *yu = fptr_mut(outputU, "outputU");
    const c10::cuda::CUDAGuard guard(inputL.device());
    check(ldn_bound_inf_dist_forward_nograd(xl, xu, w, inputL.size(0), outputL.size(1), inputL.size(1), G, inputL.size(2),
                                            yl, yu, stream()),
          "bound_inf_dist_forward_nograd");
}

void bound_inf_dist_backward_input(Tensor& grad_outputL, Tensor& grad_outputU, Tensor& posL, Tensor& posU,
                                   Tensor& grad_inputL, Tensor& grad_inputU, int G) {
    const float *gl = fptr(grad_outputL, "grad_outputL"), *gu = fptr(grad_outputU, "grad_outputU");
    const int *pl = iptr(posL, "posL"), *pu = iptr(posU, "posU");
    float *gxl = fptr_mut(grad_inputL, "grad_inputL"), *gxu = fptr_mut(grad_inputU, "grad_inputU");
    const c10::cuda::CUDAGuard guard(grad_outputL.device());
    check(ldn_bound_inf_dist_backward_input(gl, gu, pl, pu, grad_outputL.size(0), grad_outputL.size(1), grad_inputL.size(1),
                                            G, grad_inputL.size(2), gxl, gxu, stream()),
          "bound_inf_dist_backward_input");
}

void bound_inf_dist_backward_input_weight(Tensor& grad_outputL, Tensor& grad_outputU, Tensor& posL, Tensor& posU,
                                          Tensor& grad_inputL, Tensor& grad_inputU, Tensor& grad_weight, int G) {
    const float *gl = fptr(grad_outputL, "grad_outputL"), *gu = fptr(grad_outputU, "grad_outputU");
    const int *pl = iptr(posL, "posL"), *pu = iptr(posU, "posU");
    float *gxl = fptr_mut(grad_inputL, "grad_inputL"), *gxu = fptr_mut(grad_inputU, "grad_inputU");
    float* gw = fptr_mut(grad_weight, "grad_weight");
    const c10::cuda::CUDAGuard guard(grad_outputL.device());
    check(ldn_bound_inf_dist_backward_input_weight(gl, gu, pl, pu, grad_outputL.size(0), grad_outputL.size(1),
                                                   grad_weight.size(1) * G, G, grad_outputL.size(2), gxl, gxu, gw,
                                                   stream()),
          "bound_inf_dist_backward_input_weight");
}

void check_status() { check(ldn_check_status(stream()), "device status check"); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("norm_dist_forward", &norm_dist_forward);
    m.def("norm_dist_forward_with_max", &norm_dist_forward_with_max);
    m.def("norm_dist_backward_input", &norm_dist_backward_input);
    m.def("norm_dist_backward_input_weight", &norm_dist_backward_input_weight);
    m.def("inf_dist_forward", &inf_dist_forward);
    m.def("inf_dist_forward_nograd", &inf_dist_forward_nograd);
    m.def("inf_dist_backward_input", &inf_dist_backward_input);
    m.def("inf_dist_backward_input_weight", &inf_dist_backward_input_weight);
    m.def("bound_inf_dist_forward", &bound_inf_dist_forward);
    m.def("bound_inf_dist_forward_nograd", &bound_inf_dist_forward_nograd);
    m.def("bound_inf_dist_backward_input", &bound_inf_dist_backward_input);
    m.def("bound_inf_dist_backward_input_weight", &bound_inf_dist_backward_input_weight);
    m.def("check_status", &check_status);
}
