// TEST INFRASTRUCTURE ONLY.  extern "C" entry points in front of the upstream reference's own CUDA
// launchers (declared in its core/cuda/norm_dist.h), so that GPU tests and the benchmark can run the
// reference kernels themselves beside the kernels of this repository.  This file is compiled together
// with the reference's .cu files where they lie (see oracle/build.py); it contains no reference code.
// The run-time p -> template dispatch below restates core/cuda/norm_dist.cpp:17-35,45-52,74,88.
#include <cuda_runtime.h>
#include "norm_dist.h"

#define LDN_REF_DISPATCH(P, FUN, ...)                                 \
    do {                                                              \
        float p_ = (P);                                               \
        int ip_ = (p_ == float(int(p_))) ? int(p_) : -1;              \
        switch (ip_) {                                                \
            case 0: norm_dist<0>::FUN(__VA_ARGS__); break;            \
            case 1: norm_dist<1>::FUN(__VA_ARGS__); break;            \
            case 2: norm_dist<2>::FUN(__VA_ARGS__); break;            \
            case 3: norm_dist<3>::FUN(__VA_ARGS__); break;            \
            case 4: norm_dist<4>::FUN(__VA_ARGS__); break;            \
            case 5: norm_dist<5>::FUN(__VA_ARGS__); break;            \
            case 6: norm_dist<6>::FUN(__VA_ARGS__); break;            \
            case 7: norm_dist<7>::FUN(__VA_ARGS__); break;            \
            case 8: norm_dist<8>::FUN(__VA_ARGS__); break;            \
            default: norm_dist<-1>::FUN(__VA_ARGS__);                 \
        }                                                             \
    } while (0)

extern "C" {

int ldn_ref_norm_dist_forward(const float* x, const float* w, float* y, int B, int CO, int CI, int G, int HW, float p) {
    if (p <= 10.0f) LDN_REF_DISPATCH(p, forward_with_max, x, w, nullptr, B, CO, CI, G, HW, y, p);
    else LDN_REF_DISPATCH(p, forward, x, w, B, CO, CI, G, HW, y, p);
    return (int)cudaGetLastError();
}

int ldn_ref_norm_dist_forward_with_max(const float* x, const float* w, const float* mx, float* y,
                                       int B, int CO, int CI, int G, int HW, float p) {
    LDN_REF_DISPATCH(p, forward_with_max, x, w, mx, B, CO, CI, G, HW, y, p);
    return (int)cudaGetLastError();
}

int ldn_ref_norm_dist_backward_input(const float* go, const float* x, const float* w, const float* y, float* gx,
                                     int B, int CO, int CI, int G, int HW, float p) {
    LDN_REF_DISPATCH(p - 1, backward_input, go, x, w, y, B, CO, CI, G, HW, gx, p);
    return (int)cudaGetLastError();
}

int ldn_ref_norm_dist_backward_input_weight(const float* go, const float* x, const float* w, const float* y,
                                            float* gx, float* gw, int B, int CO, int CI, int G, int HW, float p) {
    LDN_REF_DISPATCH(p - 1, backward_input_weight, go, x, w, y, B, CO, CI, G, HW, gx, gw, p);
    return (int)cudaGetLastError();
}

int ldn_ref_inf_dist_forward(const float* x, const float* w, float* y, int* pos, int B, int CO, int CI, int G, int HW) {
    inf_dist::forward(x, w, B, CO, CI, G, HW, y, pos);
    return (int)cudaGetLastError();
}

int ldn_ref_inf_dist_forward_nograd(const float* x, const float* w, float* y, int B, int CO, int CI, int G, int HW) {
    inf_dist::forward_nograd(x, w, B, CO, CI, G, HW, y);
    return (int)cudaGetLastError();
}

int ldn_ref_inf_dist_backward_input(const float* go, const int* pos, float* gx, int B, int CO, int CI, int G, int HW) {
    inf_dist::backward_input(go, pos, B, CO, CI, G, HW, gx);
    return (int)cudaGetLastError();
}

int ldn_ref_inf_dist_backward_input_weight(const float* go, const int* pos, float* gx, float* gw,
                                           int B, int CO, int CI, int G, int HW) {
    inf_dist::backward_input_weight(go, pos, B, CO, CI, G, HW, gx, gw);
    return (int)cudaGetLastError();
}

int ldn_ref_bound_inf_dist_forward(const float* xL, const float* xU, const float* w, float* yL, float* yU,
                                   int* posL, int* posU, int B, int CO, int CI, int G, int HW) {
    bound_inf_dist::forward(xL, xU, w, B, CO, CI, G, HW, yL, yU, posL, posU);
    return (int)cudaGetLastError();
}

int ldn_ref_bound_inf_dist_forward_nograd(const float* xL, const float* xU, const float* w, float* yL, float* yU,
                                          int B, int CO, int CI, int G, int HW) {
    bound_inf_dist::forward_nograd(xL, xU, w, B, CO, CI, G, HW, yL, yU);
    return (int)cudaGetLastError();
}

int ldn_ref_bound_inf_dist_backward_input(const float* goL, const float* goU, const int* posL, const int* posU,
                                          float* gxL, float* gxU, int B, int CO, int CI, int G, int HW) {
    bound_inf_dist::backward_input(goL, goU, posL, posU, B, CO, CI, G, HW, gxL, gxU);
    return (int)cudaGetLastError();
}

int ldn_ref_bound_inf_dist_backward_input_weight(const float* goL, const float* goU, const int* posL, const int* posU,
                                                 float* gxL, float* gxU, float* gw,
                                                 int B, int CO, int CI, int G, int HW) {
    bound_inf_dist::backward_input_weight(goL, goU, posL, posU, B, CO, CI, G, HW, gxL, gxU, gw);
    return (int)cudaGetLastError();
}

}  // extern "C"
