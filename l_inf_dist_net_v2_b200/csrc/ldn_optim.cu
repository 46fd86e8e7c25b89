// Parameter updates as one kernel over a list of tensors (memory-bound: every array is read and written once).
//
// The reference's driver updates ~120 M parameters per step with torch.optim.Adam(betas = (0.9, 0.99),
// eps = 1e-10) (main.py:388-392), which runs as several elementwise passes per tensor list; at p = inf the
// distance kernels of a step take only a few milliseconds, so those passes are a visible share of it.  Here the
// whole update of up to kMaxTensors tensors is one launch: the tensors' chunks are laid out one after the other
// in a virtual index space and every CTA finds its tensor by a short search in the argument block.
#include <math.h>

#include "ldn_b200.h"
#include "ldn_common.cuh"

namespace ldn {
namespace {

constexpr int kMaxTensors = 32;
constexpr int kChunk = 256 * 4 * 8;  // elements per CTA pass: 256 threads x 8 vectors of 4

struct TensorList {
    float* param[kMaxTensors];
    const float* grad[kMaxTensors];
    float* s0[kMaxTensors];   // Adam: exp_avg;    SGD: momentum buffer (or null)
    float* s1[kMaxTensors];   // Adam: exp_avg_sq; SGD: unused
    long long size[kMaxTensors];
    long long first_chunk[kMaxTensors + 1];  // prefix sums of the tensors' chunk counts
    int count;
};

struct AdamArgs {
    float beta1, beta2, eps;
    float step_size;           // lr / (1 - beta1^t)
    float inv_sqrt_bias2;      // 1 / sqrt(1 - beta2^t)
    float grad_scale;
    float lr;
    const float* step_dev;     // not null: t is read from device memory (a launch recorded in a CUDA graph must not
                               // carry the step count as an argument), and the two factors above are derived from it
};

struct SgdArgs {
    float lr, momentum, dampening, weight_decay, grad_scale;
    int nesterov, first;       // first: the momentum buffer is initialised with the gradient (torch's first step)
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamArgs& a) {
    g *= a.grad_scale;
    m = m + (g - m) * (1.0f - a.beta1);                 // lerp, as torch evaluates it
    v = v * a.beta2 + (1.0f - a.beta2) * g * g;
    const float denom = sqrtf(v) * a.inv_sqrt_bias2 + a.eps;
    p = p - a.step_size * (m / denom);
}

__device__ __forceinline__ void sgd_one(float& p, float g, float* m, const SgdArgs& a) {
    g *= a.grad_scale;
    if (a.weight_decay != 0.0f) g = g + a.weight_decay * p;
    if (m) {
        *m = a.first ? g : (*m * a.momentum + (1.0f - a.dampening) * g);
        g = a.nesterov ? g + a.momentum * *m : *m;
    }
    p = p - a.lr * g;
}

template <bool ADAM>
__global__ void __launch_bounds__(256) update_kernel(const __grid_constant__ TensorList L, const AdamArgs aa_in,
                                                     const SgdArgs sa) {
    AdamArgs aa = aa_in;
    if (ADAM && aa.step_dev != nullptr) {
        const float t = *aa.step_dev;
        aa.step_size = aa.lr / (1.0f - powf(aa.beta1, t));
        aa.inv_sqrt_bias2 = rsqrtf(1.0f - powf(aa.beta2, t));
    }
    const long long total_chunks = L.first_chunk[L.count];
    for (long long c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        int t = 0;
        while (t + 1 < L.count && L.first_chunk[t + 1] <= c) ++t;
        const long long base = (c - L.first_chunk[t]) * kChunk;
        const long long n = L.size[t];
        float* p = L.param[t];
        const float* g = L.grad[t];
        float* s0 = L.s0[t];
        float* s1 = L.s1[t];
        const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                           reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(s1)) & 15u) == 0;
        if (vec && base + kChunk <= n) {
#pragma unroll 2
            for (int q = 0; q < kChunk / (256 * 4); ++q) {
                const long long i = base + (static_cast<long long>(q) * 256 + threadIdx.x) * 4;
                float4 pv = *reinterpret_cast<float4*>(p + i);
                const float4 gv = *reinterpret_cast<const float4*>(g + i);
                if (ADAM) {
                    float4 mv = *reinterpret_cast<float4*>(s0 + i);
                    float4 vv = *reinterpret_cast<float4*>(s1 + i);
                    adam_one(pv.x, gv.x, mv.x, vv.x, aa);
                    adam_one(pv.y, gv.y, mv.y, vv.y, aa);
                    adam_one(pv.z, gv.z, mv.z, vv.z, aa);
                    adam_one(pv.w, gv.w, mv.w, vv.w, aa);
                    *reinterpret_cast<float4*>(s0 + i) = mv;
                    *reinterpret_cast<float4*>(s1 + i) = vv;
                } else if (s0) {
                    float4 mv = *reinterpret_cast<float4*>(s0 + i);
                    sgd_one(pv.x, gv.x, &mv.x, sa);
                    sgd_one(pv.y, gv.y, &mv.y, sa);
                    sgd_one(pv.z, gv.z, &mv.z, sa);
                    sgd_one(pv.w, gv.w, &mv.w, sa);
                    *reinterpret_cast<float4*>(s0 + i) = mv;
                } else {
                    sgd_one(pv.x, gv.x, nullptr, sa);
                    sgd_one(pv.y, gv.y, nullptr, sa);
                    sgd_one(pv.z, gv.z, nullptr, sa);
                    sgd_one(pv.w, gv.w, nullptr, sa);
                }
                *reinterpret_cast<float4*>(p + i) = pv;
            }
        } else {
            const long long end = base + kChunk < n ? base + kChunk : n;
            for (long long i = base + threadIdx.x; i < end; i += 256) {
                float pv = p[i];
                if (ADAM) {
                    float mv = s0[i], vv = s1[i];
                    adam_one(pv, g[i], mv, vv, aa);
                    s0[i] = mv;
                    s1[i] = vv;
                } else if (s0) {
                    float mv = s0[i];
                    sgd_one(pv, g[i], &mv, sa);
                    s0[i] = mv;
                } else {
                    sgd_one(pv, g[i], nullptr, sa);
                }
                p[i] = pv;
            }
        }
    }
}

template <bool ADAM>
int run_update(int count, float* const* params, const float* const* grads, float* const* s0, float* const* s1,
               const long long* sizes, const AdamArgs& aa, const SgdArgs& sa, cudaStream_t st) {
    if (count < 0) return kBadArgument;
    if (count > 0 && (!params || !grads || !sizes)) return kBadArgument;
    if (ADAM && count > 0 && (!s0 || !s1)) return kBadArgument;
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    for (int first = 0; first < count; first += kMaxTensors) {
        TensorList L;
        L.count = 0;
        L.first_chunk[0] = 0;
        for (int t = first; t < count && L.count < kMaxTensors; ++t) {
            if (sizes[t] < 0) return kBadArgument;
            if (sizes[t] == 0) continue;
            if (!params[t] || !grads[t] || (ADAM && (!s0[t] || !s1[t]))) return kBadArgument;
            const int k = L.count++;
            L.param[k] = params[t];
            L.grad[k] = grads[t];
            L.s0[k] = s0 ? s0[t] : nullptr;
            L.s1[k] = (ADAM && s1) ? s1[t] : nullptr;
            L.size[k] = sizes[t];
            L.first_chunk[k + 1] = L.first_chunk[k] + (sizes[t] + kChunk - 1) / kChunk;
        }
        if (L.count == 0) continue;
        const long long chunks = L.first_chunk[L.count];
        const long long cap = static_cast<long long>(ctx->sm_count) * 16;
        const unsigned grid = static_cast<unsigned>(chunks < cap ? chunks : cap);
        update_kernel<ADAM><<<grid, 256, 0, st>>>(L, aa, sa);
        count_launches(1);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_status(e);
    }
    return kOk;
}

}  // namespace
}  // namespace ldn

using namespace ldn;

extern "C" {

LDN_API int ldn_adam_update_device_step(int count, float* const* params, const float* const* grads,
                                        float* const* exp_avg, float* const* exp_avg_sq, const long long* sizes, float lr,
                                        float beta1, float beta2, float eps, const float* step_device, float grad_scale,
                                        ldn_stream_t stream) {
    if (!step_device || !(beta1 >= 0.0f && beta1 < 1.0f) || !(beta2 >= 0.0f && beta2 < 1.0f)) return kBadArgument;
    AdamArgs aa;
    aa.beta1 = beta1;
    aa.beta2 = beta2;
    aa.eps = eps;
    aa.step_size = 0.0f;
    aa.inv_sqrt_bias2 = 0.0f;
    aa.grad_scale = grad_scale;
    aa.lr = lr;
    aa.step_dev = step_device;
    return run_update<true>(count, params, grads, exp_avg, exp_avg_sq, sizes, aa, SgdArgs{},
                            reinterpret_cast<cudaStream_t>(stream));
}

LDN_API int ldn_adam_update(int count, float* const* params, const float* const* grads, float* const* exp_avg,
                            float* const* exp_avg_sq, const long long* sizes, float lr, float beta1, float beta2,
                            float eps, int step, float grad_scale, ldn_stream_t stream) {
    if (step < 1 || !(beta1 >= 0.0f && beta1 < 1.0f) || !(beta2 >= 0.0f && beta2 < 1.0f)) return kBadArgument;
    AdamArgs aa;
    aa.beta1 = beta1;
    aa.beta2 = beta2;
    aa.eps = eps;
    aa.step_size = static_cast<float>(lr / (1.0 - pow(static_cast<double>(beta1), step)));
    aa.inv_sqrt_bias2 = static_cast<float>(1.0 / sqrt(1.0 - pow(static_cast<double>(beta2), step)));
    aa.grad_scale = grad_scale;
    aa.lr = lr;
    aa.step_dev = nullptr;
    return run_update<true>(count, params, grads, exp_avg, exp_avg_sq, sizes, aa, SgdArgs{},
                            reinterpret_cast<cudaStream_t>(stream));
}

LDN_API int ldn_sgd_update(int count, float* const* params, const float* const* grads, float* const* momentum_buf,
                           const long long* sizes, float lr, float momentum, float dampening, float weight_decay,
                           int nesterov, int first_step, float grad_scale, ldn_stream_t stream) {
    SgdArgs sa;
    sa.lr = lr;
    sa.momentum = momentum;
    sa.dampening = dampening;
    sa.weight_decay = weight_decay;
    sa.nesterov = nesterov;
    sa.first = first_step;
    sa.grad_scale = grad_scale;
    return run_update<false>(count, params, grads, momentum != 0.0f ? momentum_buf : nullptr, nullptr, sizes, AdamArgs{},
                             sa, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
