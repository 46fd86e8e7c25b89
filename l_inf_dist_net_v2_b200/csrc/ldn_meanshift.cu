// Training-mode MeanShift of a fully connected distance layer in one kernel: per-channel batch mean, update of
// the running mean, subtraction.  The reference does this with separate torch operators
// (core/modules/basic_modules.py:104-135: x.mean(dim=[0, 2]), running_mean.mul_(1 - m).add_(mean, alpha = m),
// x - mean); the same kernel without a running mean is its backward pass (grad - mean over the batch of grad).
#include "ldn_b200.h"
#include "ldn_common.cuh"

namespace ldn {
namespace {
constexpr int kCols = 32;      // channels per CTA (one 128-byte row segment per warp-wide load)
constexpr int kRowLanes = 32;  // row groups per CTA (1024 threads: 8 of them took 20 us at 512 x 5120, latency bound)

// x, out: [B][C] row-major.  Thread (lane = channel in the CTA's 32, rl = row group) sums rows rl, rl + 8, ...;
// the 8 partial sums of a channel are folded in shared memory in a fixed order, so the result is deterministic.
__global__ void __launch_bounds__(kCols * kRowLanes)
mean_shift_rows_kernel(const float* __restrict__ x, float* __restrict__ out, float* __restrict__ running_mean,
                       float* __restrict__ mean_out, float momentum, int B, int C) {
    __shared__ float part[kRowLanes][kCols];
    const int lane = threadIdx.x & (kCols - 1);
    const int rl = threadIdx.x / kCols;
    const int col = blockIdx.x * kCols + lane;
    const bool live = col < C;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    if (live) {
        int r = rl;
        for (; r + 3 * kRowLanes < B; r += 4 * kRowLanes) {
            s0 += x[static_cast<size_t>(r) * C + col];
            s1 += x[static_cast<size_t>(r + kRowLanes) * C + col];
            s2 += x[static_cast<size_t>(r + 2 * kRowLanes) * C + col];
            s3 += x[static_cast<size_t>(r + 3 * kRowLanes) * C + col];
        }
        for (; r < B; r += kRowLanes) s0 += x[static_cast<size_t>(r) * C + col];
    }
    part[rl][lane] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    float mean = 0.0f;
#pragma unroll
    for (int q = 0; q < kRowLanes; ++q) mean += part[q][lane];
    mean /= static_cast<float>(B);
    if (!live) return;
    if (rl == 0) {
        if (running_mean) running_mean[col] = running_mean[col] * (1.0f - momentum) + momentum * mean;
        if (mean_out) mean_out[col] = mean;
    }
    for (int r = rl; r < B; r += kRowLanes) {
        const size_t i = static_cast<size_t>(r) * C + col;
        out[i] = x[i] - mean;
    }
}
}  // namespace
}  // namespace ldn

using namespace ldn;

extern "C" LDN_API int ldn_mean_shift_rows(const float* x, int B, int C, float* running_mean, float momentum,
                                           float* out, float* mean_out, ldn_stream_t stream) {
    if (B < 0 || C <= 0) return kBadArgument;
    if (B == 0) return kOk;
    if (!x || !out) return kBadArgument;
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    const unsigned blocks = static_cast<unsigned>((C + kCols - 1) / kCols);
    mean_shift_rows_kernel<<<blocks, kCols * kRowLanes, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, out, running_mean, mean_out, momentum, B, C);
    count_launches(1);
    return cuda_status(cudaGetLastError());
}
