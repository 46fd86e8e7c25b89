// Diagnostics exported next to the operators: a host-side count of kernel launches and two
// pipe-throughput probes (dependent-chain-free FFMA and MUFU loops) that give the measured
// denominators for the compute rooflines.
#include <atomic>

#include "ldn_b200.h"
#include "ldn_common.cuh"
#include "ldn_ops.cuh"

namespace ldn {
std::atomic<unsigned long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

unsigned long long* g_trace = nullptr;
unsigned long long* trace_buffer() { return g_trace; }

// Event pair around the latest tile-kernel launch, for per-kernel roofline numbers.
bool g_timing = false;
cudaEvent_t g_ev0 = nullptr, g_ev1 = nullptr;
void timing_before(cudaStream_t st) {
    if (!g_timing) return;
    if (!g_ev0) {
        cudaEventCreate(&g_ev0);
        cudaEventCreate(&g_ev1);
    }
    cudaEventRecord(g_ev0, st);
}
void timing_after(cudaStream_t st) {
    if (g_timing && g_ev1) cudaEventRecord(g_ev1, st);
}

namespace {
constexpr int kProbeThreads = 256;
constexpr int kProbeIlp = 16;

// kind 0: 16 independent FFMA chains per thread.  kind 1: 16 independent ex2(lg2(x)) chains (2 MUFU each).
// kind 2: the FFMA chains issued as 8 packed fma.rn.f32x2 instructions.
template <int KIND>
__global__ void __launch_bounds__(kProbeThreads) probe_kernel(int iters, float seed, float* sink) {
    float v[kProbeIlp];
#pragma unroll
    for (int i = 0; i < kProbeIlp; ++i) v[i] = seed + 0.001f * (threadIdx.x + i);
    const float a = 0.999f, b = 0.0005f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < kProbeIlp; ++i) {
            if (KIND == 0) {
                v[i] = fmaf(v[i], a, b);
            } else if (KIND == 3) {
                // mixed: chains 0..7 are MUFU (lg2 then ex2), chains 8..15 each run 8 packed FMAs per step
                if (i < 8) {
                    float l, e;
                    asm volatile("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(v[i]));
                    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(l));
                    v[i] = e;
                } else if ((i & 1) == 0) {
                    float2 r = make_float2(v[i], v[i + 1]);
#pragma unroll
                    for (int q = 0; q < 16; ++q) r = __ffma2_rn(r, make_float2(a, a), make_float2(b, b));
                    v[i] = r.x;
                    v[i + 1] = r.y;
                }
            } else if (KIND == 2) {
                // packed FP32: one instruction, two lane operations; chains pair up (i, i ^ 1)
                if ((i & 1) == 0) {
                    const float2 r = __ffma2_rn(make_float2(v[i], v[i + 1]), make_float2(a, a), make_float2(b, b));
                    v[i] = r.x;
                    v[i + 1] = r.y;
                }
            } else {
                float l, e;
                asm volatile("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(v[i]));
                asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(l));
                v[i] = e;
            }
        }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < kProbeIlp; ++i) s += v[i];
    if (s == 12345.678f) sink[0] = s;  // keeps the loop alive, practically never true
}

// kinds 4 / 5: the per-pair instruction stream of the general-p kernels on register operands only (no shared
// memory, 8 independent packed chains per thread, 4 CTAs per SM): what the MUFU + FMA-pipe mix can sustain.
// BWD: t = x - w, 2^(q lg2|t| + c) with every second exponential on MUFU, sign copy, two accumulations
// (BwdFusedGen).  Forward: 2^(p lg2|t| + c) with one exponential in eight on MUFU, one accumulation
// (FwdPowNorm).  Every chain step is two pairs.
constexpr int kMixIlp = 8;
template <bool BWD>
__global__ void __launch_bounds__(kProbeThreads, 4) mix_probe_kernel(int iters, float q, float* sink) {
    float2 x[kMixIlp], acc[kMixIlp], col[kMixIlp];
    const float w0 = 0.3f + threadIdx.x * 1e-4f, off = -0.01f, g = 0.7f;
#pragma unroll
    for (int i = 0; i < kMixIlp; ++i) {
        x[i] = make_float2(0.1f * i + threadIdx.x * 1e-3f, 0.2f * i + 0.05f);
        acc[i] = make_float2(0.0f, 0.0f);
        col[i] = make_float2(0.0f, 0.0f);
    }
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < kMixIlp; ++i) {
            x[i] = __fadd2_rn(x[i], make_float2(1e-4f, 1e-4f));  // keeps the chain from being hoisted
            if (BWD) {
                const float2 t = pk_sub(x[i], make_float2(w0, w0));
                const float2 l = make_float2(lg2_approx(fabsf(t.x)), lg2_approx(fabsf(t.y)));
                const float2 v = ex2_mixed2<4, kMufuEveryBwd>(__ffma2_rn(make_float2(q, q), l, make_float2(off, off)), i);
                const float2 sv = make_float2(copysignf(v.x, t.x), copysignf(v.y, t.y));
                acc[i] = __ffma2_rn(sv, make_float2(g, g), acc[i]);
                col[i] = __ffma2_rn(sv, make_float2(g, g), col[i]);
            } else {
                const float2 l = make_float2(lg2_approx(fabsf(x[i].x - w0)), lg2_approx(fabsf(x[i].y - w0)));
                acc[i] = __fadd2_rn(acc[i], ex2_mixed2<4, kMufuEveryFwd>(
                                                 __ffma2_rn(make_float2(q, q), l, make_float2(off, off)), i));
            }
        }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < kMixIlp; ++i) s += acc[i].x + acc[i].y + col[i].x + col[i].y;
    if (s == 12345.678f) sink[0] = s;
}
}  // namespace
}  // namespace ldn

using namespace ldn;

extern "C" {

LDN_API void ldn_set_trace_buffer(unsigned long long* device_buffer) { g_trace = device_buffer; }

LDN_API void ldn_enable_kernel_timing(int enabled) { g_timing = enabled != 0; }

LDN_API float ldn_last_tile_kernel_ms(void) {
    if (!g_ev0 || !g_ev1) return -1.0f;
    if (cudaEventSynchronize(g_ev1) != cudaSuccess) return -1.0f;
    float ms = -1.0f;
    if (cudaEventElapsedTime(&ms, g_ev0, g_ev1) != cudaSuccess) return -1.0f;
    return ms;
}

LDN_API unsigned long long ldn_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

LDN_API int ldn_probe_pipe(int kind, int iters, float* sink, unsigned long long* lane_ops, ldn_stream_t stream) {
    if (!sink || !lane_ops || iters <= 0 || (kind < 0 || kind > 5)) return kBadArgument;
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    const int blocks = ctx->sm_count * 8;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (kind >= 4) {
        if (kind == 4) mix_probe_kernel<true><<<blocks, kProbeThreads, 0, st>>>(iters, 36.5f, sink);
        else mix_probe_kernel<false><<<blocks, kProbeThreads, 0, st>>>(iters, 37.5f, sink);
        *lane_ops = static_cast<unsigned long long>(blocks) * kProbeThreads * iters * (2ull * kMixIlp);  // pairs
        count_launches(1);
        return cuda_status(cudaGetLastError());
    }
    if (kind == 0) probe_kernel<0><<<blocks, kProbeThreads, 0, st>>>(iters, 1.0f, sink);
    else if (kind == 2) probe_kernel<2><<<blocks, kProbeThreads, 0, st>>>(iters, 1.0f, sink);
    else if (kind == 3) probe_kernel<3><<<blocks, kProbeThreads, 0, st>>>(iters, 1.5f, sink);
    else probe_kernel<1><<<blocks, kProbeThreads, 0, st>>>(iters, 1.5f, sink);
    // kinds 0 and 2: one FMA lane operation per chain step; kind 1: two MUFU operations per chain step;
    // kind 3: 8 of the 16 chains are MUFU chains (two operations per step), only those are counted
    const unsigned long long per_step = kind == 1 ? 2ull * kProbeIlp : (kind == 3 ? 16ull : 1ull * kProbeIlp);
    *lane_ops = static_cast<unsigned long long>(blocks) * kProbeThreads * iters * per_step;
    count_launches(1);
    return cuda_status(cudaGetLastError());
}

}  // extern "C"
