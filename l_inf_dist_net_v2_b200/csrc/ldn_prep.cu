#include "ldn_prep.cuh"

namespace ldn {

namespace {
constexpr int kBlock = 256;
constexpr int kRescanInplaceMaxSmem = 200 * 1024;  // input slab of rescan_inplace_kernel
constexpr int kRescanChunk = 1024;  // outputs a block of rescan_kernel handles in one pass (a multiple of kBlock / 8)
// grid of a kernel that usually returns at once (gated): small, the grid-stride loops cover the rest when it runs
inline unsigned gated_blocks(unsigned blocks, const int* gate) { return (gate && blocks > 592u) ? 592u : blocks; }
inline unsigned blocks_for(long long n) {
    long long b = (n + kBlock - 1) / kBlock;
    if (b < 1) b = 1;
    if (b > 1184 * 8) b = 1184 * 8;  // grid-stride beyond this
    return static_cast<unsigned>(b);
}

// index helpers -------------------------------------------------------------------------------
// canonical arrays are [g][m][pitch]; thread index runs over (g, m, c) with c fastest
struct CanonIdx {
    int g, c;
    long long m;
};
__device__ __forceinline__ CanonIdx canon_idx(long long i, int inner, long long M) {
    CanonIdx r;
    r.c = static_cast<int>(i % inner);
    const long long t = i / inner;
    r.m = t % M;
    r.g = static_cast<int>(t / M);
    return r;
}

__global__ void canon_x_kernel(const float* __restrict__ x, float* __restrict__ xc, Shape s, int pitch) {
    const long long total = static_cast<long long>(s.G) * s.M * s.CIg;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const CanonIdx q = canon_idx(i, s.CIg, s.M);
        const long long b = q.m / s.HW, hw = q.m % s.HW;
        xc[(static_cast<long long>(q.g) * s.M + q.m) * pitch + q.c] = x[((b * s.G + q.g) * s.CIg + q.c) * s.HW + hw];
    }
}

__global__ void canon_bounds_kernel(const float* __restrict__ xl, const float* __restrict__ xu, float* __restrict__ lc,
                                    float* __restrict__ uc, Shape s, int pitch) {
    const long long total = static_cast<long long>(s.G) * s.M * s.CIg;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const CanonIdx q = canon_idx(i, s.CIg, s.M);
        const long long b = q.m / s.HW, hw = q.m % s.HW;
        const long long src = ((b * s.G + q.g) * s.CIg + q.c) * s.HW + hw;
        float lo = xl[src], up = xu[src];
        if (lo > up) lo = up = (lo + up) * 0.5f;
        const long long dst = (static_cast<long long>(q.g) * s.M + q.m) * pitch + q.c;
        lc[dst] = lo;
        uc[dst] = up;
    }
}

// HW > 1: tiled transpose through shared memory.  Source rows (b, g, c, :) are contiguous in hw, destination
// rows (g, m = b HW + hw, :) are contiguous in c; a 32 x 32 tile makes both sides coalesced.  grid = (ceil(HW/32),
// ceil(CIg/32), B*G).  With `second` non-null the pair (x, second) is treated as interval bounds and sanitised.
__global__ void canon_transpose_kernel(const float* __restrict__ x, const float* __restrict__ second,
                                       float* __restrict__ xc, float* __restrict__ sc, Shape s, int pitch) {
    __shared__ float t0[32][33], t1[32][33];
    const int bg = blockIdx.z, b = bg / s.G, g = bg % s.G;
    const int hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const float* src = x + (static_cast<long long>(bg) * s.CIg) * s.HW;
    const float* src2 = second ? second + (static_cast<long long>(bg) * s.CIg) * s.HW : nullptr;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int c = c0 + r, hw = hw0 + threadIdx.x;
        if (c < s.CIg && hw < s.HW) {
            float lo = src[static_cast<long long>(c) * s.HW + hw];
            if (src2) {
                float up = src2[static_cast<long long>(c) * s.HW + hw];
                if (lo > up) lo = up = (lo + up) * 0.5f;
                t1[r][threadIdx.x] = up;
            }
            t0[r][threadIdx.x] = lo;
        }
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int hw = hw0 + r, c = c0 + threadIdx.x;
        if (c < s.CIg && hw < s.HW) {
            const long long dst = (static_cast<long long>(g) * s.M + static_cast<long long>(b) * s.HW + hw) * pitch + c;
            xc[dst] = t0[threadIdx.x][r];
            if (src2) sc[dst] = t1[threadIdx.x][r];
        }
    }
}

__global__ void canon_w_kernel(const float* __restrict__ w, float* __restrict__ wc, Shape s, int pitch) {
    const long long total = static_cast<long long>(s.CO) * s.CIg;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / s.CIg;
        const int c = static_cast<int>(i - row * s.CIg);
        wc[row * pitch + c] = w[i];
    }
}

// thread index runs over (g, m, o) with o fastest; source offset in output layout
__device__ __forceinline__ long long y_offset(const Shape& s, const CanonIdx& q) {
    const long long b = q.m / s.HW, hw = q.m % s.HW;
    if (s.co_src != s.CO) return (b * s.co_src + s.co_off + q.c) * s.HW + hw;  // channel range, G == 1
    return ((b * s.G + q.g) * s.COg + q.c) * s.HW + hw;
}

// Range guard of the integer-q coefficient g / y^q: *flag is raised when some y^-q is outside [kRqMin, kRqMax]
// (beyond: y^-q overflows or |t|^q <= y^q goes denormal; below: the coefficient loses its bits).  The caller clears
// the word beforehand; flag may be null (q = 0).
constexpr float kRqMin = 1e-30f, kRqMax = 1e24f;
__device__ __forceinline__ bool rq_unsafe(float rq) { return !(rq >= kRqMin && rq <= kRqMax); }

__global__ void coef_int_kernel(const float* __restrict__ go, const float* __restrict__ y, float* __restrict__ coef,
                                Shape s, int pitch, int iq, int* flag) {
    const long long total = static_cast<long long>(s.G) * s.M * s.COg;
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const CanonIdx q = canon_idx(i, s.COg, s.M);
        const long long src = y_offset(s, q);
        const float r = 1.0f / y[src];
        float rq = 1.0f;
        for (int k = 0; k < iq; ++k) rq *= r;
        bad |= rq_unsafe(rq);
        coef[(static_cast<long long>(q.g) * s.M + q.m) * pitch + q.c] = go[src] * rq;
    }
    if (flag && bad) *flag = 1;
}

// flat fast paths (HW == 1, G == 1, pitch == COg: source and destination have the same element order)
__global__ void coef_int_flat_kernel(const float4* __restrict__ go, const float4* __restrict__ y,
                                     float4* __restrict__ coef, long long n4, int iq, int* flag) {
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 yv = y[i];
        const float4 gv = go[i];
        const float4 r = make_float4(1.0f / yv.x, 1.0f / yv.y, 1.0f / yv.z, 1.0f / yv.w);
        float4 rq = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        for (int k = 0; k < iq; ++k) {
            rq.x *= r.x; rq.y *= r.y; rq.z *= r.z; rq.w *= r.w;
        }
        bad |= rq_unsafe(rq.x) | rq_unsafe(rq.y) | rq_unsafe(rq.z) | rq_unsafe(rq.w);
        coef[i] = make_float4(gv.x * rq.x, gv.y * rq.y, gv.z * rq.z, gv.w * rq.w);
    }
    if (flag && bad) *flag = 1;
}
__global__ void coef_gen_flat_kernel(const float4* __restrict__ go, const float4* __restrict__ y,
                                     float4* __restrict__ rinv, float4* __restrict__ gcp, long long n4, float q, bool fold,
                                     const int* gate) {
    if (gate && *gate == 0) return;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 yv = y[i];
        rinv[i] = fold ? make_float4(-q * log2f(yv.x), -q * log2f(yv.y), -q * log2f(yv.z), -q * log2f(yv.w))
                       : make_float4(1.0f / yv.x, 1.0f / yv.y, 1.0f / yv.z, 1.0f / yv.w);
        gcp[i] = go[i];
    }
}

// The general-p coefficient arrays are padded to whole tiles (rows to a multiple of 128, the inner extent to the
// pitch, a multiple of 32): padding gets the offset -1e30 (folded form) or the factor 0 (1 / y form), which sends
// the power to (almost) zero whatever |t| the zero-filled partner operand produces, and a zero gradient factor.
__global__ void coef_gen_kernel(const float* __restrict__ go, const float* __restrict__ y, float* __restrict__ rinv,
                                float* __restrict__ gcp, Shape s, int pitch, long long rows_pad, float q, bool fold,
                                const int* gate) {
    if (gate && *gate == 0) return;
    const long long total = static_cast<long long>(s.G) * rows_pad * pitch;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const CanonIdx ci = canon_idx(i, pitch, rows_pad);
        float off = fold ? -1e30f : 0.0f, gv = 0.0f;
        if (ci.m < s.M && ci.c < s.COg) {
            const long long src = y_offset(s, ci);
            off = fold ? -q * log2f(y[src]) : 1.0f / y[src];
            gv = go[src];
        }
        rinv[i] = off;
        gcp[i] = gv;
    }
}

// Eight lanes per output element: lane q of a group loads the q-th 16-byte piece of the recorded 32-channel stage of
// each operand row (one full 128-byte line per group and operand: operand views are 16-byte aligned with row
// pitches that are multiples of 4 floats), finds the lowest matching channel among its four, and a minimum over the
// group's lanes keeps the lowest channel of the stage -- the index a strictly-greater scan in ascending order ends with.
// blockIdx.x = (sample, group); blockIdx.y walks that pair's CO/G * HW outputs in chunks, so the index arithmetic
// per output is one division by HW (none for fully connected layers) and, for those, a block keeps rereading one
// input row, which stays in the L1 cache: only the weight pieces come from L2.
template <int mode>
__global__ void rescan_kernel(Operand a0, Operand a1, Operand b, const float* __restrict__ y,
                              int* __restrict__ pos, Shape s, long long a_stride_k) {
    const int kpad = (s.CIg + 3) & ~3;
    const int q = threadIdx.x & 7;
    const int group_in_block = threadIdx.x >> 3;
    const unsigned cohw = static_cast<unsigned>(s.COg) * static_cast<unsigned>(s.HW);  // < 2^31, checked by the launcher
    const long long bg = blockIdx.x;
    const int bi = static_cast<int>(bg / s.G), g = static_cast<int>(bg - static_cast<long long>(bi) * s.G);
    const float* arow = a0.ptr + g * a0.stride_group;
    const float* urow = a1.ptr + g * a1.stride_group;
    const float* brow = b.ptr + g * b.stride_group;
    // (the trip counts are the same for all lanes of a warp: its four groups handle consecutive outputs)
    for (unsigned j0 = blockIdx.y * kRescanChunk; j0 < cohw; j0 += gridDim.y * kRescanChunk)
        for (unsigned step = 0; step < kRescanChunk && j0 + step < cohw; step += kBlock / 8) {
            const unsigned j = j0 + step + group_in_block;
            const bool valid = j < cohw;
            const long long i = bg * cohw + j;
            const int stage = valid ? pos[i] : -1;
            int best = 0x7fffffff;
            if (stage >= 0) {
                const unsigned o = s.HW == 1 ? j : j / static_cast<unsigned>(s.HW);
                const unsigned hw = j - o * s.HW;
                const long long m = static_cast<long long>(bi) * s.HW + hw;
                const int k = stage * 32 + 4 * q;
                if (k < kpad) {
                    float4 av;
                    if (a_stride_k == 1) {
                        av = *reinterpret_cast<const float4*>(arow + m * a0.stride_row + k);
                    } else {
                        // input read in place (channels HW apart, no padding behind the last one)
                        const float* ap = a0.ptr + bg * a0.stride_group + hw * a0.stride_row + k * a_stride_k;
                        av.x = ap[0];
                        av.y = k + 1 < s.CIg ? ap[a_stride_k] : 0.0f;
                        av.z = k + 2 < s.CIg ? ap[2 * a_stride_k] : 0.0f;
                        av.w = k + 3 < s.CIg ? ap[3 * a_stride_k] : 0.0f;
                    }
                    const float4 bv = *reinterpret_cast<const float4*>(brow + o * b.stride_row + k);
                    float4 uv = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (mode != 0) uv = *reinterpret_cast<const float4*>(urow + m * a1.stride_row + k);
                    const float yv = y[i];
                    const float ae[4] = {av.x, av.y, av.z, av.w};
                    const float be[4] = {bv.x, bv.y, bv.z, bv.w};
                    const float ue[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                    for (int e = 3; e >= 0; --e) {
                        bool hit, flag;
                        if (mode == 0) {
                            const float d = ae[e] - be[e];
                            hit = fabsf(d) == yv;
                            flag = d < 0.0f;
                        } else {
                            const float t1 = be[e] - ae[e], t2v = ue[e] - be[e];
                            hit = (mode == 1) ? (fminf(t1, t2v) == -yv) : (fmaxf(t1, t2v) == yv);
                            flag = !(t1 <= t2v);
                        }
                        if (hit && k + e < s.CIg) best = ((k + e) << 1) | (flag ? 1 : 0);
                    }
                }
            }
            best = min(best, __shfl_xor_sync(0xffffffffu, best, 1));
            best = min(best, __shfl_xor_sync(0xffffffffu, best, 2));
            best = min(best, __shfl_xor_sync(0xffffffffu, best, 4));
            if (valid && q == 0) {
                int result = (mode == 1) ? static_cast<int>(0xffffffffu) : 0;
                if (best != 0x7fffffff) result = (best >> 1) | ((best & 1) ? static_cast<int>(0x80000000u) : 0);
                pos[i] = result;
            }
        }
}

// The same search for inputs read in place (x[B, C, HW]: the channels of an output are HW floats apart, so the
// kernel above pulls one 32-byte sector per channel and output from L2).  Here a block owns P neighbouring
// positions of one (sample, group): it copies their CI/G x P input values to shared memory once (rows of P floats,
// coalesced), then every thread scans the 32 channels of its output's stage there; a warp holds P consecutive
// positions of 32 / P outputs, so y / pos are read and written coalesced and the shared-memory reads are
// conflict-free whatever the lanes' stages.  The weight pieces (one 128-byte run per output and stage) come from L1 / L2.
template <int P>
__global__ void __launch_bounds__(kBlock) rescan_inplace_kernel(Operand a0, Operand b, const float* __restrict__ y,
                                                                int* __restrict__ pos, Shape s) {
    extern __shared__ float4 xs4[];
    float* xs = reinterpret_cast<float*>(xs4);  // [CI/G][P]
    constexpr int V = P / 4;
    const long long bg = blockIdx.x;
    const int g = static_cast<int>(bg % s.G);
    const int hw0 = blockIdx.y * P;
    const float* xsrc = a0.ptr + bg * a0.stride_group;
    for (int idx = threadIdx.x; idx < s.CIg * V; idx += kBlock) {
        const int c = idx / V, v = idx - c * V;
        const int hw = hw0 + 4 * v;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (hw < s.HW) val = *reinterpret_cast<const float4*>(xsrc + static_cast<long long>(c) * s.HW + hw);
        xs4[idx] = val;
    }
    __syncthreads();
    const int hl = threadIdx.x % P;
    const int hw = hw0 + hl;
    if (hw >= s.HW) return;
    const int kpad = (s.CIg + 3) & ~3;
    const float* brow = b.ptr + g * b.stride_group;
    const long long base = bg * (static_cast<long long>(s.COg) * s.HW) + hw;
    for (int o = threadIdx.x / P; o < s.COg; o += kBlock / P) {
        const long long i = base + static_cast<long long>(o) * s.HW;
        const int stage = pos[i];
        int result = 0;
        if (stage >= 0) {
            const float yv = y[i];
            const int k0 = stage * 32;
            const float* wr = brow + o * b.stride_row + k0;
            int best = -1;
            bool neg = false;
#pragma unroll
            for (int c4 = 7; c4 >= 0; --c4) {
                const int k = k0 + 4 * c4;
                if (k < kpad) {
                    const float4 wv = *reinterpret_cast<const float4*>(wr + 4 * c4);
                    const float we[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int e = 3; e >= 0; --e) {
                        if (k + e < s.CIg) {
                            const float d = xs[(k + e) * P + hl] - we[e];
                            if (fabsf(d) == yv) {
                                best = k + e;
                                neg = d < 0.0f;
                            }
                        }
                    }
                }
            }
            if (best >= 0) result = best | (neg ? static_cast<int>(0x80000000u) : 0);
        }
        pos[i] = result;
    }
}

template <int P>
int launch_rescan_inplace(Operand a0, Operand b, const float* y, int* pos, const Shape& s, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = s.CIg * P * static_cast<int>(sizeof(float));
    if (dev >= 64 || !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(rescan_inplace_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   kRescanInplaceMaxSmem);
        if (e != cudaSuccess) return cuda_status(e);
        if (dev < 64) configured[dev] = true;
    }
    const dim3 grid(static_cast<unsigned>(static_cast<long long>(s.B) * s.G), static_cast<unsigned>((s.HW + P - 1) / P));
    rescan_inplace_kernel<P><<<grid, kBlock, smem, st>>>(a0, b, y, pos, s);
    count_launches(1);
    return cuda_status(cudaGetLastError());
}

// out[g * rows + r] = max_k |v[g][r][k]|.  Contiguous k: one warp per row; k `stride_k` apart with neighbouring rows
// contiguous (inputs read in place): one thread per row.  clear (may be null): a flag word the first thread resets.
__global__ void row_absmax_kernel(Operand v, long long rows, int inner, int groups, float* __restrict__ out, int* clear) {
    if (clear && blockIdx.x == 0 && threadIdx.x == 0) *clear = 0;
    const int lane = threadIdx.x & 31;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const long long total = rows * groups;
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
        const long long g = i / rows, r = i - g * rows;
        const float* src = v.ptr + g * v.stride_group + r * v.stride_row;
        float m = 0.0f;
        for (int k = lane; k < inner; k += 32) m = fmaxf(m, fabsf(src[k]));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        if (lane == 0) out[i] = m;
    }
}
__global__ void row_absmax_strided_kernel(Operand v, long long rows, int inner, int groups, long long stride_k,
                                          float* __restrict__ out, int* clear) {
    if (clear && blockIdx.x == 0 && threadIdx.x == 0) *clear = 0;
    const long long total = rows * groups;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long g = i / rows, r = i - g * rows;
        const float* src = v.ptr + g * v.stride_group + r * v.stride_row;
        float m = 0.0f;
        for (int k = 0; k < inner; ++k) m = fmaxf(m, fabsf(src[k * stride_k]));
        out[i] = m;
    }
}

// gate (may be null): the kernel runs only if (*gate != 0) == run_if_nonzero
__global__ void side_reduce_kernel(const float* __restrict__ part, float* __restrict__ gw, long long count, int tiles,
                                   bool accumulate, const int* gate, bool run_if_nonzero) {
    if (gate && (*gate != 0) != run_if_nonzero) return;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int t = 0; t < tiles; ++t) s += part[t * count + i];
        gw[i] = accumulate ? gw[i] - s : -s;
    }
}

// One thread per output element, in output-layout order (coalesced reads of go / pos).
__global__ void inf_scatter_kernel(const float* __restrict__ go, const int* __restrict__ pos, float* gx, float* gw,
                                   Shape s) {
    const long long total = static_cast<long long>(s.B) * s.CO * s.HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int hw = static_cast<int>(i % s.HW);
        const long long t = i / s.HW;
        const int o = static_cast<int>(t % s.COg);
        const long long t2 = t / s.COg;
        const int g = static_cast<int>(t2 % s.G);
        const long long b = t2 / s.G;
        const int ps = pos[i];
        const int idx = ps & 0x7fffffff;
        const float v = ps >= 0 ? go[i] : -go[i];
        if (gx) atomicAdd(&gx[((b * s.G + g) * s.CIg + idx) * s.HW + hw], v);
        if (gw) atomicAdd(&gw[(static_cast<long long>(g) * s.COg + o) * s.CIg + idx], -v);
    }
}

__global__ void bound_scatter_kernel(const float* __restrict__ gol, const float* __restrict__ gou,
                                     const int* __restrict__ posl, const int* __restrict__ posu, float* gxl, float* gxu,
                                     float* gw, Shape s) {
    const long long total = static_cast<long long>(s.B) * s.CO * s.HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int hw = static_cast<int>(i % s.HW);
        const long long t = i / s.HW;
        const int o = static_cast<int>(t % s.COg);
        const long long t2 = t / s.COg;
        const int g = static_cast<int>(t2 % s.G);
        const long long b = t2 / s.G;
        const int pl = posl[i], pu = posu[i];
        const int il = pl & 0x7fffffff, iu = pu & 0x7fffffff;
        const float vl = pl >= 0 ? gol[i] : -gol[i];
        const float vu = pu >= 0 ? gou[i] : -gou[i];
        const long long xrow = ((b * s.G + g) * s.CIg) * (long long)s.HW + hw;
        const long long wrow = (static_cast<long long>(g) * s.COg + o) * s.CIg;
        if (pl != static_cast<int>(0xffffffffu)) {
            float* dst = pl >= 0 ? gxl : gxu;
            atomicAdd(&dst[xrow + static_cast<long long>(il) * s.HW], vl);
            if (gw) atomicAdd(&gw[wrow + il], -vl);
        }
        float* dst = pu >= 0 ? gxu : gxl;
        atomicAdd(&dst[xrow + static_cast<long long>(iu) * s.HW], vu);
        if (gw) atomicAdd(&gw[wrow + iu], -vu);
    }
}
}  // namespace

#define LDN_LAUNCH_RET() \
    do {                  \
        count_launches(1); \
        return cuda_status(cudaGetLastError()); \
    } while (0)

static bool transpose_grid(const Shape& s, dim3* grid) {
    const long long bg = static_cast<long long>(s.B) * s.G;
    if (s.HW < 8 || bg > 65535 || (s.CIg + 31) / 32 > 65535) return false;
    *grid = dim3((s.HW + 31) / 32, (s.CIg + 31) / 32, static_cast<unsigned>(bg));
    return true;
}

int launch_canon_x(const float* x, float* xc, const Shape& s, int pitch, cudaStream_t st) {
    dim3 grid;
    if (transpose_grid(s, &grid)) {
        canon_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(x, nullptr, xc, nullptr, s, pitch);
        LDN_LAUNCH_RET();
    }
    canon_x_kernel<<<blocks_for((long long)s.G * s.M * s.CIg), kBlock, 0, st>>>(x, xc, s, pitch);
    LDN_LAUNCH_RET();
}
int launch_canon_bounds(const float* xl, const float* xu, float* lc, float* uc, const Shape& s, int pitch,
                        cudaStream_t st) {
    dim3 grid;
    if (transpose_grid(s, &grid)) {
        canon_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(xl, xu, lc, uc, s, pitch);
        LDN_LAUNCH_RET();
    }
    canon_bounds_kernel<<<blocks_for((long long)s.G * s.M * s.CIg), kBlock, 0, st>>>(xl, xu, lc, uc, s, pitch);
    LDN_LAUNCH_RET();
}
int launch_canon_w(const float* w, float* wc, const Shape& s, int pitch, cudaStream_t st) {
    canon_w_kernel<<<blocks_for((long long)s.CO * s.CIg), kBlock, 0, st>>>(w, wc, s, pitch);
    LDN_LAUNCH_RET();
}
static bool flat_ok(const Shape& s, int pitch, const void* a, const void* b) {
    return s.HW == 1 && s.G == 1 && s.co_src == s.CO && pitch == s.COg && (s.COg & 3) == 0 &&
           ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

int launch_coef_int(const float* go, const float* y, float* coef, const Shape& s, int pitch, int iq, int* flag,
                    cudaStream_t st) {
    if (flat_ok(s, pitch, go, y)) {
        const long long n4 = static_cast<long long>(s.M) * s.COg / 4;
        coef_int_flat_kernel<<<blocks_for(n4), kBlock, 0, st>>>(reinterpret_cast<const float4*>(go),
                                                              reinterpret_cast<const float4*>(y),
                                                              reinterpret_cast<float4*>(coef), n4, iq, flag);
        LDN_LAUNCH_RET();
    }
    coef_int_kernel<<<blocks_for((long long)s.G * s.M * s.COg), kBlock, 0, st>>>(go, y, coef, s, pitch, iq, flag);
    LDN_LAUNCH_RET();
}
int launch_coef_gen(const float* go, const float* y, float* rinv, float* gcp, const Shape& s, int pitch,
                    long long rows_pad, float q, bool fold, const int* gate, cudaStream_t st) {
    if (flat_ok(s, pitch, go, y) && rows_pad == s.M) {
        const long long n4 = static_cast<long long>(s.M) * s.COg / 4;
        coef_gen_flat_kernel<<<gated_blocks(blocks_for(n4), gate), kBlock, 0, st>>>(reinterpret_cast<const float4*>(go),
                                                              reinterpret_cast<const float4*>(y),
                                                              reinterpret_cast<float4*>(rinv),
                                                              reinterpret_cast<float4*>(gcp), n4, q, fold, gate);
        LDN_LAUNCH_RET();
    }
    coef_gen_kernel<<<gated_blocks(blocks_for((long long)s.G * rows_pad * pitch), gate), kBlock, 0, st>>>(
        go, y, rinv, gcp, s, pitch, rows_pad, q, fold, gate);
    LDN_LAUNCH_RET();
}

int launch_rescan(int mode, Operand a0, Operand a1, Operand b, const float* y, int* pos, const Shape& s,
                  cudaStream_t st, long long a_stride_k) {
    if (a_stride_k != 1 && mode != 0) return kBadArgument;
    const long long cohw = static_cast<long long>(s.COg) * s.HW;
    const long long bg = static_cast<long long>(s.B) * s.G;
    if (cohw > 0x7fffffffLL || bg > 0x7fffffffLL) return kBadArgument;
    if (mode == 0 && a_stride_k != 1 && a_stride_k == s.HW && a0.stride_row == 1 && (s.HW & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(a0.ptr) & 15u) == 0 && (s.HW + 7) / 8 <= 65535) {
        // inputs read in place: the largest slab of positions that leaves room for two blocks per SM, else the
        // largest that fits at all; beyond that (CI/G > 6400) the general kernel
        const long long row = static_cast<long long>(s.CIg) * sizeof(float);
        for (int pass = 0; pass < 2; ++pass) {
            const long long limit = pass == 0 ? 96 * 1024 : kRescanInplaceMaxSmem;
            if (row * 32 <= limit) return launch_rescan_inplace<32>(a0, b, y, pos, s, st);
            if (row * 16 <= limit) return launch_rescan_inplace<16>(a0, b, y, pos, s, st);
            if (row * 8 <= limit) return launch_rescan_inplace<8>(a0, b, y, pos, s, st);
        }
    }
    long long chunks = (cohw + kRescanChunk - 1) / kRescanChunk;
    if (chunks > 65535) chunks = 65535;  // the kernel strides over the rest
    const dim3 grid(static_cast<unsigned>(bg), static_cast<unsigned>(chunks));
    if (mode == 0) rescan_kernel<0><<<grid, kBlock, 0, st>>>(a0, a1, b, y, pos, s, a_stride_k);
    else if (mode == 1) rescan_kernel<1><<<grid, kBlock, 0, st>>>(a0, a1, b, y, pos, s, a_stride_k);
    else rescan_kernel<2><<<grid, kBlock, 0, st>>>(a0, a1, b, y, pos, s, a_stride_k);
    LDN_LAUNCH_RET();
}

int launch_row_absmax(Operand v, long long rows, int inner, int groups, long long stride_k, float* out, int* clear,
                      cudaStream_t st) {
    if (stride_k == 1)
        row_absmax_kernel<<<blocks_for(rows * groups * 32), kBlock, 0, st>>>(v, rows, inner, groups, out, clear);
    else
        row_absmax_strided_kernel<<<blocks_for(rows * groups), kBlock, 0, st>>>(v, rows, inner, groups, stride_k, out,
                                                                               clear);
    LDN_LAUNCH_RET();
}

int launch_side_reduce(const float* part, float* gw, long long count, int tiles, bool accumulate, const int* gate,
                       bool run_if_nonzero, cudaStream_t st) {
    side_reduce_kernel<<<gated_blocks(blocks_for(count), run_if_nonzero ? gate : nullptr), kBlock, 0, st>>>(
        part, gw, count, tiles, accumulate, gate, run_if_nonzero);
    LDN_LAUNCH_RET();
}

int launch_inf_scatter(const float* go, const int* pos, float* gx, float* gw, const Shape& s, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    if (gx) e = cudaMemsetAsync(gx, 0, sizeof(float) * (size_t)s.B * s.CI * s.HW, st);
    if (e == cudaSuccess && gw) e = cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)s.CO * s.CIg, st);
    if (e != cudaSuccess) return cuda_status(e);
    inf_scatter_kernel<<<blocks_for((long long)s.B * s.CO * s.HW), kBlock, 0, st>>>(go, pos, gx, gw, s);
    LDN_LAUNCH_RET();
}

int launch_bound_scatter(const float* gol, const float* gou, const int* posl, const int* posu, float* gxl, float* gxu,
                         float* gw, const Shape& s, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(gxl, 0, sizeof(float) * (size_t)s.B * s.CI * s.HW, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(gxu, 0, sizeof(float) * (size_t)s.B * s.CI * s.HW, st);
    if (e == cudaSuccess && gw) e = cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)s.CO * s.CIg, st);
    if (e != cudaSuccess) return cuda_status(e);
    bound_scatter_kernel<<<blocks_for((long long)s.B * s.CO * s.HW), kBlock, 0, st>>>(gol, gou, posl, posu, gxl, gxu,
                                                                                     gw, s);
    LDN_LAUNCH_RET();
}

}  // namespace ldn
