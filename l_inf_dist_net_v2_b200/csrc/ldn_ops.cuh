// Per-pair arithmetic of every kernel family, as policy classes for the tile engine (ldn_tile.cuh).
//
// Every op is written so that zero-filled operand elements (TMA out-of-range fill) are neutral:
// |0 - 0|^p = 0 for p > 0, |0 - 0| never exceeds the 1e-10 floor, and backward coefficients of padded
// entries are zero.
#pragma once
#include <float.h>
#include "ldn_tile.cuh"

namespace ldn {

constexpr float kEps = 1e-10f;                  // value floor of the p = inf family and of the p > 10 sum
constexpr float kUnderflow = 1.175494351e-38f;  // floor of the p <= 10 sum before the root
constexpr int kSignBit = static_cast<int>(0x80000000u);
constexpr int kNoGrad = static_cast<int>(0xffffffffu);

__device__ __forceinline__ float lg2_approx(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// 2^e on the FMA pipe: round e to the nearest integer n with the 1.5 * 2^23 trick, evaluate a minimax
// polynomial of 2^f on f = e - n in [-0.5, 0.5] and add n to the exponent field.  Maximum relative
// error 7.5e-5 (DEG 3) / 2.7e-6 (DEG 4).  e is clamped at -125 (the result is then ~2e-38 instead of 0);
// e must stay below 126.
template <int DEG>
__device__ __forceinline__ float ex2_fma(float e) {
    static_assert(DEG == 3 || DEG == 4, "supported polynomial degrees");
    e = fmaxf(e, -125.0f);
    const float magic = 12582912.0f;
    const float z = e + magic;
    const float f = e - (z - magic);
    float pl;
    if (DEG == 3) {
        pl = fmaf(0.05517162010073662f, f, 0.2426111251115799f);
        pl = fmaf(pl, f, 0.6932609677314758f);
        pl = fmaf(pl, f, 0.9999280571937561f);
    } else {
        pl = fmaf(0.009570096619427204f, f, 0.05591785907745361f);
        pl = fmaf(pl, f, 0.240247443318367f);
        pl = fmaf(pl, f, 0.6931217908859253f);
        pl = fmaf(pl, f, 0.9999992847442627f);
    }
    return __int_as_float(__float_as_int(pl) + (__float_as_int(z) << 23));
}

// The general-p kernels need two transcendentals per pair and are bound by the MUFU pipe (16 lanes per SM
// against 128 FP32 lanes).  The logarithm stays on MUFU; the exponential goes to MUFU for one pair in
// kMufuEvery and to the FMA-pipe polynomial for the others, which balances the two pipes.  `sel` is a
// compile-time constant after unrolling (output slot + k).
constexpr int kMufuEvery = 4;
template <int DEG>
__device__ __forceinline__ float ex2_mixed(float e, int sel) {
    return (sel % kMufuEvery) == 0 ? ex2_approx(e) : ex2_fma<DEG>(e);
}

// Two-lane versions (packed FP32 instructions for the range reduction and the polynomial).  In the packed
// kernels the exponential goes to MUFU for one output pair in EVERY.
template <int DEG>
__device__ __forceinline__ float2 ex2_fma2(float2 e) {
    static_assert(DEG == 3 || DEG == 4, "supported polynomial degrees");
    e.x = fmaxf(e.x, -125.0f);
    e.y = fmaxf(e.y, -125.0f);
    const float2 z = __fadd2_rn(e, make_float2(12582912.0f, 12582912.0f));
    const float2 r = __fadd2_rn(z, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = __ffma2_rn(r, make_float2(-1.0f, -1.0f), e);
    float2 pl;
    if (DEG == 3) {
        pl = __ffma2_rn(make_float2(0.05517162010073662f, 0.05517162010073662f), f,
                        make_float2(0.2426111251115799f, 0.2426111251115799f));
        pl = __ffma2_rn(pl, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
        pl = __ffma2_rn(pl, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
    } else {
        pl = __ffma2_rn(make_float2(0.009570096619427204f, 0.009570096619427204f), f,
                        make_float2(0.05591785907745361f, 0.05591785907745361f));
        pl = __ffma2_rn(pl, f, make_float2(0.240247443318367f, 0.240247443318367f));
        pl = __ffma2_rn(pl, f, make_float2(0.6931217908859253f, 0.6931217908859253f));
        pl = __ffma2_rn(pl, f, make_float2(0.9999992847442627f, 0.9999992847442627f));
    }
    return make_float2(__int_as_float(__float_as_int(pl.x) + (__float_as_int(z.x) << 23)),
                       __int_as_float(__float_as_int(pl.y) + (__float_as_int(z.y) << 23)));
}
template <int DEG, int EVERY>
__device__ __forceinline__ float2 ex2_mixed2(float2 e, int sel) {
    if ((sel % EVERY) == 0) return make_float2(ex2_approx(e.x), ex2_approx(e.y));
    return ex2_fma2<DEG>(e);
}
// measured best on B200 (degree-4 polynomial in both): the forward sends one exponential in 3 to MUFU (3.23 ms
// for the sum pass of 512 x 3072 -> 5120 against 3.27 / 3.31 / 3.43 with one in 4 / 6 / 8), the backward, with two
// accumulations per term, every second one.  (A degree-3 polynomial in the forward was 9 % faster but left the
// output 2e-6 off, which the backward multiplies by p - 1: the gradients then missed 1e-4 on small problems.)
constexpr int kMufuEveryFwd = 3;
constexpr int kMufuEveryBwd = 2;

// |t|^IP by repeated multiplication, IP in 1..8
template <int IP>
__device__ __forceinline__ float abs_pow(float t) {
    static_assert(IP >= 1 && IP <= 8, "integer power out of range");
    const float a = fabsf(t);
    if (IP == 1) return a;
    const float t2 = t * t;
    if (IP == 2) return t2;
    if (IP == 3) return t2 * a;
    const float t4 = t2 * t2;
    if (IP == 4) return t4;
    if (IP == 5) return t4 * a;
    if (IP == 6) return t4 * t2;
    if (IP == 7) return t4 * (t2 * a);
    return t4 * t4;
}

// acc + |t|^IP with the last multiply fused into the accumulation
template <int IP>
__device__ __forceinline__ float acc_abs_pow(float acc, float t) {
    const float a = fabsf(t);
    if (IP == 1) return acc + a;
    if (IP == 2) return fmaf(t, t, acc);
    const float t2 = t * t;
    if (IP == 3) return fmaf(t2, a, acc);
    if (IP == 4) return fmaf(t2, t2, acc);
    const float t4 = t2 * t2;
    if (IP == 5) return fmaf(t4, a, acc);
    if (IP == 6) return fmaf(t4, t2, acc);
    if (IP == 7) return fmaf(t4, t2 * a, acc);
    return fmaf(t4, t4, acc);
}

// sgn(t) |t|^IQ with sgn(t) = +1 for t >= 0 (IQ in 0..8); used by the backward kernels
template <int IQ>
__device__ __forceinline__ float signed_pow(float t) {
    static_assert(IQ >= 0 && IQ <= 8, "integer power out of range");
    if (IQ == 0) return t >= 0.0f ? 1.0f : -1.0f;
    if (IQ == 1) return t;
    const float u = t * fabsf(t);  // sgn(t) t^2
    if (IQ == 2) return u;
    const float t2 = t * t;
    if (IQ == 3) return t2 * t;
    if (IQ == 4) return t2 * u;
    const float t4 = t2 * t2;
    if (IQ == 5) return t4 * t;
    if (IQ == 6) return t4 * u;
    if (IQ == 7) return t4 * (t2 * t);
    return (t4 * t2) * u;
}

// ---- packed two-lane FP32 (sm_100 fma/mul/add .f32x2): one issue slot, two lane operations ---------
__device__ __forceinline__ float2 pk(float x, float y) { return make_float2(x, y); }
__device__ __forceinline__ float2 pk_abs(float2 t) { return make_float2(fabsf(t.x), fabsf(t.y)); }
// x - y
__device__ __forceinline__ float2 pk_sub(float2 x, float2 y) { return __ffma2_rn(y, make_float2(-1.0f, -1.0f), x); }

// acc + |t|^IP on two lanes
template <int IP>
__device__ __forceinline__ float2 acc_abs_pow2(float2 acc, float2 t) {
    if (IP == 1) return __fadd2_rn(acc, pk_abs(t));
    if (IP == 2) return __ffma2_rn(t, t, acc);
    const float2 t2 = __fmul2_rn(t, t);
    if (IP == 3) return __ffma2_rn(t2, pk_abs(t), acc);
    if (IP == 4) return __ffma2_rn(t2, t2, acc);
    const float2 t4 = __fmul2_rn(t2, t2);
    if (IP == 5) return __ffma2_rn(t4, pk_abs(t), acc);
    if (IP == 6) return __ffma2_rn(t4, t2, acc);
    if (IP == 7) return __ffma2_rn(t4, __fmul2_rn(t2, pk_abs(t)), acc);
    return __ffma2_rn(t4, t4, acc);
}

// sgn(t) |t|^IQ on two lanes, IQ in 1..8 (sgn(t) = +1 for t >= 0; IQ = 0 is handled by the scalar path)
template <int IQ>
__device__ __forceinline__ float2 signed_pow2(float2 t) {
    if (IQ == 1) return t;
    if (IQ == 2) return __fmul2_rn(t, pk_abs(t));
    const float2 t2 = __fmul2_rn(t, t);
    if (IQ == 3) return __fmul2_rn(t2, t);
    if (IQ == 4) return __fmul2_rn(t2, __fmul2_rn(t, pk_abs(t)));
    const float2 t4 = __fmul2_rn(t2, t2);
    if (IQ == 5) return __fmul2_rn(t4, t);
    if (IQ == 6) return __fmul2_rn(t4, __fmul2_rn(t, pk_abs(t)));
    if (IQ == 7) return __fmul2_rn(t4, __fmul2_rn(t2, t));
    return __fmul2_rn(__fmul2_rn(t4, t2), __fmul2_rn(t, pk_abs(t)));
}

struct FwdLayout {
    static constexpr Layout LA = Layout::RowMajor;
    static constexpr Layout LB = Layout::RowMajor;
    static constexpr int KSTEP = 2;  // k values per rolled inner-loop step
    static constexpr bool PACKED = false;
    static constexpr bool PREFETCH = true;  // register double buffering of the operand slabs
    static constexpr bool FUSED_W = false;
    static constexpr bool STAGE_HOOK = false;  // op has a stage_end(f, n, stage) step after every 32-wide stage
    static constexpr bool SHORT_STAGES = false;  // stop a partly filled last stage after its valid k-groups
    static constexpr int UNROLL = 1;             // unroll factor of the rolled k-group loop (measured per op)
    static constexpr bool N_IN_SMEM = false;     // integer accumulators live in shared memory, not registers
    static constexpr bool ROLLED_EPILOGUE = true;  // finalise a tile row by row in a rolled loop (small code)
    static constexpr bool ROLLED_PRES = true;      // the same for loading the resident per-output operand
    static constexpr int STAGES = kStages;
    static constexpr int REG_N = 8;        // output columns per thread: 8 (128 x 128 tile) or 4 (128 x 64)
    static constexpr int CTAS_PER_SM = 1;  // 2 needs REG_N = 4 (registers) and at most 113 KB of shared memory
};

// A forward op with another A layout and / or a narrower tile: LA_ = KMajor reads convolution-shaped inputs
// x[B, C, HW] in place (HW contiguous: tiles of [32 channels][128 positions], every sample its own engine group);
// RN_ = 4 / 2 are the 128 x 64 / 128 x 32 tiles for layers with few outputs per group.
template <class Base, Layout LA_, int RN_>
struct FwdVariant : Base {
    static constexpr Layout LA = LA_;
    static constexpr int REG_N = RN_;
    static constexpr int CTAS_PER_SM = 1;
};

// ------------------------------------------------------------------------------------------------
// Finite p, forward
// ------------------------------------------------------------------------------------------------

// sum of |t|^IP, then the p-th root with the underflow floor
template <int IP>
struct FwdPowInt : FwdLayout {
    static constexpr int UNROLL = 2;  // measured best: 4-wide k-groups, two per trip, no register double buffering
    static constexpr int KSTEP = 4;
    static constexpr bool PREFETCH = false;
    static constexpr int NUM_A = 1, NF = 1, NI = 0;
    static constexpr bool HAS_P = false;
    static constexpr bool PACKED = true;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    template <int KS>
    __device__ static void update_pair(float& s0, float& s1, float, float, const float* a, const float*,
                                       const float* b0, const float* b1, int, const TileParams&) {
        float2 acc = pk(s0, s1);
#pragma unroll
        for (int k = 0; k < KS; ++k) acc = acc_abs_pow2<IP>(acc, pk(a[k] - b0[k], a[k] - b1[k]));
        s0 = acc.x;
        s1 = acc.y;
    }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* a, const float*, const float* b, int, int,
                                   const TileParams&) {
#pragma unroll
        for (int k = 0; k < KS; ++k) f[0] = acc_abs_pow<IP>(f[0], a[k] - b[k]);
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        P.out_f0[out_offset(P.out, m, n, g)] = powf(fmaxf(f[0], kUnderflow), 1.0f / P.p);
    }
};

// sum of |t|^p = 2^(p lg2 |t|) for non-integer (or > 8) p <= 10
struct FwdPowGen : FwdLayout {
    static constexpr bool SHORT_STAGES = true;
    static constexpr int NUM_A = 1, NF = 1, NI = 0;
    static constexpr bool HAS_P = false;
    static constexpr bool PACKED = true;
    static constexpr bool PREFETCH = false;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    template <int KS>
    __device__ static void update_pair(float& s0, float& s1, float, float, const float* a, const float*,
                                       const float* b0, const float* b1, int sel, const TileParams& P) {
        float2 acc = make_float2(s0, s1);
        const float2 pp = make_float2(P.p, P.p);
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float2 l = make_float2(lg2_approx(fabsf(a[k] - b0[k])), lg2_approx(fabsf(a[k] - b1[k])));
            acc = __fadd2_rn(acc, ex2_mixed2<4, kMufuEveryFwd>(__fmul2_rn(pp, l), sel + k));
        }
        s0 = acc.x;
        s1 = acc.y;
    }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* a, const float*, const float* b, int, int sel,
                                   const TileParams& P) {
#pragma unroll
        for (int k = 0; k < KS; ++k) f[0] += ex2_mixed<4>(P.p * lg2_approx(fabsf(a[k] - b[k])), sel + k);
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        P.out_f0[out_offset(P.out, m, n, g)] = powf(fmaxf(f[0], kUnderflow), 1.0f / P.p);
    }
};

// sum of (|t| / M)^p with a per-output normaliser M; resident value = -p lg2 M;  y = M (sum + (1e-10 / M)^p)^(1/p).
// The value of y does not depend on M (it cancels), only the fp32 range of the terms does.  M is either read from
// P.pres (layout of the output: the exact maximum of |t|, or the caller's array), or -- P.norm_rows set -- the
// separable upper bound max_c |x| + max_c |w| of that maximum, which costs two small row reductions instead of a
// full max pass; a sum below kNormGuard then means the bound was too loose for this output's terms to stay well
// inside the fp32 range, and the kernel raises P.guard (the caller recomputes with the exact maximum).
constexpr float kNormGuard = 1e-27f;
__device__ __forceinline__ float pow_norm_of(const TileParams& P, int m, int n, int g, long long off) {
    if (P.norm_rows == nullptr) return P.pres.ptr[off];
    const int gb = P.b_group_mod > 0 ? g % P.b_group_mod : g;
    return fmaxf(P.norm_rows[static_cast<long long>(g) * P.M + m] + P.norm_cols[static_cast<long long>(gb) * P.N + n], kEps);
}

struct FwdPowNorm : FwdLayout {
    static constexpr bool SHORT_STAGES = true;
    static constexpr int NUM_A = 1, NF = 1, NI = 0;
    static constexpr bool HAS_P = true;
    static constexpr bool PACKED = true;
    static constexpr bool PREFETCH = false;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    template <int KS>
    __device__ static void update_pair(float& s0, float& s1, float cm0, float cm1, const float* a, const float*,
                                       const float* b0, const float* b1, int sel, const TileParams& P) {
        float2 acc = make_float2(s0, s1);
        const float2 pp = make_float2(P.p, P.p);
        const float2 cm = make_float2(cm0, cm1);
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float2 l = make_float2(lg2_approx(fabsf(a[k] - b0[k])), lg2_approx(fabsf(a[k] - b1[k])));
            acc = __fadd2_rn(acc, ex2_mixed2<4, kMufuEveryFwd>(__ffma2_rn(pp, l, cm), sel + k));
        }
        s0 = acc.x;
        s1 = acc.y;
    }
    template <int KS>
    __device__ static void update(float* f, int*, float cm, const float* a, const float*, const float* b, int, int sel,
                                   const TileParams& P) {
#pragma unroll
        for (int k = 0; k < KS; ++k) f[0] += ex2_mixed<4>(fmaf(P.p, lg2_approx(fabsf(a[k] - b[k])), cm), sel + k);
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static float load_pres(const TileParams& P, int m, int n, int g) {
        return -P.p * log2f(pow_norm_of(P, m, n, g, out_offset(P.out, m, n, g)));
    }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        const long long off = out_offset(P.out, m, n, g);
        const float M = pow_norm_of(P, m, n, g, off);
        if (P.guard != nullptr && !(f[0] >= kNormGuard)) *P.guard = 1;
        const float s = f[0] + exp2f(P.p * (log2f(kEps) - log2f(M)));
        P.out_f0[off] = M * powf(s, 1.0f / P.p);
    }
};

// ------------------------------------------------------------------------------------------------
// p = inf, forward.  The running maximum is exact whatever the evaluation order.  With POS the kernel
// also records in which 32-channel stage the maximum first strictly increased to its final value (one
// compare per output per stage, the inner loop stays the plain maximum) and stores that stage id in the
// index array; rescan_kernel (ldn_prep.cu, one thread per output) then finds the
// first channel equal to the maximum, which is the index a strictly-greater scan in ascending channel
// order ends with.
// ------------------------------------------------------------------------------------------------
// Epilogue of the no-grad p = inf kernels: subtract the layer's running mean, add its bias (the two elementwise
// passes of an eval-mode layer, core/modules/basic_modules.py:128-132 and core/modules/norm_dist.py:37-38, with the
// same two roundings).  Channel = layer group * outputs per group + n.
__device__ __forceinline__ float col_epilogue(float v, int n, int g, const TileParams& P) {
    if (P.col_sub == nullptr && P.col_add == nullptr) return v;
    const int ch = (P.b_group_mod > 0 ? g % P.b_group_mod : g) * P.N + n;
    if (P.col_sub) v = __fsub_rn(v, P.col_sub[ch]);
    if (P.col_add) v = __fadd_rn(v, P.col_add[ch]);
    return v;
}

template <bool POS, bool PACK_K = true>
struct FwdInf : FwdLayout {
    static constexpr bool N_IN_SMEM = POS;  // frees 64 registers of the indexed kernel (0.83 -> 0.79 ms)
    static constexpr bool ROLLED_EPILOGUE = !POS;
    static constexpr bool SHORT_STAGES = !POS;
    static constexpr int UNROLL = 4;  // (128 x 64 tiles with two CTAs per SM: 0.556 ms against 0.548 ms)
    static constexpr int KSTEP = 4;  // few instructions per pair: wide shared-memory reads, fewer loop trips
    static constexpr bool PREFETCH = false;  // two 4-wide slabs would not fit the register file
    // POS: f[1] = running maximum, f[0] = its value when a stage last ended with a strict increase, n[0] = that stage
    // (-1: never); the result is f[0] (== f[1] after the last stage)
    static constexpr int NUM_A = 1, NF = POS ? 2 : 1, NI = POS ? 1 : 0;
    static constexpr bool HAS_P = false;
    static constexpr bool STAGE_HOOK = POS;
    __device__ static void init(float* f, int* n) {
        f[0] = kEps;
        if (POS) {
            f[1] = kEps;
            n[0] = -1;
        }
    }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* a, const float*, const float* b, int, int,
                                  const TileParams&) {
        float& m = f[POS ? 1 : 0];
        // The subtraction is packed along k (both operands arrive as neighbouring registers of a 16-byte shared-memory
        // read): one issue slot for two differences.  Every kernel of this family is bound by the issue rate
        // (one warp instruction per scheduler and clock), not by a pipe; measured 0.572 -> 0.548 ms.
        // (PACK_K = false: a k-major A operand delivers one k of four rows per read, so two neighbouring k of a row
        // are not neighbouring registers and every packed operand would first be moved together)
        static_assert(KS % 2 == 0, "packed subtraction walks k in pairs");
        if constexpr (PACK_K) {
#pragma unroll
            for (int k = 0; k < KS; k += 2) {
                const float2 d = pk_sub(make_float2(a[k], a[k + 1]), make_float2(b[k], b[k + 1]));
                m = fmaxf(fmaxf(m, fabsf(d.x)), fabsf(d.y));
            }
        } else {
#pragma unroll
            for (int k = 0; k < KS; ++k) m = fmaxf(m, fabsf(a[k] - b[k]));
        }
    }
    // end of a 32-channel stage: stages are visited in ascending order, so a strict comparison keeps the
    // first stage that reaches the final maximum
    __device__ static void stage_end(float* f, int* n, int stage) {
        if (POS) {
            if (f[1] > f[0]) {
                f[0] = f[1];
                n[0] = stage;
            }
        }
    }
    __device__ static void combine(float* f, int* n, const float* pf, const int* pn) {
        if (POS) {
            if (pf[0] > f[0]) {
                f[0] = pf[0];
                n[0] = pn[0];
            }
        } else {
            f[0] = fmaxf(f[0], pf[0]);
        }
    }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int* nn, float, int m, int n, int g, const TileParams& P) {
        const long long off = out_offset(P.out, m, n, g);
        P.out_f0[off] = POS ? f[0] : col_epilogue(f[0], n, g, P);
        if (POS) P.out_i0[off] = nn[0];  // stage id (or -1); turned into the index by rescan_kernel
    }
};

// ------------------------------------------------------------------------------------------------
// p = inf interval bounds, forward.  A operands are the (sanitised) lower and upper inputs; with
// t1 = w - lower, t2 = upper - w the lower bound is -min(-1e-10, min_c min(t1, t2)) and the upper
// bound max(1e-10, max_c max(t1, t2)).  FwdBound produces both values.  The variant with argmin /
// argmax indices would need four accumulators per output, so it runs as two passes of FwdBoundPos
// (one per bound), each tracking the 4-channel group like FwdInf<true>.
// ------------------------------------------------------------------------------------------------
struct FwdBound : FwdLayout {
    static constexpr bool SHORT_STAGES = true;
    static constexpr int KSTEP = 4;  // measured best: 4-wide k-groups, no register double buffering, one per trip
    static constexpr bool PREFETCH = false;
    static constexpr int UNROLL = 1;  // packed subtractions (see FwdInf): 1.484 -> 1.418 ms
    static constexpr int NUM_A = 2, NF = 2, NI = 0;
    static constexpr bool HAS_P = false;
    __device__ static void init(float* f, int*) {
        f[0] = -kEps;
        f[1] = kEps;
    }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* lo, const float* up, const float* w, int, int,
                                   const TileParams&) {
#pragma unroll
        for (int k = 0; k < KS; k += 2) {
            const float2 w2 = make_float2(w[k], w[k + 1]);
            const float2 t1 = pk_sub(w2, make_float2(lo[k], lo[k + 1]));
            const float2 t2 = pk_sub(make_float2(up[k], up[k + 1]), w2);
            f[0] = fminf(fminf(f[0], t1.x), t2.x);
            f[1] = fmaxf(fmaxf(f[1], t1.x), t2.x);
            f[0] = fminf(fminf(f[0], t1.y), t2.y);
            f[1] = fmaxf(fmaxf(f[1], t1.y), t2.y);
        }
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) {
        f[0] = fminf(f[0], pf[0]);
        f[1] = fmaxf(f[1], pf[1]);
    }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        const long long off = out_offset(P.out, m, n, g);
        P.out_f0[off] = col_epilogue(-f[0], n, g, P);
        P.out_f1[off] = col_epilogue(f[1], n, g, P);
    }
};

template <bool UPPER>
struct FwdBoundPos : FwdLayout {
    static constexpr bool N_IN_SMEM = true;
    static constexpr bool ROLLED_EPILOGUE = false;
    static constexpr int STAGES = 3;  // 3 x 48 KB of operand tiles + 64 KB of stage ids
    static constexpr int KSTEP = 4;
    static constexpr int UNROLL = 2;
    static constexpr bool PREFETCH = false;
    // f[0] = running extremum, f[1] = extremum inside the current stage, n[0] = stage of the last strict
    // improvement (-1: never), as in FwdInf<true>
    static constexpr int NUM_A = 2, NF = 2, NI = 1;
    static constexpr bool HAS_P = false;
    static constexpr bool STAGE_HOOK = true;
    __device__ static void init(float* f, int* n) {
        f[0] = UPPER ? kEps : -kEps;
        f[1] = UPPER ? -FLT_MAX : FLT_MAX;
        n[0] = -1;
    }
    __device__ static float pick(float t1, float t2) { return UPPER ? fmaxf(t1, t2) : fminf(t1, t2); }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* lo, const float* up, const float* w, int, int,
                                  const TileParams&) {
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float t1 = w[k] - lo[k], t2 = up[k] - w[k];
            f[1] = UPPER ? fmaxf(fmaxf(f[1], t1), t2) : fminf(fminf(f[1], t1), t2);
        }
    }
    __device__ static void stage_end(float* f, int* n, int stage) {
        if (UPPER ? (f[1] > f[0]) : (f[1] < f[0])) {
            f[0] = f[1];
            n[0] = stage;
        }
        f[1] = UPPER ? -FLT_MAX : FLT_MAX;
    }
    __device__ static void combine(float* f, int* n, const float* pf, const int* pn) {
        if (UPPER ? (pf[0] > f[0]) : (pf[0] < f[0])) {
            f[0] = pf[0];
            n[0] = pn[0];
        }
    }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int* nn, float, int m, int n, int g, const TileParams& P) {
        const long long off = out_offset(P.out, m, n, g);
        const int pos = nn[0];  // stage id (or -1); turned into the index by rescan_kernel
        if (UPPER) {
            P.out_f1[off] = f[0];
            P.out_i1[off] = pos;
        } else {
            P.out_f0[off] = -f[0];
            P.out_i0[off] = pos;
        }
    }
};

// Both bounds with both stage ids in one pass: four accumulators per output (running and current-stage minimum,
// running and current-stage maximum) fit the register file on the 128 x 64 tile (32 outputs per thread).  The two
// stage ids share one shared-memory word per output: bits 0..15 hold (stage of the minimum) + 1, bits 16..31
// (stage of the maximum) + 1, 0 meaning "never improved"; reductions of more than 65534 stages take the two-pass
// kernels above.
struct FwdBoundBoth : FwdLayout {
    static constexpr bool N_IN_SMEM = true;
    static constexpr bool ROLLED_EPILOGUE = false;
    static constexpr int REG_N = 4;
    static constexpr int KSTEP = 4;
    static constexpr int UNROLL = 1;
    static constexpr bool PREFETCH = false;
    // f[1] / f[3] = running minimum / maximum, f[0] / f[2] = their values when a stage last ended with a strict
    // improvement; n[0] = the two 16-bit stage ids
    static constexpr int NUM_A = 2, NF = 4, NI = 1;
    static constexpr bool HAS_P = false;
    static constexpr bool STAGE_HOOK = true;
    static constexpr int kMaxStages = 65534;
    __device__ static void init(float* f, int* n) {
        f[0] = f[1] = -kEps;
        f[2] = f[3] = kEps;
        n[0] = 0;
    }
    template <int KS>
    __device__ static void update(float* f, int*, float, const float* lo, const float* up, const float* w, int, int,
                                  const TileParams&) {
#pragma unroll
        for (int k = 0; k < KS; k += 2) {
            const float2 w2 = make_float2(w[k], w[k + 1]);
            const float2 t1 = pk_sub(w2, make_float2(lo[k], lo[k + 1]));
            const float2 t2 = pk_sub(make_float2(up[k], up[k + 1]), w2);
            f[1] = fminf(fminf(f[1], t1.x), t2.x);
            f[3] = fmaxf(fmaxf(f[3], t1.x), t2.x);
            f[1] = fminf(fminf(f[1], t1.y), t2.y);
            f[3] = fmaxf(fmaxf(f[3], t1.y), t2.y);
        }
    }
    // the halves of the id word are written as 16-bit stores: no read-modify-write
    __device__ static void stage_end(float* f, int* n, int stage) {
        unsigned short* ids = reinterpret_cast<unsigned short*>(n);
        if (f[1] < f[0]) {
            f[0] = f[1];
            ids[0] = static_cast<unsigned short>(stage + 1);
        }
        if (f[3] > f[2]) {
            f[2] = f[3];
            ids[1] = static_cast<unsigned short>(stage + 1);
        }
    }
    __device__ static void combine(float* f, int* n, const float* pf, const int* pn) {
        if (pf[0] < f[0]) {
            f[0] = pf[0];
            n[0] = (n[0] & static_cast<int>(0xffff0000u)) | (pn[0] & 0xffff);
        }
        if (pf[2] > f[2]) {
            f[2] = pf[2];
            n[0] = (n[0] & 0xffff) | (pn[0] & static_cast<int>(0xffff0000u));
        }
    }
    __device__ static float load_pres(const TileParams&, int, int, int) { return 0.0f; }
    __device__ static void finalize(const float* f, const int* nn, float, int m, int n, int g, const TileParams& P) {
        const long long off = out_offset(P.out, m, n, g);
        P.out_f0[off] = -f[0];
        P.out_f1[off] = f[2];
        // stage ids (or -1); turned into the indices by rescan_kernel
        P.out_i0[off] = (nn[0] & 0xffff) - 1;
        P.out_i1[off] = static_cast<int>(static_cast<unsigned>(nn[0]) >> 16) - 1;
    }
};

// ------------------------------------------------------------------------------------------------
// Finite p, backward.  One engine problem per gradient:
//   grad_x: out (m = (b, hw), n = c), k = o;  A = coefficient [m][k] (RowMajor), B = w [k][n] (KMajor),
//           resident = x[m][n], t = resident - B
//   grad_w: out (m = o, n = c), k = (b, hw);  A = coefficient [k][m] (KMajor),  B = x [k][n] (KMajor),
//           resident = w[m][n], t = B - resident, result negated
// Integer p - 1: coefficient = g / y^(p-1), term = coefficient * sgn(t) |t|^(p-1).
// General p:     coefficients c = -(p-1) lg2 y and g, term = g * sgn(t) * 2^((p-1) lg2|t| + c).
// ------------------------------------------------------------------------------------------------
template <bool WEIGHT>
struct BwdLayout {
    static constexpr Layout LA = WEIGHT ? Layout::KMajor : Layout::RowMajor;
    static constexpr Layout LB = Layout::KMajor;
    static constexpr int KSTEP = 2;
    static constexpr bool PACKED = false;
    static constexpr bool PREFETCH = false;  // the resident operand leaves no registers for it
    static constexpr bool FUSED_W = false;
    static constexpr bool STAGE_HOOK = false;
    static constexpr bool SHORT_STAGES = false;
    static constexpr int UNROLL = 1;
    static constexpr bool N_IN_SMEM = false;
    static constexpr bool ROLLED_EPILOGUE = false;  // measured: no gain for the backward kernels (160-stage tiles)
    static constexpr bool ROLLED_PRES = false;
    static constexpr int STAGES = kStages;
    static constexpr int REG_N = 8;
    static constexpr int CTAS_PER_SM = 1;
    static constexpr bool HAS_P = true;
    __device__ static float load_pres(const TileParams& P, int m, int n, int g) {
        return P.pres.ptr[n + m * P.pres.stride_row + g * P.pres.stride_group];
    }
    __device__ static float diff(float pres, float b) { return WEIGHT ? b - pres : pres - b; }
    __device__ static void store(float v, int m, int n, int g, const TileParams& P) {
        float* dst = P.out_f0 + out_offset(P.out, m, n, g);
        v = WEIGHT ? -v : v;
        *dst = P.accumulate_out ? *dst + v : v;
    }
};

template <int IQ, bool WEIGHT>
struct BwdPowInt : BwdLayout<WEIGHT> {
    using L = BwdLayout<WEIGHT>;
    static constexpr int KSTEP = 4;                 // measured best per gradient
    static constexpr int UNROLL = WEIGHT ? 1 : 2;
    static constexpr int NUM_A = 1, NF = 1, NI = 0;
    static constexpr bool PACKED = IQ >= 1;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    template <int KS>
    __device__ static void update_pair(float& s0, float& s1, float p0, float p1, const float* c, const float*,
                                       const float* b0, const float* b1, int, const TileParams&) {
        const float2 pr = pk(p0, p1);
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float2 bb = pk(b0[k], b1[k]);
            const float2 sp = signed_pow2<(IQ >= 1 ? IQ : 1)>(WEIGHT ? pk_sub(bb, pr) : pk_sub(pr, bb));
            s0 = fmaf(c[k], sp.x, s0);
            s1 = fmaf(c[k], sp.y, s1);
        }
    }
    template <int KS>
    __device__ static void update(float* f, int*, float pres, const float* c, const float*, const float* b, int, int,
                                   const TileParams&) {
#pragma unroll
        for (int k = 0; k < KS; ++k) f[0] = fmaf(c[k], signed_pow<IQ>(L::diff(pres, b[k])), f[0]);
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        L::store(f[0], m, n, g, P);
    }
};

// FOLD: coefficient 0 is the exponent offset c = -q lg2 y and the power is 2^(q lg2|t| + c); otherwise it is
// 1 / y and the power is 2^(q lg2(|t| / y)) -- one multiply more per pair, but the logarithm is taken near 1 where
// its absolute error is smallest, which matters once q reaches the hundreds.
__device__ __forceinline__ float2 gen_exponent(float2 t, float c, float q, bool fold) {
    if (fold) {
        const float2 l = make_float2(lg2_approx(fabsf(t.x)), lg2_approx(fabsf(t.y)));
        return __ffma2_rn(make_float2(q, q), l, make_float2(c, c));
    }
    const float2 u = __fmul2_rn(t, make_float2(c, c));
    const float2 l = make_float2(lg2_approx(fabsf(u.x)), lg2_approx(fabsf(u.y)));
    return __fmul2_rn(make_float2(q, q), l);
}

template <bool WEIGHT, bool FOLD>
struct BwdPowGen : BwdLayout<WEIGHT> {
    using L = BwdLayout<WEIGHT>;
    static constexpr int NUM_A = 2, NF = 1, NI = 0;
    static constexpr bool PACKED = true;
    // two CTAs of the 128 x 64 tile per SM (see BwdFusedGen)
    static constexpr int UNROLL = 4;
    static constexpr int STAGES = 2;
    static constexpr int REG_N = 4;
    static constexpr int CTAS_PER_SM = 2;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    template <int KS>
    __device__ static void update_pair(float& s0, float& s1, float p0, float p1, const float* r, const float* gr,
                                       const float* b0, const float* b1, int sel, const TileParams& P) {
        const float2 pr = make_float2(p0, p1);
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float2 bb = make_float2(b0[k], b1[k]);
            const float2 t = WEIGHT ? pk_sub(bb, pr) : pk_sub(pr, bb);
            const float2 v = ex2_mixed2<4, kMufuEveryBwd>(gen_exponent(t, r[k], P.q, FOLD), sel + k);
            s0 = fmaf(gr[k], copysignf(v.x, t.x), s0);
            s1 = fmaf(gr[k], copysignf(v.y, t.y), s1);
        }
    }
    template <int KS>
    __device__ static void update(float* f, int*, float pres, const float* r, const float* gr, const float* b, int, int sel,
                                   const TileParams& P) {
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const float t = L::diff(pres, b[k]);
            const float v = ex2_mixed<4>(FOLD ? fmaf(P.q, lg2_approx(fabsf(t)), r[k]) : P.q * lg2_approx(fabsf(t) * r[k]),
                                         sel + k);
            f[0] = fmaf(gr[k], copysignf(v, t), f[0]);
        }
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        L::store(f[0], m, n, g, P);
    }
};

// ------------------------------------------------------------------------------------------------
// Fused backward (grad_input and grad_weight from one evaluation of every term).  The problem is the
// grad_x one (out (m = (b, hw), n = c), k = o, resident x); in addition the engine sums every term over
// the 128 rows of the CTA's tile and writes those column sums per row tile, [tile_m][g][o][c]; a small
// kernel adds the row tiles and negates (side_reduce_kernel).  Every (tile_m, o, c) is produced by
// exactly one CTA, so the result is deterministic.
// ------------------------------------------------------------------------------------------------
template <int IQ>
struct BwdFusedInt : BwdLayout<false> {
    using L = BwdLayout<false>;
    static constexpr int NUM_A = 1, NF = 1, NI = 0;
    static constexpr bool PACKED = true;
    static constexpr bool FUSED_W = true;
    static constexpr int KSTEP = 4;  // measured best: 4-wide k-groups, two per trip
    static constexpr int UNROLL = 2;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    // term = coef * returned value
    __device__ static float2 term_pair(float p0, float p1, float c, float, float b0, float b1, int,
                                       const TileParams&, float2& coef) {
        coef = make_float2(c, c);
        return signed_pow2<IQ>(pk_sub(make_float2(p0, p1), make_float2(b0, b1)));
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        L::store(f[0], m, n, g, P);
    }
};

template <bool FOLD>
struct BwdFusedGen : BwdLayout<false> {
    using L = BwdLayout<false>;
    static constexpr int NUM_A = 2, NF = 1, NI = 0;
    static constexpr bool PACKED = true;
    static constexpr bool FUSED_W = true;
    // two CTAs of the 128 x 64 tile per SM: twice the warps to cover the MUFU / polynomial dependency chains
    static constexpr int UNROLL = 2;
    static constexpr int STAGES = 2;
    static constexpr int REG_N = 4;
    static constexpr int CTAS_PER_SM = 2;
    __device__ static void init(float* f, int*) { f[0] = 0.0f; }
    __device__ static float2 term_pair(float p0, float p1, float r, float gr, float b0, float b1, int sel,
                                       const TileParams& P, float2& coef) {
        const float2 t = pk_sub(make_float2(p0, p1), make_float2(b0, b1));
        const float2 v = ex2_mixed2<4, kMufuEveryBwd>(gen_exponent(t, r, P.q, FOLD), sel);
        coef = make_float2(gr, gr);
        return make_float2(copysignf(v.x, t.x), copysignf(v.y, t.y));
    }
    __device__ static void combine(float* f, int*, const float* pf, const int*) { f[0] += pf[0]; }
    __device__ static void finalize(const float* f, const int*, float, int m, int n, int g, const TileParams& P) {
        L::store(f[0], m, n, g, P);
    }
};

}  // namespace ldn
