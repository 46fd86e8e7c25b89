// The tile engine shared by every compute-bound kernel of the library.
//
// All of them have the shape  out[m, n] = REDUCE_k  f(A[m or k, ...], B[n or k, ...], resident[m, n])
// over a per-group problem (M, N, K).  The engine is a persistent kernel: the global iteration space
// (tile, k-step of 32) is cut into one contiguous, equally long range per CTA ("stream-K"), so that
// all SMs finish together whatever the tile count.  A CTA that owns a whole tile finalises it itself;
// a CTA that owns only part of a tile's k-range stores its raw accumulators into scratch, and a small
// second kernel (`tile_fixup_kernel`) folds those partials in k order and finalises -- there is no
// inter-CTA waiting anywhere.
//
// Operand tiles are fetched by TMA (cp.async.bulk.tensor, 3-D, no multicast) into a shared-memory ring of
// Op::STAGES (2 to 4) stages, completion on one mbarrier per stage; out-of-range rows / k are zero-filled by
// the TMA unit, and every op is written so that zero padding is neutral.  Two tile shapes exist:
//   RowMajor: [128 rows][32 k]  (k contiguous in global memory), stored with the 128-byte swizzle;
//   KMajor:   [32 k][128 cols]  (cols contiguous in global memory), stored linearly.
// Register blocking: thread (tm, tn) of the 16 x 16 thread grid owns 8 x 8 outputs; with a RowMajor
// operand its rows are t + 16 r (conflict-free with the swizzle), with a KMajor operand its columns
// are 4 t .. 4 t + 3 and 64 + 4 t .. 64 + 4 t + 3 (conflict-free 128-bit reads).
#pragma once
#include "ldn_common.cuh"

namespace ldn {

enum class Layout { RowMajor, KMajor };

constexpr int kStages = 4;  // default depth of the operand ring (Op::STAGES)

// R = number of rows / columns a thread owns in that dimension (8; 4 or 2 for the narrow 128 x 64 / 128 x 32 tiles,
// the latter with row-major operands only)
template <Layout L, int R = 8>
__device__ __forceinline__ int own_index(int t, int r) {
    if (L == Layout::RowMajor) return t + 16 * r;
    static_assert(L == Layout::RowMajor || R == 8 || R == 4, "a k-major tile is 128 or 64 columns wide");
    if (R == 4) return t * 4 + r;
    return (r >> 2) * 64 + t * 4 + (r & 3);
}

// Fetch the 8 x KS register slab (8 owned rows/cols x KS consecutive k, KS in {1, 2, 4}) of one operand
// tile for k-group `ps` (k = ps * KS .. ps * KS + KS - 1 inside the 32-wide stage).
template <Layout L, int KS, int R>
__device__ __forceinline__ void fetch_slab(const char* tile, int t, int ps, float (&v)[R][KS]) {
    static_assert(R == 8 || R == 4 || R == 2, "a thread owns 8, 4 or 2 rows / columns");
    static_assert(L == Layout::RowMajor || R != 2, "a k-major tile is 128 or 64 columns wide");
    static_assert(KS == 1 || KS == 2 || KS == 4, "k-step must be 1, 2 or 4");
    if (L == Layout::RowMajor) {
        const int k = ps * KS;
        const int off = (((k >> 2) ^ (t & 7)) << 4) + ((k & 3) << 2);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const char* src = tile + (t + 16 * r) * 128 + off;
            if constexpr (KS == 4) {
                const float4 x = *reinterpret_cast<const float4*>(src);
                v[r][0] = x.x; v[r][1] = x.y; v[r][2] = x.z; v[r][3] = x.w;
            } else if constexpr (KS == 2) {
                const float2 x = *reinterpret_cast<const float2*>(src);
                v[r][0] = x.x; v[r][1] = x.y;
            } else {
                v[r][0] = *reinterpret_cast<const float*>(src);
            }
        }
    } else {
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            // a k-major tile row holds 16 * R floats
            const char* row = tile + (ps * KS + kk) * (R * 64) + t * 16;
            const float4 lo = *reinterpret_cast<const float4*>(row);
            v[0][kk] = lo.x; v[1][kk] = lo.y; v[2][kk] = lo.z; v[3][kk] = lo.w;
            if constexpr (R == 8) {
                const float4 hi = *reinterpret_cast<const float4*>(row + 256);
                v[4][kk] = hi.x; v[5][kk] = hi.y; v[6][kk] = hi.z; v[7][kk] = hi.w;
            }
        }
    }
}

struct TileCoord {
    int g, m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(const TileParams& P, long long tile, int tile_n) {
    TileCoord c;
    const int per_group = P.tiles_m * P.tiles_n;
    c.g = static_cast<int>(tile / per_group);
    const int r = static_cast<int>(tile - static_cast<long long>(c.g) * per_group);
    c.m0 = (r % P.tiles_m) * kTileM;
    c.n0 = (r / P.tiles_m) * tile_n;
    return c;
}

__device__ __forceinline__ long long out_offset(const OutAddr& o, int m, int n, int g) {
    const int b = (o.hw_div == 1) ? m : m / o.hw_div;
    const int hw = (o.hw_div == 1) ? 0 : m - b * o.hw_div;
    return static_cast<long long>(b) * o.s_b + static_cast<long long>(hw) * o.s_hw +
           static_cast<long long>(g) * o.s_g + static_cast<long long>(n) * o.s_n;
}

// first iteration of CTA c when `total` iterations are spread over `grid` CTAs
__host__ __device__ __forceinline__ long long range_begin(long long total, int grid, int c) {
    return (total * c) / grid;
}

// Position of a thread in the 16 x 16 thread grid.  Default: a warp holds 2 rows x 16 columns of threads.
// Fused-backward ops put 16 rows x 2 columns into a warp, so that the sum over the tile's rows is a
// shuffle reduction inside the warp.
template <class Op>
__device__ __forceinline__ int thread_row(int tid) {
    return Op::FUSED_W ? (tid & 15) : (tid >> 4);
}
template <class Op>
__device__ __forceinline__ int thread_col(int tid) {
    return Op::FUSED_W ? (((tid >> 4) & 1) + 2 * (tid >> 5)) : (tid & 15);
}


template <class Op>
struct TileSmem {
    static constexpr int kTileN = 16 * Op::REG_N;
    static constexpr int kStage = Op::NUM_A * kOperandTileBytes + kTileN * kTileK * 4;
    static constexpr int kSideBuffer = kTileK * kTileN * 4;  // column sums of one stage (fused backward)
    static constexpr int kSide = Op::FUSED_W ? 2 * kSideBuffer : 0;
    // ops with N_IN_SMEM keep their integer accumulators (one per output, rarely written) in shared memory
    static constexpr int kInts = Op::N_IN_SMEM ? kThreads * kRegM * Op::REG_N * Op::NI * 4 : 0;
    static constexpr int kTotal = Op::STAGES * kStage + kSide + kInts + 1024 /*alignment slack*/ + 64 /*barriers*/;
};

// RM = how many of a thread's 8 register rows are computed: 8, or 4 when the whole problem has at most 64 rows
// (small batches) -- rows t + 16 r with r >= 4 are then all beyond M, in every tile and for every thread.
template <class Op, int RM = kRegM>
__global__ void __launch_bounds__(kThreads, Op::CTAS_PER_SM)
tile_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
            const __grid_constant__ CUtensorMap map_b, const TileParams P) {
    constexpr int NA = Op::NUM_A;
    constexpr int NF = Op::NF;
    constexpr int NI = Op::NI;
    constexpr int NIA = NI > 0 ? NI : 1;
    constexpr int STAGE = TileSmem<Op>::kStage;
    constexpr int STAGES = Op::STAGES;
    constexpr int RN = Op::REG_N;          // output columns per thread
    constexpr int TN = 16 * RN;            // output columns per tile
    constexpr int TELEMS = kTileM * TN;    // outputs per tile
    static_assert(RN == 8 || RN == 4 || RN == 2, "a thread owns 8, 4 or 2 output columns");

    extern __shared__ char smem_raw[];
    char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* side = reinterpret_cast<float*>(smem + STAGES * STAGE);  // two column-sum buffers (fused backward)
    int* ints = reinterpret_cast<int*>(smem + STAGES * STAGE + TileSmem<Op>::kSide);  // N_IN_SMEM ops
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE + TileSmem<Op>::kSide + TileSmem<Op>::kInts);

    if (P.gate != nullptr && (*P.gate != 0) == (P.gate_invert != 0)) return;
    const int tid = threadIdx.x;
    const int tn = thread_col<Op>(tid);
    const int tm = thread_row<Op>(tid);
    const int grid = gridDim.x;
    const long long it0 = range_begin(P.total_iters, grid, blockIdx.x);
    const long long it1 = range_begin(P.total_iters, grid, blockIdx.x + 1);
    if (it0 >= it1) return;
    const int KT = P.kt;
    unsigned long long t_start = 0;
    if (P.trace && tid == 0) t_start = global_timer_ns();

    if (tid == 0) {
        tma_prefetch_desc(&map_a0);
        if (NA == 2) tma_prefetch_desc(&map_a1);
        tma_prefetch_desc(&map_b);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // producer side (thread 0): fill stage `ls % STAGES` with the operands of iteration `it`
    auto issue = [&](long long it, int ls) {
        const long long tile = it / KT;
        const int kt = static_cast<int>(it - tile * KT);
        const TileCoord tc = tile_coord(P, tile, TN);
        char* st = smem + (ls % STAGES) * STAGE;
        uint64_t* bar = &full[ls % STAGES];
        mbar_expect_tx(bar, STAGE);
        const int k0 = kt * kTileK;
        {
            int c0, c1, c2;
            if (Op::LA == Layout::RowMajor) { c0 = k0; c1 = tc.m0; } else { c0 = tc.m0; c1 = k0; }
            c2 = tc.g;
            if (P.a_row_coord == 2) { int t = c1; c1 = c2; c2 = t; }
            tma_load_3d(st, &map_a0, bar, c0, c1, c2);
            if (NA == 2) tma_load_3d(st + kOperandTileBytes, &map_a1, bar, c0, c1, c2);
        }
        {
            int c0, c1, c2;
            if (Op::LB == Layout::RowMajor) { c0 = k0; c1 = tc.n0; } else { c0 = tc.n0; c1 = k0; }
            // (when every sample is its own engine group, B -- the weight -- still has only the layer's groups)
            c2 = P.b_group_mod > 0 ? tc.g % P.b_group_mod : tc.g;
            if (P.b_row_coord == 2) { int t = c1; c1 = c2; c2 = t; }
            tma_load_3d(st + NA * kOperandTileBytes, &map_b, bar, c0, c1, c2);
        }
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES - 1; ++s)
            if (it0 + s < it1) issue(it0 + s, s);
    }

    // fused backward: write the column sums of a finished stage (rows = its 32 k values) to
    // side_out[tile_m][g][k][n]
    auto flush_side = [&](long long it_done, int buf) {
        const long long tile_d = it_done / KT;
        const int kt_d = static_cast<int>(it_done - tile_d * KT);
        const TileCoord cd = tile_coord(P, tile_d, TN);
        float* src = side + buf * (kTileK * TN);
        float* dst_tile = P.side_out + (static_cast<size_t>(cd.m0 / kTileM) * P.G + cd.g) * (size_t)P.K * P.N;
        const bool vec = (P.N & 3) == 0;
#pragma unroll
        for (int q = 0; q < (kTileK * TN / 4) / kThreads; ++q) {
            const int idx4 = tid + kThreads * q;
            const int r = idx4 / (TN / 4);
            const int c4 = (idx4 % (TN / 4)) * 4;
            float4* sp = reinterpret_cast<float4*>(src + r * TN + c4);
            const float4 v = *sp;
            const int o = kt_d * kTileK + r;
            const int n = cd.n0 + c4;
            if (o < P.K && n < P.N) {
                float* dst = dst_tile + static_cast<size_t>(o) * P.N + n;
                if (vec) {
                    *reinterpret_cast<float4*>(dst) = v;
                } else {
                    dst[0] = v.x;
                    if (n + 1 < P.N) dst[1] = v.y;
                    if (n + 2 < P.N) dst[2] = v.z;
                    if (n + 3 < P.N) dst[3] = v.w;
                }
            }
        }
    };

    float accf[kRegM][RN][NF];
    static_assert(!Op::N_IN_SMEM || NI == 1, "one integer accumulator per output in shared memory");
    int acci[Op::N_IN_SMEM ? 1 : kRegM][Op::N_IN_SMEM ? 1 : RN][NIA];
    // integer accumulators of output (i, j): registers, or this thread's slots of the shared array
    // ([array][output][thread]: neighbouring threads touch neighbouring words)
    auto iacc = [&](int i, int j) -> int* {
        if constexpr (Op::N_IN_SMEM) return ints + (i * RN + j) * kThreads + tid;
        else return acci[i][j];
    };
    float pres[kRegM][RN];
    TileCoord tc = {0, 0, 0};
    long long seg_begin = it0;
    const long long first_tile = it0 / KT;

    for (long long it = it0; it < it1; ++it) {
        const int ls = static_cast<int>(it - it0);
        const long long tile = it / KT;
        const int kt = static_cast<int>(it - tile * KT);
        if (it == it0 || kt == 0) {
            seg_begin = it;
            tc = tile_coord(P, tile, TN);
#pragma unroll
            for (int i = 0; i < kRegM; ++i)
#pragma unroll
                for (int j = 0; j < RN; ++j) {
                    Op::init(accf[i][j], iacc(i, j));
                    if (Op::HAS_P && !Op::ROLLED_PRES) {
                        const int m = tc.m0 + own_index<Op::LA>(tm, i);
                        const int n = tc.n0 + own_index<Op::LB, RN>(tn, j);
                        pres[i][j] = (m < P.M && n < P.N) ? Op::load_pres(P, m, n, tc.g) : 0.0f;
                    } else {
                        pres[i][j] = 0.0f;
                    }
                }
            if constexpr (Op::HAS_P && Op::ROLLED_PRES) {
                // one register row per trip of a rolled loop (see the epilogue below): the rows move down one
                // slot per trip, the row loaded in trip i ends in slot i
#pragma unroll 1
                for (int i = 0; i < kRegM; ++i) {
#pragma unroll
                    for (int r = 0; r + 1 < kRegM; ++r)
#pragma unroll
                        for (int j = 0; j < RN; ++j) pres[r][j] = pres[r + 1][j];
                    const int m = tc.m0 + own_index<Op::LA>(tm, i);
#pragma unroll
                    for (int j = 0; j < RN; ++j) {
                        const int n = tc.n0 + own_index<Op::LB, RN>(tn, j);
                        pres[kRegM - 1][j] = (m < P.M && n < P.N) ? Op::load_pres(P, m, n, tc.g) : 0.0f;
                    }
                }
            }
        }

        // A wait that runs out: the thread records the status and returns; the host reads the status word
        // (ldn_check_status).  All threads of a CTA wait on the same barrier with the same budget, so they give up
        // together.  (Variants that made the outcome CTA-uniform -- through the barrier that follows, or a shared flag
        // checked behind it -- or that first waited for the loads still in flight cost the forward and general-p
        // kernels 1 - 7 % in same-GPU A/B runs and were dropped: the schedule of this loop is that sensitive.)
        if (!mbar_wait_bounded(&full[ls % STAGES], (ls / STAGES) & 1)) {
            atomicExch(P.status, static_cast<int>(kDeviceTimeout));
            return;
        }
        __syncthreads();  // every warp is done with the stage that is refilled next
        if (tid == 0 && it + (STAGES - 1) < it1) issue(it + (STAGES - 1), ls + (STAGES - 1));
        if constexpr (Op::FUSED_W) {
            if (ls > 0) flush_side(it - 1, (ls - 1) & 1);
        }

        const char* sa0 = smem + (ls % STAGES) * STAGE;
        const char* sa1 = sa0 + (NA == 2 ? kOperandTileBytes : 0);
        const char* sb = sa0 + NA * kOperandTileBytes;
        // The k-groups of a stage are walked in a rolled loop so that the loop body (64 outputs x KS k x
        // a few FP32 instructions) stays resident in the instruction cache.  Threads with tn >= 8 visit
        // each pair of neighbouring k-groups in swapped order (KS < 4): with the 128-byte swizzle that
        // makes the narrower shared-memory reads of a RowMajor B tile bank-conflict free.  The order in
        // which a thread visits k does not matter to any op (sums, exact min / max, 4-channel groups).
        constexpr int KS = Op::KSTEP;
        constexpr int NSTEP = kTileK / KS;
        // (fused-backward ops reduce across the lanes of a warp per k, so all lanes must visit k in the same
        // order: no swap there, at the price of a 2-way conflict on their narrow RowMajor reads)
        const int perm = (KS < 4 && !Op::FUSED_W) ? (tn >> 3) : 0;
        struct Slab {
            float a0[8][KS], a1[8][KS], b[RN][KS];
        };
        auto load = [&](Slab& sl, int ks) {
            const int ps = ks ^ perm;
            fetch_slab<Op::LA, KS, 8>(sa0, tm, ps, sl.a0);
            if (NA == 2) fetch_slab<Op::LA, KS, 8>(sa1, tm, ps, sl.a1);
            fetch_slab<Op::LB, KS, RN>(sb, tn, ps, sl.b);
        };
        auto compute = [&](const Slab& sl, int ks) {
            const int ps = ks ^ perm;
            const int chunk = kt * (kTileK / 4) + ((ps * KS) >> 2);
            if constexpr (Op::FUSED_W) {
                // Fused backward: every term feeds the thread's own accumulator (grad_input, reduced over k)
                // and a column sum over the CTA's 128 rows (grad_weight of this row tile): summed over the
                // thread's 8 rows in registers and over the warp's 16 row groups by shuffles; the finished
                // column sums go to the stage's buffer with plain stores (every column has one owner).
                float* buf = side + (ls & 1) * (kTileK * TN);
#pragma unroll
                for (int k = 0; k < KS; ++k) {
                    float2 col[RN / 2];
#pragma unroll
                    for (int jp = 0; jp < RN / 2; ++jp) col[jp] = make_float2(0.0f, 0.0f);
#pragma unroll
                    for (int i = 0; i < RM; ++i)
#pragma unroll
                        for (int jp = 0; jp < RN / 2; ++jp) {
                            // term = coef * base, folded into both accumulations as one FMA each
                            float2 coef;
                            const float2 base = Op::term_pair(pres[i][2 * jp], pres[i][2 * jp + 1], sl.a0[i][k],
                                                              NA == 2 ? sl.a1[i][k] : 0.0f, sl.b[2 * jp][k],
                                                              sl.b[2 * jp + 1][k], i + jp + k, P, coef);
                            const float2 acc =
                                __ffma2_rn(base, coef, make_float2(accf[i][2 * jp][0], accf[i][2 * jp + 1][0]));
                            accf[i][2 * jp][0] = acc.x;
                            accf[i][2 * jp + 1][0] = acc.y;
                            col[jp] = __ffma2_rn(base, coef, col[jp]);
                        }
                    // Sum over the 16 row groups of the warp (lane bits 0..3) with a halving butterfly:
                    // each exchange step passes on half of the values a lane still holds, so 8 values need
                    // 4 + 2 + 1 shuffles plus one full step (4 values: 2 + 1 plus two full steps), and the
                    // storing lanes end with one finished column each.
                    const bool b3 = (tid & 8) != 0, b2 = (tid & 4) != 0, b1 = (tid & 2) != 0;
                    if constexpr (RN == 8) {
                        float v4[4], v2[2], v1;
                        {
                            const float c0 = col[0].x, c1 = col[0].y, c2 = col[1].x, c3 = col[1].y;
                            const float c4 = col[2].x, c5 = col[2].y, c6 = col[3].x, c7 = col[3].y;
                            v4[0] = (b3 ? c4 : c0) + __shfl_xor_sync(0xffffffffu, b3 ? c0 : c4, 8);
                            v4[1] = (b3 ? c5 : c1) + __shfl_xor_sync(0xffffffffu, b3 ? c1 : c5, 8);
                            v4[2] = (b3 ? c6 : c2) + __shfl_xor_sync(0xffffffffu, b3 ? c2 : c6, 8);
                            v4[3] = (b3 ? c7 : c3) + __shfl_xor_sync(0xffffffffu, b3 ? c3 : c7, 8);
                        }
                        v2[0] = (b2 ? v4[2] : v4[0]) + __shfl_xor_sync(0xffffffffu, b2 ? v4[0] : v4[2], 4);
                        v2[1] = (b2 ? v4[3] : v4[1]) + __shfl_xor_sync(0xffffffffu, b2 ? v4[1] : v4[3], 4);
                        v1 = (b1 ? v2[1] : v2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? v2[0] : v2[1], 2);
                        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                        if ((tid & 1) == 0) {
                            const int j = (b3 ? 4 : 0) + (b2 ? 2 : 0) + (b1 ? 1 : 0);
                            buf[(ps * KS + k) * TN + own_index<Layout::KMajor, RN>(tn, j)] = v1;
                        }
                    } else {
                        const float c0 = col[0].x, c1 = col[0].y, c2 = col[1].x, c3 = col[1].y;
                        const float u0 = (b3 ? c2 : c0) + __shfl_xor_sync(0xffffffffu, b3 ? c0 : c2, 8);
                        const float u1 = (b3 ? c3 : c1) + __shfl_xor_sync(0xffffffffu, b3 ? c1 : c3, 8);
                        float v1 = (b2 ? u1 : u0) + __shfl_xor_sync(0xffffffffu, b2 ? u0 : u1, 4);
                        v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                        if ((tid & 3) == 0) {
                            const int j = (b3 ? 2 : 0) + (b2 ? 1 : 0);
                            buf[(ps * KS + k) * TN + own_index<Layout::KMajor, RN>(tn, j)] = v1;
                        }
                    }
                }
            } else if constexpr (Op::PACKED) {
                // two neighbouring outputs (j, j + 1) at a time, so that the op can use the packed
                // two-lane FP32 instructions (fma.rn.f32x2 ...): half the issue slots per lane operation
#pragma unroll
                for (int i = 0; i < RM; ++i)
#pragma unroll
                    for (int j = 0; j < RN; j += 2)
                        Op::template update_pair<KS>(accf[i][j][0], accf[i][j + 1][0], pres[i][j], pres[i][j + 1],
                                                     sl.a0[i], NA == 2 ? sl.a1[i] : sl.a0[i], sl.b[j], sl.b[j + 1],
                                                     i + (j >> 1), P);
            } else {
#pragma unroll
                for (int i = 0; i < RM; ++i)
#pragma unroll
                    for (int j = 0; j < RN; ++j)
                        Op::template update<KS>(accf[i][j], iacc(i, j), pres[i][j], sl.a0[i],
                                                NA == 2 ? sl.a1[i] : sl.a0[i], sl.b[j], chunk, i + j, P);
            }
        };
        // Op::SHORT_STAGES: the last stage of a reduction that is no multiple of 32 (or a short one, K < 32) stops
        // after its valid k-groups; an even count keeps the pairwise swap above and the double buffering below
        // intact.  (The run-time trip count also changes how the compiler schedules the rolled loop: measured per
        // op family at 512 x 3072 -> 5120, it is on where that was no slower.)
        int nsteps = NSTEP;
        if constexpr (Op::SHORT_STAGES) {
            const int kvalid = P.K - kt * kTileK;
            if (kvalid < kTileK) nsteps = (((kvalid + KS - 1) / KS) + 1) & ~1;
        }
        if constexpr (Op::PREFETCH) {
            // register double buffering: the operands of the next k-group are read from shared memory
            // while the current group is computed (the loop is rolled, the compiler cannot do this itself)
            Slab s0, s1;
            load(s0, 0);
            constexpr int UNR = Op::UNROLL;
#pragma unroll UNR
            for (int ks = 0; ks < nsteps; ks += 2) {
                load(s1, ks + 1);
                compute(s0, ks);
                if (ks + 2 < nsteps) load(s0, ks + 2);
                compute(s1, ks + 1);
            }
        } else {
            constexpr int UNR = Op::UNROLL;  // 1 = rolled; a few ops schedule better with two k-groups per trip
#pragma unroll UNR
            for (int ks = 0; ks < nsteps; ++ks) {
                Slab sl;
                load(sl, ks);
                compute(sl, ks);
            }
        }

        if constexpr (Op::STAGE_HOOK) {
#pragma unroll
            for (int i = 0; i < kRegM; ++i)
#pragma unroll
                for (int j = 0; j < RN; ++j) Op::stage_end(accf[i][j], iacc(i, j), kt);
        }

        if (kt == KT - 1 || it == it1 - 1) {
            const bool whole = (seg_begin == tile * KT) && (kt == KT - 1);
            if (whole && Op::ROLLED_EPILOGUE) {
                // Ops with ROLLED_EPILOGUE finalise one register row per trip of a rolled loop: each trip handles row 0
                // and moves the other rows down one slot (registers cannot be indexed by the trip count).  As
                // straight-line code for all 64 outputs the epilogue is tens of KB of instructions that run once per
                // tile and are fetched from memory every time: for the forward kernels 4 - 5 % of a 96-stage tile and
                // 12 - 16 % of an 18-stage one.  (The backward and the index-tracking kernels were no faster with it.)
#pragma unroll 1
                for (int i = 0; i < RM; ++i) {
                    const int m = tc.m0 + own_index<Op::LA>(tm, i);
#pragma unroll
                    for (int j = 0; j < RN; ++j) {
                        const int n = tc.n0 + own_index<Op::LB, RN>(tn, j);
                        int* ia;
                        if constexpr (Op::N_IN_SMEM) ia = ints + (i * RN + j) * kThreads + tid;
                        else ia = acci[0][j];
                        if (m < P.M && n < P.N) Op::finalize(accf[0][j], ia, pres[0][j], m, n, tc.g, P);
                    }
#pragma unroll
                    for (int r = 0; r + 1 < RM; ++r)
#pragma unroll
                        for (int j = 0; j < RN; ++j) {
#pragma unroll
                            for (int a = 0; a < NF; ++a) accf[r][j][a] = accf[r + 1][j][a];
                            if (Op::HAS_P) pres[r][j] = pres[r + 1][j];
                            if constexpr (!Op::N_IN_SMEM) {
#pragma unroll
                                for (int a = 0; a < NI; ++a) acci[r][j][a] = acci[r + 1][j][a];
                            }
                        }
                }
            } else if (whole) {
                if constexpr (!Op::ROLLED_EPILOGUE) {
#pragma unroll
                    for (int i = 0; i < kRegM; ++i)
#pragma unroll
                        for (int j = 0; j < RN; ++j) {
                            const int m = tc.m0 + own_index<Op::LA>(tm, i);
                            const int n = tc.n0 + own_index<Op::LB, RN>(tn, j);
                            if (m < P.M && n < P.N) Op::finalize(accf[i][j], iacc(i, j), pres[i][j], m, n, tc.g, P);
                        }
                }
            } else {
                const int slot = (tile == first_tile) ? 0 : 1;
                float* dst = P.partials +
                             (static_cast<size_t>(blockIdx.x) * 2 + slot) * (size_t)(NF + NI) * TELEMS;
#pragma unroll
                for (int i = 0; i < kRegM; ++i)
#pragma unroll
                    for (int j = 0; j < RN; ++j) {
                        const int e = (i * RN + j) * kThreads + tid;
#pragma unroll
                        for (int a = 0; a < NF; ++a) dst[a * TELEMS + e] = accf[i][j][a];
#pragma unroll
                        for (int a = 0; a < NI; ++a) dst[(NF + a) * TELEMS + e] = __int_as_float(iacc(i, j)[a]);
                    }
            }
        }
    }
    if constexpr (Op::FUSED_W) {
        __syncthreads();
        flush_side(it1 - 1, static_cast<int>((it1 - 1 - it0) & 1));
    }
    if (P.trace && tid == 0) {
        unsigned long long* tr = P.trace + 4ull * blockIdx.x;
        tr[0] = sm_id();
        tr[1] = t_start;
        tr[2] = global_timer_ns();
        tr[3] = static_cast<unsigned long long>(it1 - it0);
    }
}

// Folds the partial accumulators of every tile that was shared between CTAs, in k order, and
// finalises it.  Launched with kRegM CTAs per tile (CTA r of a tile handles register-row r of every
// thread's block, i.e. 8 outputs per thread) and the grid size of the main kernel as an argument; CTAs
// of unshared tiles return at once.
template <class Op>
__global__ void __launch_bounds__(kThreads)
tile_fixup_kernel(const TileParams P, const int main_grid) {
    constexpr int NF = Op::NF;
    constexpr int NI = Op::NI;
    constexpr int NIA = NI > 0 ? NI : 1;
    constexpr int RN = Op::REG_N;
    constexpr int TN = 16 * RN;
    constexpr int TELEMS = kTileM * TN;
    if (P.gate != nullptr && (*P.gate != 0) == (P.gate_invert != 0)) return;
    const long long tile = blockIdx.x / kRegM;
    const int i = blockIdx.x % kRegM;
    const int KT = P.kt;
    const long long t0 = tile * KT, t1 = t0 + KT;
    // CTA whose range contains iteration t0
    int c = static_cast<int>(((t0 + 1) * main_grid - 1) / P.total_iters);
    if (range_begin(P.total_iters, main_grid, c + 1) >= t1) return;  // owned whole by one CTA

    const int tid = threadIdx.x;
    const int tn = thread_col<Op>(tid);
    const int tm = thread_row<Op>(tid);
    const TileCoord tc = tile_coord(P, tile, TN);
    float accf[RN][NF];
    int acci[RN][NIA];
#pragma unroll
    for (int j = 0; j < RN; ++j) Op::init(accf[j], acci[j]);

    for (; c < main_grid; ++c) {
        const long long b0 = range_begin(P.total_iters, main_grid, c);
        const long long b1 = range_begin(P.total_iters, main_grid, c + 1);
        if (b0 >= t1) break;
        if (b1 <= b0) continue;
        const int slot = (b0 / KT == tile) ? 0 : 1;
        const float* src = P.partials + (static_cast<size_t>(c) * 2 + slot) * (size_t)(NF + NI) * TELEMS;
        float pf[RN][NF];
        int pn[RN][NIA];
#pragma unroll
        for (int j = 0; j < RN; ++j) {
            const int e = (i * RN + j) * kThreads + tid;
#pragma unroll
            for (int a = 0; a < NF; ++a) pf[j][a] = src[a * TELEMS + e];
#pragma unroll
            for (int a = 0; a < NI; ++a) pn[j][a] = __float_as_int(src[(NF + a) * TELEMS + e]);
        }
#pragma unroll
        for (int j = 0; j < RN; ++j) Op::combine(accf[j], acci[j], pf[j], pn[j]);
    }
#pragma unroll
    for (int j = 0; j < RN; ++j) {
        const int m = tc.m0 + own_index<Op::LA>(tm, i);
        const int n = tc.n0 + own_index<Op::LB, RN>(tn, j);
        if (m < P.M && n < P.N) {
            const float pr = Op::HAS_P ? Op::load_pres(P, m, n, tc.g) : 0.0f;
            Op::finalize(accf[j], acci[j], pr, m, n, tc.g, P);
        }
    }
}

// Host launcher (ldn_launch.cuh provides the definition used by the .cu files).
struct TileLaunch {
    CUtensorMap map_a0, map_a1, map_b;
    TileParams params;
    int grid;
};

template <class Op>
int launch_tile(const TileLaunch& L, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr int SMEM = TileSmem<Op>::kTotal;
    // ops whose rows are batch rows also exist with half of the register rows, for problems of at most 64 rows
    constexpr bool HALF = Op::LA == Layout::RowMajor;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tile_kernel<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess && HALF)
            e = cudaFuncSetAttribute(tile_kernel<Op, (HALF ? kRegM / 2 : kRegM)>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return cuda_status(e);
        configured[dev] = true;
    }
    // (a gated launch usually returns at once: the optional timing brackets the ungated kernels only)
    const bool timed = L.params.gate == nullptr;
    if (timed) timing_before(stream);
    if (HALF && L.params.M <= kTileM / 2)
        tile_kernel<Op, (HALF ? kRegM / 2 : kRegM)><<<L.grid, kThreads, SMEM, stream>>>(L.map_a0, L.map_a1, L.map_b,
                                                                                      L.params);
    else
        tile_kernel<Op><<<L.grid, kThreads, SMEM, stream>>>(L.map_a0, L.map_a1, L.map_b, L.params);
    if (timed) timing_after(stream);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_status(e);
    count_launches(1);
    const long long tiles = L.params.total_iters / L.params.kt;
    // a tile can only be shared when the ranges do not fall on tile boundaries
    if (L.params.total_iters % L.grid != 0 || (L.params.total_iters / L.grid) % L.params.kt != 0) {
        tile_fixup_kernel<Op><<<static_cast<unsigned>(tiles * kRegM), kThreads, 0, stream>>>(L.params, L.grid);
        e = cudaGetLastError();
        count_launches(1);
    }
    return cuda_status(e);
}

}  // namespace ldn
