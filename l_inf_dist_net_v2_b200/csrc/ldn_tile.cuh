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
// Operand tiles are fetched by TMA (cp.async.bulk.tensor, 3-D, no multicast) into a 4-stage
// shared-memory ring, completion on one mbarrier per stage; out-of-range rows / k are zero-filled by
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

constexpr int kStages = 4;

template <Layout L>
__device__ __forceinline__ int own_index(int t, int r) {
    if (L == Layout::RowMajor) return t + 16 * r;
    return (r >> 2) * 64 + t * 4 + (r & 3);
}

// Fetch the 8 x KS register slab (8 owned rows/cols x KS consecutive k, KS in {1, 2, 4}) of one operand
// tile for k-group `ps` (k = ps * KS .. ps * KS + KS - 1 inside the 32-wide stage).
template <Layout L, int KS>
__device__ __forceinline__ void fetch_slab(const char* tile, int t, int ps, float (&v)[8][KS]) {
    static_assert(KS == 1 || KS == 2 || KS == 4, "k-step must be 1, 2 or 4");
    if (L == Layout::RowMajor) {
        const int k = ps * KS;
        const int off = (((k >> 2) ^ (t & 7)) << 4) + ((k & 3) << 2);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
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
            const char* row = tile + (ps * KS + kk) * 512 + t * 16;
            const float4 lo = *reinterpret_cast<const float4*>(row);
            const float4 hi = *reinterpret_cast<const float4*>(row + 256);
            v[0][kk] = lo.x; v[1][kk] = lo.y; v[2][kk] = lo.z; v[3][kk] = lo.w;
            v[4][kk] = hi.x; v[5][kk] = hi.y; v[6][kk] = hi.z; v[7][kk] = hi.w;
        }
    }
}

struct TileCoord {
    int g, m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(const TileParams& P, long long tile) {
    TileCoord c;
    const int per_group = P.tiles_m * P.tiles_n;
    c.g = static_cast<int>(tile / per_group);
    const int r = static_cast<int>(tile - static_cast<long long>(c.g) * per_group);
    c.m0 = (r % P.tiles_m) * kTileM;
    c.n0 = (r / P.tiles_m) * kTileN;
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

template <class Op>
struct TileSmem {
    static constexpr int kStage = (Op::NUM_A + 1) * kOperandTileBytes;
    static constexpr int kTotal = kStages * kStage + 1024 /*alignment slack*/ + 64 /*barriers*/;
};

template <class Op>
__global__ void __launch_bounds__(kThreads, 1)
tile_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
            const __grid_constant__ CUtensorMap map_b, const TileParams P) {
    constexpr int NA = Op::NUM_A;
    constexpr int NF = Op::NF;
    constexpr int NI = Op::NI;
    constexpr int NIA = NI > 0 ? NI : 1;
    constexpr int STAGE = TileSmem<Op>::kStage;

    extern __shared__ char smem_raw[];
    char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * STAGE);

    const int tid = threadIdx.x;
    const int tn = tid & 15;
    const int tm = tid >> 4;
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
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // producer side (thread 0): fill stage `ls % kStages` with the operands of iteration `it`
    auto issue = [&](long long it, int ls) {
        const long long tile = it / KT;
        const int kt = static_cast<int>(it - tile * KT);
        const TileCoord tc = tile_coord(P, tile);
        char* st = smem + (ls % kStages) * STAGE;
        uint64_t* bar = &full[ls % kStages];
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
            c2 = tc.g;
            if (P.b_row_coord == 2) { int t = c1; c1 = c2; c2 = t; }
            tma_load_3d(st + NA * kOperandTileBytes, &map_b, bar, c0, c1, c2);
        }
    };

    if (tid == 0) {
        for (int s = 0; s < kStages - 1; ++s)
            if (it0 + s < it1) issue(it0 + s, s);
    }

    float accf[kRegM][kRegN][NF];
    int acci[kRegM][kRegN][NIA];
    float pres[kRegM][kRegN];
    TileCoord tc = {0, 0, 0};
    long long seg_begin = it0;
    const long long first_tile = it0 / KT;

    for (long long it = it0; it < it1; ++it) {
        const int ls = static_cast<int>(it - it0);
        const long long tile = it / KT;
        const int kt = static_cast<int>(it - tile * KT);
        if (it == it0 || kt == 0) {
            seg_begin = it;
            tc = tile_coord(P, tile);
#pragma unroll
            for (int i = 0; i < kRegM; ++i)
#pragma unroll
                for (int j = 0; j < kRegN; ++j) {
                    Op::init(accf[i][j], acci[i][j]);
                    if (Op::HAS_P) {
                        const int m = tc.m0 + own_index<Op::LA>(tm, i);
                        const int n = tc.n0 + own_index<Op::LB>(tn, j);
                        pres[i][j] = (m < P.M && n < P.N) ? Op::load_pres(P, m, n, tc.g) : 0.0f;
                    } else {
                        pres[i][j] = 0.0f;
                    }
                }
        }

        if (!mbar_wait_bounded(&full[ls % kStages], (ls / kStages) & 1)) {
            atomicExch(P.status, static_cast<int>(kDeviceTimeout));
            return;
        }
        __syncthreads();  // every warp is done with the stage that is refilled next
        if (tid == 0 && it + (kStages - 1) < it1) issue(it + (kStages - 1), ls + (kStages - 1));

        const char* sa0 = smem + (ls % kStages) * STAGE;
        const char* sa1 = sa0 + (NA == 2 ? kOperandTileBytes : 0);
        const char* sb = sa0 + NA * kOperandTileBytes;
        // The k-groups of a stage are walked in a rolled loop so that the loop body (64 outputs x KS k x
        // a few FP32 instructions) stays resident in the instruction cache.  Threads with tn >= 8 visit
        // each pair of neighbouring k-groups in swapped order (KS < 4): with the 128-byte swizzle that
        // makes the narrower shared-memory reads of a RowMajor B tile bank-conflict free.  The order in
        // which a thread visits k does not matter to any op (sums, exact min / max, 4-channel groups).
        constexpr int KS = Op::KSTEP;
        const int perm = (KS < 4) ? (tn >> 3) : 0;
#pragma unroll 1
        for (int ks = 0; ks < kTileK / KS; ++ks) {
            const int ps = ks ^ perm;
            float a0[8][KS], a1[8][KS], b[8][KS];
            fetch_slab<Op::LA, KS>(sa0, tm, ps, a0);
            if (NA == 2) fetch_slab<Op::LA, KS>(sa1, tm, ps, a1);
            fetch_slab<Op::LB, KS>(sb, tn, ps, b);
            const int chunk = kt * (kTileK / 4) + ((ps * KS) >> 2);
#pragma unroll
            for (int i = 0; i < kRegM; ++i)
#pragma unroll
                for (int j = 0; j < kRegN; ++j)
                    Op::template update<KS>(accf[i][j], acci[i][j], pres[i][j], a0[i], NA == 2 ? a1[i] : a0[i], b[j],
                                            chunk, i + j, P);
        }

        if (kt == KT - 1 || it == it1 - 1) {
            const bool whole = (seg_begin == tile * KT) && (kt == KT - 1);
            if (whole) {
#pragma unroll
                for (int i = 0; i < kRegM; ++i)
#pragma unroll
                    for (int j = 0; j < kRegN; ++j) {
                        const int m = tc.m0 + own_index<Op::LA>(tm, i);
                        const int n = tc.n0 + own_index<Op::LB>(tn, j);
                        if (m < P.M && n < P.N) Op::finalize(accf[i][j], acci[i][j], pres[i][j], m, n, tc.g, P);
                    }
            } else {
                const int slot = (tile == first_tile) ? 0 : 1;
                float* dst = P.partials +
                             (static_cast<size_t>(blockIdx.x) * 2 + slot) * (size_t)(NF + NI) * kTileElems;
#pragma unroll
                for (int i = 0; i < kRegM; ++i)
#pragma unroll
                    for (int j = 0; j < kRegN; ++j) {
                        const int e = (i * kRegN + j) * kThreads + tid;
#pragma unroll
                        for (int a = 0; a < NF; ++a) dst[a * kTileElems + e] = accf[i][j][a];
#pragma unroll
                        for (int a = 0; a < NI; ++a) dst[(NF + a) * kTileElems + e] = __int_as_float(acci[i][j][a]);
                    }
            }
        }
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
// finalises it.  Launched with one CTA per tile and the grid size of the main kernel as an argument;
// CTAs of unshared tiles return at once.
template <class Op>
__global__ void __launch_bounds__(kThreads)
tile_fixup_kernel(const TileParams P, const int main_grid) {
    constexpr int NF = Op::NF;
    constexpr int NI = Op::NI;
    constexpr int NIA = NI > 0 ? NI : 1;
    const long long tile = blockIdx.x;
    const int KT = P.kt;
    const long long t0 = tile * KT, t1 = t0 + KT;
    // CTA whose range contains iteration t0
    int c = static_cast<int>(((t0 + 1) * main_grid - 1) / P.total_iters);
    if (range_begin(P.total_iters, main_grid, c + 1) >= t1) return;  // owned whole by one CTA

    const int tid = threadIdx.x;
    const int tn = tid & 15;
    const int tm = tid >> 4;
    const TileCoord tc = tile_coord(P, tile);
    float accf[kRegM][kRegN][NF];
    int acci[kRegM][kRegN][NIA];
#pragma unroll
    for (int i = 0; i < kRegM; ++i)
#pragma unroll
        for (int j = 0; j < kRegN; ++j) Op::init(accf[i][j], acci[i][j]);

    for (; c < main_grid; ++c) {
        const long long b0 = range_begin(P.total_iters, main_grid, c);
        const long long b1 = range_begin(P.total_iters, main_grid, c + 1);
        if (b0 >= t1) break;
        if (b1 <= b0) continue;
        const int slot = (b0 / KT == tile) ? 0 : 1;
        const float* src = P.partials + (static_cast<size_t>(c) * 2 + slot) * (size_t)(NF + NI) * kTileElems;
#pragma unroll
        for (int i = 0; i < kRegM; ++i)
#pragma unroll
            for (int j = 0; j < kRegN; ++j) {
                const int e = (i * kRegN + j) * kThreads + tid;
                float pf[NF];
                int pn[NIA];
#pragma unroll
                for (int a = 0; a < NF; ++a) pf[a] = src[a * kTileElems + e];
#pragma unroll
                for (int a = 0; a < NI; ++a) pn[a] = __float_as_int(src[(NF + a) * kTileElems + e]);
                Op::combine(accf[i][j], acci[i][j], pf, pn);
            }
    }
#pragma unroll
    for (int i = 0; i < kRegM; ++i)
#pragma unroll
        for (int j = 0; j < kRegN; ++j) {
            const int m = tc.m0 + own_index<Op::LA>(tm, i);
            const int n = tc.n0 + own_index<Op::LB>(tn, j);
            if (m < P.M && n < P.N) {
                const float pr = Op::HAS_P ? Op::load_pres(P, m, n, tc.g) : 0.0f;
                Op::finalize(accf[i][j], acci[i][j], pr, m, n, tc.g, P);
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
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tile_kernel<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return cuda_status(e);
        configured[dev] = true;
    }
    tile_kernel<Op><<<L.grid, kThreads, SMEM, stream>>>(L.map_a0, L.map_a1, L.map_b, L.params);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_status(e);
    count_launches(1);
    const long long tiles = L.params.total_iters / L.params.kt;
    // a tile can only be shared when the ranges do not fall on tile boundaries
    if (L.params.total_iters % L.grid != 0 || (L.params.total_iters / L.grid) % L.params.kt != 0) {
        tile_fixup_kernel<Op><<<static_cast<unsigned>(tiles), kThreads, 0, stream>>>(L.params, L.grid);
        e = cudaGetLastError();
        count_launches(1);
    }
    return cuda_status(e);
}

}  // namespace ldn
