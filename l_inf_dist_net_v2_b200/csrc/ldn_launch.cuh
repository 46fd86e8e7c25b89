// Non-template launch entry points of the tile-engine instantiations (one translation unit per family
// so that they compile in parallel).
#pragma once
#include "ldn_tile.cuh"

namespace ldn {

enum class FwdKind { PowInt, PowGen, PowNorm, Inf, InfPos, Bound, BoundPosLower, BoundPosUpper, BoundPosBoth };
constexpr int kBoundBothMaxStages = 65534;  // 16 bits per stage id (FwdBoundBoth)

// number of accumulator arrays (float + int) an op keeps per output: sizes the stream-K scratch
inline int fwd_acc_arrays(FwdKind k) {
    switch (k) {
        case FwdKind::InfPos: return 3;
        case FwdKind::Bound: return 2;
        case FwdKind::BoundPosLower: return 3;
        case FwdKind::BoundPosUpper: return 3;
        case FwdKind::BoundPosBoth: return 5;
        default: return 1;
    }
}

// tile width and resident CTAs per SM of the kernel a launch function will pick
struct OpGeom {
    int tile_n;
    int ctas_per_sm;
};
template <class Op>
constexpr OpGeom geom_of() {
    return OpGeom{16 * Op::REG_N, Op::CTAS_PER_SM};
}
OpGeom fwd_pow_geom(FwdKind kind, int ip);
OpGeom fwd_inf_geom(FwdKind kind);
OpGeom bwd_fused_geom(int iq);
OpGeom bwd_x_geom(int iq);
OpGeom bwd_w_geom(int iq);

// Forward ops that also exist with a k-major A operand (inputs with HW > 1 read in place) and with 64- / 32-wide
// tiles: PowInt with ip == 8, PowGen, PowNorm, Inf, InfPos.  reg_n = 8, 4 or 2 (tile width 16 * reg_n).
inline bool fwd_variant_supported(FwdKind kind, int ip) {
    return (kind == FwdKind::PowInt && ip == 8) || kind == FwdKind::PowGen || kind == FwdKind::PowNorm ||
           kind == FwdKind::Inf || kind == FwdKind::InfPos;
}
int launch_fwd_variant_row(FwdKind kind, int reg_n, const TileLaunch& L, cudaStream_t st);  // row-major A, reg_n 4 or 2
int launch_fwd_variant_k(FwdKind kind, int reg_n, const TileLaunch& L, cudaStream_t st);    // k-major A, reg_n 8, 4, 2

int launch_fwd_pow(FwdKind kind, int ip, const TileLaunch& L, cudaStream_t st);   // PowInt (ip 1..8), PowGen, PowNorm
int launch_fwd_inf(FwdKind kind, const TileLaunch& L, cudaStream_t st);           // Inf, InfPos, Bound, BoundPos{Lower,Upper,Both}
// iq 0..8: integer p - 1; -1: general p with 1/y folded into the exponent offset; -2: general p, unfolded
int launch_bwd_x(int iq, const TileLaunch& L, cudaStream_t st);
int launch_bwd_w(int iq, const TileLaunch& L, cudaStream_t st);
int launch_bwd_fused(int iq, const TileLaunch& L, cudaStream_t st);             // iq 1..8, -1 or -2

}  // namespace ldn
