#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
int launch_fwd_inf(FwdKind kind, const TileLaunch& L, cudaStream_t st) {
    switch (kind) {
        case FwdKind::Inf: return launch_tile<FwdInf<false>>(L, st);
        case FwdKind::InfPos: return launch_tile<FwdInf<true>>(L, st);
        case FwdKind::Bound: return launch_tile<FwdBound>(L, st);
        case FwdKind::BoundPosLower: return launch_tile<FwdBoundPos<false>>(L, st);
        case FwdKind::BoundPosUpper: return launch_tile<FwdBoundPos<true>>(L, st);
        default: return kBadArgument;
    }
}
}  // namespace ldn
