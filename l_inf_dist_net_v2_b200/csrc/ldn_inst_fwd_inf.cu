#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
OpGeom fwd_inf_geom(FwdKind kind) {
    switch (kind) {
        case FwdKind::Inf: return geom_of<FwdInf<false>>();
        case FwdKind::InfPos: return geom_of<FwdInf<true>>();
        case FwdKind::Bound: return geom_of<FwdBound>();
        case FwdKind::BoundPosLower: return geom_of<FwdBoundPos<false>>();
        case FwdKind::BoundPosBoth: return geom_of<FwdBoundBoth>();
        default: return geom_of<FwdBoundPos<true>>();
    }
}

int launch_fwd_inf(FwdKind kind, const TileLaunch& L, cudaStream_t st) {
    switch (kind) {
        case FwdKind::Inf: return launch_tile<FwdInf<false>>(L, st);
        case FwdKind::InfPos: return launch_tile<FwdInf<true>>(L, st);
        case FwdKind::Bound: return launch_tile<FwdBound>(L, st);
        case FwdKind::BoundPosLower: return launch_tile<FwdBoundPos<false>>(L, st);
        case FwdKind::BoundPosUpper: return launch_tile<FwdBoundPos<true>>(L, st);
        case FwdKind::BoundPosBoth:
            static_assert(FwdBoundBoth::kMaxStages == kBoundBothMaxStages, "stage-id width");
            return launch_tile<FwdBoundBoth>(L, st);
        default: return kBadArgument;
    }
}
}  // namespace ldn
