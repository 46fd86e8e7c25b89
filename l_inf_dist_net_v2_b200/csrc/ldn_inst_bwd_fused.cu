#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
OpGeom bwd_fused_geom(int iq) { return iq >= 1 ? geom_of<BwdFusedInt<7>>() : geom_of<BwdFusedGen<true>>(); }

int launch_bwd_fused(int iq, const TileLaunch& L, cudaStream_t st) {
    switch (iq) {
        case 1: return launch_tile<BwdFusedInt<1>>(L, st);
        case 2: return launch_tile<BwdFusedInt<2>>(L, st);
        case 3: return launch_tile<BwdFusedInt<3>>(L, st);
        case 4: return launch_tile<BwdFusedInt<4>>(L, st);
        case 5: return launch_tile<BwdFusedInt<5>>(L, st);
        case 6: return launch_tile<BwdFusedInt<6>>(L, st);
        case 7: return launch_tile<BwdFusedInt<7>>(L, st);
        case 8: return launch_tile<BwdFusedInt<8>>(L, st);
        case -2: return launch_tile<BwdFusedGen<false>>(L, st);
        default: return launch_tile<BwdFusedGen<true>>(L, st);
    }
}
}  // namespace ldn
