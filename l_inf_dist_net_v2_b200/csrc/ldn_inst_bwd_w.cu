#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
OpGeom bwd_w_geom(int iq) { return iq >= 0 ? geom_of<BwdPowInt<7, true>>() : geom_of<BwdPowGen<true, true>>(); }

int launch_bwd_w(int iq, const TileLaunch& L, cudaStream_t st) {
    switch (iq) {
        case 0: return launch_tile<BwdPowInt<0, true>>(L, st);
        case 1: return launch_tile<BwdPowInt<1, true>>(L, st);
        case 2: return launch_tile<BwdPowInt<2, true>>(L, st);
        case 3: return launch_tile<BwdPowInt<3, true>>(L, st);
        case 4: return launch_tile<BwdPowInt<4, true>>(L, st);
        case 5: return launch_tile<BwdPowInt<5, true>>(L, st);
        case 6: return launch_tile<BwdPowInt<6, true>>(L, st);
        case 7: return launch_tile<BwdPowInt<7, true>>(L, st);
        case 8: return launch_tile<BwdPowInt<8, true>>(L, st);
        case -2: return launch_tile<BwdPowGen<true, false>>(L, st);
        default: return launch_tile<BwdPowGen<true, true>>(L, st);
    }
}
}  // namespace ldn
