#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
OpGeom bwd_x_geom(int iq) { return iq >= 0 ? geom_of<BwdPowInt<7, false>>() : geom_of<BwdPowGen<false, true>>(); }

int launch_bwd_x(int iq, const TileLaunch& L, cudaStream_t st) {
    switch (iq) {
        case 0: return launch_tile<BwdPowInt<0, false>>(L, st);
        case 1: return launch_tile<BwdPowInt<1, false>>(L, st);
        case 2: return launch_tile<BwdPowInt<2, false>>(L, st);
        case 3: return launch_tile<BwdPowInt<3, false>>(L, st);
        case 4: return launch_tile<BwdPowInt<4, false>>(L, st);
        case 5: return launch_tile<BwdPowInt<5, false>>(L, st);
        case 6: return launch_tile<BwdPowInt<6, false>>(L, st);
        case 7: return launch_tile<BwdPowInt<7, false>>(L, st);
        case 8: return launch_tile<BwdPowInt<8, false>>(L, st);
        case -2: return launch_tile<BwdPowGen<false, false>>(L, st);
        default: return launch_tile<BwdPowGen<false, true>>(L, st);
    }
}
}  // namespace ldn
