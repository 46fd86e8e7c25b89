#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
OpGeom fwd_pow_geom(FwdKind kind, int) {
    if (kind == FwdKind::PowNorm) return geom_of<FwdPowNorm>();
    if (kind == FwdKind::PowGen) return geom_of<FwdPowGen>();
    return geom_of<FwdPowInt<8>>();
}

int launch_fwd_pow(FwdKind kind, int ip, const TileLaunch& L, cudaStream_t st) {
    if (kind == FwdKind::PowGen) return launch_tile<FwdPowGen>(L, st);
    if (kind == FwdKind::PowNorm) return launch_tile<FwdPowNorm>(L, st);
    if (kind != FwdKind::PowInt) return kBadArgument;
    switch (ip) {
        case 1: return launch_tile<FwdPowInt<1>>(L, st);
        case 2: return launch_tile<FwdPowInt<2>>(L, st);
        case 3: return launch_tile<FwdPowInt<3>>(L, st);
        case 4: return launch_tile<FwdPowInt<4>>(L, st);
        case 5: return launch_tile<FwdPowInt<5>>(L, st);
        case 6: return launch_tile<FwdPowInt<6>>(L, st);
        case 7: return launch_tile<FwdPowInt<7>>(L, st);
        case 8: return launch_tile<FwdPowInt<8>>(L, st);
        default: return kBadArgument;
    }
}
}  // namespace ldn
