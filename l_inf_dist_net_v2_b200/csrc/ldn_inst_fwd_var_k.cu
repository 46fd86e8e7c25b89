// Instances of the forward ops with a k-major A operand (inputs x[B, C, HW] with HW > 1 read in place).
#include "ldn_launch.cuh"
#include "ldn_ops.cuh"

namespace ldn {
namespace {
template <class Base>
int by_width(int reg_n, const TileLaunch& L, cudaStream_t st) {
    switch (reg_n) {
        case 8: return launch_tile<FwdVariant<Base, Layout::KMajor, 8>>(L, st);
        case 4: return launch_tile<FwdVariant<Base, Layout::KMajor, 4>>(L, st);
        case 2: return launch_tile<FwdVariant<Base, Layout::KMajor, 2>>(L, st);
        default: return kBadArgument;
    }
}
}  // namespace

int launch_fwd_variant_k(FwdKind kind, int reg_n, const TileLaunch& L, cudaStream_t st) {
    switch (kind) {
        case FwdKind::PowInt: return by_width<FwdPowInt<8>>(reg_n, L, st);
        case FwdKind::PowGen: return by_width<FwdPowGen>(reg_n, L, st);
        case FwdKind::PowNorm: return by_width<FwdPowNorm>(reg_n, L, st);
        // (scalar subtractions: with a k-major A operand two neighbouring k of a row are not neighbouring registers;
        // 64 x 576 x 1024 positions -> 128 outputs, value only: 0.58 -> 0.45 ms)
        case FwdKind::Inf: return by_width<FwdInf<false, false>>(reg_n, L, st);
        case FwdKind::InfPos: return by_width<FwdInf<true, false>>(reg_n, L, st);
        default: return kBadArgument;
    }
}
}  // namespace ldn
