// Memory-bound helper kernels: canonical operand copies, backward coefficients, p = inf scatters.
#pragma once
#include "ldn_common.cuh"

namespace ldn {

struct Shape {
    int B, CO, CI, G, HW;
    int CIg, COg;
    long long M;  // B * HW
    // A range of output channels of a wider layer (G == 1 only): grad_output / output rows are co_src channels long and
    // this problem's channel o is their channel co_off + o.  co_src == CO, co_off == 0: the whole layer.
    int co_src, co_off;
};

// xc[g][m][pitch] <- x[((b G + g) CIg + c) HW + hw],  m = b HW + hw
int launch_canon_x(const float* x, float* xc, const Shape& s, int pitch, cudaStream_t st);
// same for a (lower, upper) pair; elements with lower > upper are replaced by their midpoint
int launch_canon_bounds(const float* xl, const float* xu, float* lc, float* uc, const Shape& s, int pitch,
                        cudaStream_t st);
// wc[g][o][pitch] <- w[(g COg + o) CIg + c]
int launch_canon_w(const float* w, float* wc, const Shape& s, int pitch, cudaStream_t st);
// integer p - 1 = iq:  coef[g][m][pitch] <- go / y^iq   (go, y in output layout).  flag (may be null): set to 1 when
// some y^-iq is outside the range in which that coefficient times |t|^iq is accurate (cleared by the caller before).
int launch_coef_int(const float* go, const float* y, float* coef, const Shape& s, int pitch, int iq, int* flag,
                    cudaStream_t st);
// general p: rinv[g][rows_pad][pitch] <- -q lg2 y (fold: the exponent offset of (|t| / y)^q) or 1 / y,
// gcp[g][rows_pad][pitch] <- go; rows beyond M and columns beyond CO / G are padding (offset -1e30 resp. factor 0,
// gradient factor 0)
int launch_coef_gen(const float* go, const float* y, float* rinv, float* gcp, const Shape& s, int pitch,
                    long long rows_pad, float q, bool fold, const int* gate,
                    cudaStream_t st);  // gate (may be null): the kernel does nothing unless *gate != 0

// Second step of the forward kernels that save an index: `pos` holds, per output, the id of the 32-channel
// stage in which the extremum was first reached (or -1); replace it by the channel index | flag.
//   mode 0: p = inf value y = max |a - b|, flag = (a - b < 0)          (a1 unused; none: 0)
//   mode 1: lower bound, y = -min(min(t1, t2)),  t1 = b - a0, t2 = a1 - b, flag = (t1 > t2)   (none: 0xffffffff)
//   mode 2: upper bound, y = max(max(t1, t2)), same flag                (none: 0)
// Operands are given as generic views (row / group strides in elements, reduction index contiguous).  With
// a_stride_k != 1 (mode 0 only) a0 is an input read in place: element (sample-group bg, position hw, channel k) at
// a0.ptr + bg * a0.stride_group + hw * a0.stride_row + k * a_stride_k.
int launch_rescan(int mode, Operand a0, Operand a1, Operand b, const float* y, int* pos, const Shape& s,
                  cudaStream_t st, long long a_stride_k);

// out[g * rows + r] = max_k |v[g][r][k]| for an operand view with `inner` reduction elements per row, stride_k apart
// (1: contiguous).  clear (may be null): a device word that the kernel resets to 0.
int launch_row_absmax(Operand v, long long rows, int inner, int groups, long long stride_k, float* out, int* clear,
                      cudaStream_t st);

// grad_weight of the fused backward: gw[i] = -sum_t part[t * count + i], t < tiles
// gate (may be null): the kernel runs only if (*gate != 0) == run_if_nonzero
int launch_side_reduce(const float* part, float* gw, long long count, int tiles, bool accumulate, const int* gate,
                       bool run_if_nonzero, cudaStream_t st);

// p = inf backward: gx[b, idx] += v, gw[o, idx] -= v with v = pos >= 0 ? go : -go.  gx / gw may be null.
int launch_inf_scatter(const float* go, const int* pos, float* gx, float* gw, const Shape& s, cudaStream_t st);
// interval-bound backward (see ldn_bound_inf_dist_backward_input_weight).  gw may be null.
int launch_bound_scatter(const float* gol, const float* gou, const int* posl, const int* posu, float* gxl, float* gxu,
                         float* gw, const Shape& s, cudaStream_t st);

}  // namespace ldn
