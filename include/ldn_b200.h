/*
 * C ABI of libldn_b200.so -- sm_100a kernels for the L_p-distance operator
 *     y[b, o, hw] = ( sum_c |x[b, g, c, hw] - w[g, o, c]|^p )^(1/p)
 * of zbh2047/L_inf-dist-net-v2, its backward pass and its p = inf interval-bound variant.
 *
 * Each entry point replaces one static launcher of the reference's core/cuda/norm_dist.h (cited per
 * function) as it is reached through the pybind wrappers of core/cuda/norm_dist.cpp:40-189.  Argument
 * order follows those launchers; two things are added: the CUDA stream to launch on (the reference
 * uses the legacy default stream) and an int return value (0 = success, see ldn_status_string).
 *
 * Conventions (identical to the reference):
 *   - all pointers are device pointers to contiguous fp32 (int32 for pos arrays) on the current device;
 *   - x[B, CI, HW], w[CO, CI/G], y[B, CO, HW]; element offsets
 *       x: ((b*G + g)*(CI/G) + c)*HW + hw,  w: (g*(CO/G) + o)*(CI/G) + c,  y: ((b*G + g)*(CO/G) + o)*HW + hw;
 *   - the caller allocates every output; outputs need not be zeroed, the library zero-fills wherever
 *     it accumulates;
 *   - pos arrays have the layout of y; bit 31 is a flag, bits 0..30 the channel index in the group.
 * Sizes are 32-bit per dimension but all offsets are computed in 64 bits.  An empty batch (B == 0 or HW == 0) is a
 * successful no-op: nothing is launched, a weight gradient is set to zero.
 *
 * Scratch: kernels that need intermediate device memory take it from a per-(device, stream) arena that
 * the library allocates on first use and grows on demand (cudaMalloc; a growth synchronises the stream and is
 * refused with status 6 while the stream is being captured, see ldn_reserve_scratch).
 * Calls issued on the same stream may follow each other freely; the same stream must not be used from
 * two host threads at once.
 */
#ifndef LDN_B200_H
#define LDN_B200_H

#if defined(__GNUC__)
#define LDN_API __attribute__((visibility("default")))
#else
#define LDN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ldn_stream_t; /* == cudaStream_t */

/* Human-readable text for a status code returned by any function below. */
LDN_API const char* ldn_status_string(int status);

/* Library / build identification: "ldn_b200 <version> sm_100a". */
LDN_API const char* ldn_version(void);

/*
 * Copies the device status word of the stream's arena to the host, waits for the stream, clears the
 * word and returns it (0 when every kernel so far completed normally; 4 when a bounded wait inside a
 * kernel gave up).  No counterpart in the reference, which never checks launch results.
 */
LDN_API int ldn_check_status(ldn_stream_t stream);

/*
 * Releases every scratch arena of the current device (synchronises the device).  CUDA graphs that captured calls of
 * this library on the device refer to the released blocks: do not replay them afterwards.
 */
LDN_API int ldn_release_scratch(void);

/*
 * Makes the scratch arena of (current device, stream) at least `bytes` large now, so that later calls on the stream
 * find it large enough (no counterpart in the reference).  Scratch cannot grow while the stream is being captured
 * into a CUDA graph -- a call that would need to returns status 6 -- so before a capture either run the same calls
 * once eagerly or reserve here.  Once a capture has used an arena, a later growth keeps the earlier blocks until
 * ldn_release_scratch, so graphs captured before stay valid.
 */
LDN_API int ldn_reserve_scratch(ldn_stream_t stream, unsigned long long bytes);

/*
 * Test hook: cap the number of persistent CTAs of the tile kernels (0 = one per SM).  Lets tests force
 * output tiles to be shared between CTAs on small problems.
 */
LDN_API void ldn_set_max_ctas(int max_ctas);

/*
 * Test hook: ldn_bound_inf_dist_forward computes both bounds and both indices in one pass when the reduction has at
 * most 65534 stages of 32 channels (two 16-bit stage ids per output), else in one pass per bound.  This lowers that
 * limit (0: always two passes; a negative value restores the default), so that tests reach the two-pass kernels.
 */
LDN_API void ldn_set_bound_one_pass_limit(int stages);

/*
 * Scratch limit of the fused finite-p backward (bytes; 0 restores the default of 1 GiB).  The kernel keeps one
 * copy of grad_weight per 128 rows of the batch; a batch that would need more than the limit is processed in
 * chunks of whole samples whose weight gradients are added up.  No counterpart in the reference.
 */
LDN_API void ldn_set_fused_scratch_limit(unsigned long long bytes);

/*
 * Number of kernels this library has launched in the calling process so far (all devices, all streams).
 * No counterpart in the reference.
 */
LDN_API unsigned long long ldn_kernel_launches(void);

/*
 * Per-kernel timing (no counterpart in the reference): while enabled, every launch of a tile kernel is bracketed by
 * a CUDA-event pair on its stream; ldn_last_tile_kernel_ms waits for the latest pair and returns the duration of that
 * one kernel in milliseconds (-1 if nothing was recorded).  One pair per process: use from one thread, one device.
 */
LDN_API void ldn_enable_kernel_timing(int enabled);
LDN_API float ldn_last_tile_kernel_ms(void);

/*
 * Tracing hook (no counterpart in the reference): while a non-null device buffer is set, every CTA of every
 * tile-engine launch writes four 64-bit words at buffer[4 * cta]: SM id, start and end time (globaltimer, ns)
 * and its number of k-steps.  The buffer must hold 4 * (number of SMs) words; pass NULL to switch it off.
 */
LDN_API void ldn_set_trace_buffer(unsigned long long* device_buffer);

/*
 * Training-mode MeanShift of a fully connected layer in one kernel (the reference composes it from torch operators,
 * core/modules/basic_modules.py:104-135): x and out are [B][C] row-major; mean[c] = sum_b x[b][c] / B;
 * out = x - mean; if running_mean is not NULL, running_mean = running_mean * (1 - momentum) + momentum * mean;
 * if mean_out is not NULL it receives the batch mean.  out may alias x.  With running_mean = NULL the same call is
 * the backward pass (grad_in = grad_out - mean over the batch of grad_out).  Deterministic.
 */
LDN_API int ldn_mean_shift_rows(const float* x, int B, int C, float* running_mean, float momentum, float* out,
                        float* mean_out, ldn_stream_t stream);

/*
 * Pipe-throughput probe for roofline denominators (no counterpart in the reference).  kind 0 runs a loop
 * of independent FFMA chains, kind 2 the same chains issued as packed fma.rn.f32x2, kind 1 a loop of
 * independent ex2(lg2(x)) chains, kind 3 eight such MUFU chains beside eight packed-FMA chains (16 FMAs per step;
 * *lane_ops then counts the MUFU operations only), `iters` iterations, on
 * 8 CTAs of 256 threads per SM.  *lane_ops receives the number of lane operations the launch executes
 * (FFMAs, respectively MUFU operations); the caller times the launch.  sink: one device float.
 * kinds 4 and 5 run the per-pair instruction stream of the general-p kernels on register operands (4: the fused
 * backward, 5: the sum pass of the forward; no shared memory, 4 CTAs per SM resident): *lane_ops then receives the
 * number of (input, weight) pairs evaluated, so that pairs / time is the rate that instruction mix can sustain.
 */
LDN_API int ldn_probe_pipe(int kind, int iters, float* sink, unsigned long long* lane_ops, ldn_stream_t stream);

/*
 * Parameter updates over a list of tensors in one kernel (the reference uses torch.optim.Adam with betas = (0.9, 0.99),
 * eps = 1e-10, main.py:388-392; these follow torch.optim's update rules).  params / grads / state arrays are HOST
 * arrays of `count` device pointers, sizes[t] the element count of tensor t; every gradient is multiplied by
 * grad_scale first (1 / world size after a summing all-reduce, else 1).
 *   ldn_adam_update: m = m + (g - m)(1 - beta1); v = v beta2 + (1 - beta2) g g;
 *                    p = p - lr / (1 - beta1^step) * m / (sqrt(v) / sqrt(1 - beta2^step) + eps);   step counts from 1.
 *   ldn_sgd_update:  g += weight_decay p; with momentum != 0: buf = first_step ? g : buf momentum + (1 - dampening) g,
 *                    g = nesterov ? g + momentum buf : buf;  p = p - lr g.   momentum_buf may be NULL when momentum == 0.
 */
LDN_API int ldn_adam_update(int count, float* const* params, const float* const* grads, float* const* exp_avg,
                            float* const* exp_avg_sq, const long long* sizes, float lr, float beta1, float beta2,
                            float eps, int step, float grad_scale, ldn_stream_t stream);
/* ldn_adam_update with the step count t (>= 1, as a float) read from device memory at kernel time, so that the launch
 * can be recorded in a CUDA graph and replayed while the caller advances *step_device on the stream. */
LDN_API int ldn_adam_update_device_step(int count, float* const* params, const float* const* grads,
                                        float* const* exp_avg, float* const* exp_avg_sq, const long long* sizes, float lr,
                                        float beta1, float beta2, float eps, const float* step_device, float grad_scale,
                                        ldn_stream_t stream);
LDN_API int ldn_sgd_update(int count, float* const* params, const float* const* grads, float* const* momentum_buf,
                           const long long* sizes, float lr, float momentum, float dampening, float weight_decay,
                           int nesterov, int first_step, float grad_scale, ldn_stream_t stream);

/* ---- finite p ------------------------------------------------------------------------------- */

/*
 * Replaces norm_dist<ip>::forward_with_max(max = nullptr) for p <= 10 and norm_dist<ip>::forward for
 * p > 10 (core/cuda/norm_dist.h:5-8, selected in core/cuda/norm_dist.cpp:40-53).
 *   p <= 10: y = max(sum |t|^p, 1.175494351e-38)^(1/p);  p > 10: y = M (sum (|t|/M)^p + (1e-10/M)^p)^(1/p),
 *   M = max(1e-10, max |t|).  Requires p > 0 and finite.
 */
LDN_API int ldn_norm_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                          float* output, float p, ldn_stream_t stream);

/*
 * Replaces norm_dist<ip>::forward_with_max with a caller-supplied normaliser (core/cuda/norm_dist.h:7-8,
 * core/cuda/norm_dist.cpp:55-64): r = 1/max_output; y = (sum (|t| r)^p + (1e-10 r)^p)^(1/p) / r.
 */
LDN_API int ldn_norm_dist_forward_with_max(const float* input, const float* weight, const float* max_output,
                                   int B, int CO, int CI, int G, int HW, float* output, float p,
                                   ldn_stream_t stream);

/*
 * Replaces norm_dist<ip>::backward_input (core/cuda/norm_dist.h:9-10, core/cuda/norm_dist.cpp:66-77):
 *   grad_input[b, c] = sum_o grad_output * sgn(t) * (|t| / output)^(p-1),  sgn(t) = +1 for t >= 0.
 */
LDN_API int ldn_norm_dist_backward_input(const float* grad_output, const float* input, const float* weight,
                                 const float* output, int B, int CO, int CI, int G, int HW,
                                 float* grad_input, float p, ldn_stream_t stream);

/*
 * Replaces norm_dist<ip>::backward_input_weight (core/cuda/norm_dist.h:11-13, core/cuda/norm_dist.cpp:79-91):
 * grad_input as above and grad_weight[o, c] = -sum_{b,hw} of the same term.  grad_input may be NULL when
 * the caller does not need it (the reference always computes it).  Results are deterministic: no atomics.
 */
LDN_API int ldn_norm_dist_backward_input_weight(const float* grad_output, const float* input, const float* weight,
                                        const float* output, int B, int CO, int CI, int G, int HW,
                                        float* grad_input, float* grad_weight, float p, ldn_stream_t stream);

/*
 * ldn_norm_dist_backward_input_weight for a range of output channels [co_begin, co_begin + co_count) of an ungrouped
 * layer (no counterpart in the reference): grad_output and output are the whole layer's (B, CO, HW) arrays, weight and
 * grad_weight the whole (CO, CI) arrays; rows co_begin.. of grad_weight are written, and grad_input receives the
 * range's contribution -- overwritten, or added to what is there when accumulate_input != 0.  Calling it for
 * consecutive ranges (the first with accumulate_input = 0) gives the full backward pass in pieces, so that a
 * data-parallel caller can start the all-reduce of one piece of grad_weight while the next piece is computed.
 */
LDN_API int ldn_norm_dist_backward_channels(const float* grad_output, const float* input, const float* weight,
                                            const float* output, int B, int CO, int CI, int HW, int co_begin,
                                            int co_count, float* grad_input, float* grad_weight, float p,
                                            int accumulate_input, ldn_stream_t stream);

/* ---- p = inf -------------------------------------------------------------------------------- */

/* Replaces inf_dist::forward_nograd (core/cuda/norm_dist.h:17-18): y = max(1e-10, max |t|). */
LDN_API int ldn_inf_dist_forward_nograd(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                                float* output, ldn_stream_t stream);

/*
 * Replaces inf_dist::forward (core/cuda/norm_dist.h:19-20): the value above and
 * pos = first channel attaining it | (t < 0 ? 1 << 31 : 0); pos = 0 when no |t| exceeds 1e-10.
 */
LDN_API int ldn_inf_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                         float* output, int* pos, ldn_stream_t stream);

/* Replaces inf_dist::backward_input (core/cuda/norm_dist.h:21-22): grad_input[b, idx] += (pos >= 0 ? g : -g). */
LDN_API int ldn_inf_dist_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                                float* grad_input, ldn_stream_t stream);

/*
 * Replaces inf_dist::backward_input_weight (core/cuda/norm_dist.h:23-24): as above plus
 * grad_weight[o, idx] -= (pos >= 0 ? g : -g).  grad_input may be NULL.
 */
LDN_API int ldn_inf_dist_backward_input_weight(const float* grad_output, const int* pos, int B, int CO, int CI, int G,
                                       int HW, float* grad_input, float* grad_weight, ldn_stream_t stream);

/* ---- p = inf interval bounds ----------------------------------------------------------------- */

/*
 * Replaces bound_inf_dist::forward_nograd (core/cuda/norm_dist.h:28-29).  With t1 = w - xL, t2 = xU - w
 * (elements with xL > xU are first replaced by their midpoint):
 *   yL = max(1e-10, max_c -min(t1, t2)),  yU = max(1e-10, max_c max(t1, t2)).
 */
LDN_API int ldn_bound_inf_dist_forward_nograd(const float* inputL, const float* inputU, const float* weight,
                                      int B, int CO, int CI, int G, int HW, float* outputL, float* outputU,
                                      ldn_stream_t stream);

/*
 * Replaces bound_inf_dist::forward (core/cuda/norm_dist.h:30-31): the bounds above plus posL / posU =
 * first channel attaining the bound | (t1 <= t2 ? 0 : 1 << 31); posL = 0xffffffff when the lower bound is
 * the 1e-10 floor (no gradient), posU = 0 when the upper bound is the floor.
 */
LDN_API int ldn_bound_inf_dist_forward(const float* inputL, const float* inputU, const float* weight,
                               int B, int CO, int CI, int G, int HW, float* outputL, float* outputU,
                               int* posL, int* posU, ldn_stream_t stream);

/* Replaces bound_inf_dist::backward_input (core/cuda/norm_dist.h:32-34). */
LDN_API int ldn_bound_inf_dist_backward_input(const float* grad_outputL, const float* grad_outputU,
                                      const int* posL, const int* posU, int B, int CO, int CI, int G, int HW,
                                      float* grad_inputL, float* grad_inputU, ldn_stream_t stream);

/* Replaces bound_inf_dist::backward_input_weight (core/cuda/norm_dist.h:35-37). */
LDN_API int ldn_bound_inf_dist_backward_input_weight(const float* grad_outputL, const float* grad_outputU,
                                             const int* posL, const int* posU, int B, int CO, int CI, int G,
                                             int HW, float* grad_inputL, float* grad_inputU, float* grad_weight,
                                             ldn_stream_t stream);

/* ---- eval-mode layer in one kernel -------------------------------------------------------------- */

/*
 * ldn_inf_dist_forward_nograd / ldn_bound_inf_dist_forward_nograd with the rest of an eval-mode layer folded into
 * the store (no counterpart in the reference, which runs them as separate elementwise passes,
 * core/modules/basic_modules.py:128-132 and core/modules/norm_dist.py:37-38): every stored value is
 *     (y - sub[o]) + add[o],   o = output channel in 0..CO-1,
 * with the same two roundings as the separate passes; sub (the MeanShift running mean) and add (the layer bias) are
 * device arrays of CO floats, either may be NULL.
 */
LDN_API int ldn_inf_dist_forward_nograd_shifted(const float* input, const float* weight, int B, int CO, int CI, int G,
                                                int HW, float* output, const float* sub, const float* add,
                                                ldn_stream_t stream);
LDN_API int ldn_bound_inf_dist_forward_nograd_shifted(const float* inputL, const float* inputU, const float* weight,
                                                      int B, int CO, int CI, int G, int HW, float* outputL,
                                                      float* outputU, const float* sub, const float* add,
                                                      ldn_stream_t stream);

/* ---- allocation-free variant ------------------------------------------------------------------ */

/*
 * Same result as ldn_inf_dist_forward_nograd, for callers that may not allocate device memory while they
 * run (a server whose memory was handed to its own pool at start-up, a runtime that forbids cudaMalloc after
 * initialisation, code that is about to record its launches).  This function has no counterpart in the
 * reference.  It calls no cudaMalloc / cudaFree and no allocating library routine: all scratch (operand
 * copies for layouts TMA cannot read directly, the partial results of output tiles shared between CTAs) lives
 * in one fixed 32 MiB array inside the library's device image, which every GPU that loads the library holds
 * until the process exits.
 *   - Limit: the call is refused with status 3 ("scratch memory could not be provided") before anything is
 *     launched when it would need more than the fixed array.  Fully connected inputs (HW == 1) with CI/G a
 *     multiple of 4 and 16-byte aligned pointers need 18.5 MiB whatever B, CI and CO are; other layouts add a
 *     padded copy of the input (4 * G * B * HW * ceil4(CI/G) bytes) and, if CI/G is not a multiple of 4 or the
 *     weight is misaligned, of the weight.
 *   - The first call on each device looks up the array's device address (with that device current); make
 *     that first call before any stream capture begins.
 *   - All calls on a device share the array and it keeps whatever the last call left there.  Nothing in it
 *     has to start at zero (every word is written before it is read within a call), but two calls whose
 *     kernels overlap on the GPU -- different streams, or different host threads -- race on it: issue these
 *     calls on one stream, or order them with events.
 *   - A bounded-wait timeout inside a kernel is recorded in the first word of the array, not in the stream's
 *     arena: read it with ldn_noalloc_check_status (ldn_check_status does not see it).
 */
LDN_API int ldn_inf_dist_forward_nograd_noalloc(const float* input, const float* weight, int B, int CO, int CI,
                                                int G, int HW, float* output, ldn_stream_t stream);

/*
 * Status of the allocation-free entry point on the current device (no counterpart in the reference): copies the
 * status word of the fixed array to the host in stream order, clears it, waits for the stream and returns it --
 * 0 when every allocation-free call issued on this stream so far ran to completion, 4 when a bounded wait inside
 * one of their kernels gave up (its output is then incomplete).  Allocates nothing either.
 */
LDN_API int ldn_noalloc_check_status(ldn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LDN_B200_H */
