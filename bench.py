#!/usr/bin/env python
"""Benchmark of the L_p-distance hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--p 8|37.5|inf] [--impl ours|reference|reference-cuda]

One "step" is one pass of the hot path over one batch: forward, grad_input and grad_weight of a single
norm_dist layer at the headline shape 512 x 3072 -> 5120 (per rank), p = 8 by default.  With N > 1 ranks
every rank works on its own batch (weak scaling, the batch dimension shards without communication) and
the step ends with the NCCL all-reduce (mean) of grad_weight, the one exchange data-parallel training
has.  The metric is pairs per second, a pair being one (sample, output, input) interaction; a step visits
every pair three times (forward, grad_input, grad_weight).

`value` is measured with all inputs resident in HBM; `e2e` goes through the public autograd API
(`l_inf_dist_net_v2_b200.norm_dist`) with the batch and the upstream gradient copied from pinned host
memory and the layer output copied back inside the timed region.  `--impl reference` times the
reference's CPU torch path (restated in oracle/torch_port.py) on the host cores on a bounded sample of
the same workload; `--impl reference-cuda` (extra) times the reference's own CUDA kernels recompiled for
sm_100a (oracle/_ref) on the same inputs.
"""
import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "norm_dist_fwd_bwd_pairs_per_s"
UNIT = "Gpair/s"
SM_LANES = 128  # FP32 lanes per SM
MUFU_LANES = 16

# algorithmic FP32 lane-instructions per pair (an FMA counts once): forward / grad_input / grad_weight
# fused backward (both gradients from one evaluation of the term): 7
SLOTS = {"8": (4, 6, 6), "inf": (2, None, None), "general": (6, 6, 6)}
SLOTS_FUSED = 7


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--p", default="8")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--ci", type=int, default=3072)
    ap.add_argument("--co", type=int, default=5120)
    ap.add_argument("--workload", default="layer", choices=["layer", "mlp-train", "mlp-certify", "hybrid-train", "hybrid-certify"],
                    help="layer: the headline single-layer step (default); mlp-train / mlp-certify: extra end-to-end "
                         "steps of a 6-layer distance MLP (depth 6, width 5120, 3x32x32 inputs, 10 classes); "
                         "hybrid-*: 5 distance layers (width 5120) + interval-bound linear head (hidden 512)")
    ap.add_argument("--certify-samples", type=int, default=50000)
    ap.add_argument("--reserve-sms", type=int, default=8,
                    help="N > 1, model steps: SMs the persistent distance kernels leave free while gradient collectives "
                         "are in flight; the collectives run in an NCCL group limited to as many CTAs (0: no limit)")
    ap.add_argument("--shard-updates", action="store_true",
                    help="N > 1, model training: reduce-scatter, update of the rank's 1/N slice, all-gather instead of "
                         "all-reduce and a full update on every rank (measured slower on 2 GPUs: the slice updates "
                         "share the reserved SMs with the collectives)")
    ap.add_argument("--bwd-chunks", type=int, default=1,
                    help="N > 1, layer step at finite p: ranges of output channels the backward pass is cut into, so that "
                         "each range's grad_weight all-reduce overlaps the next range's kernels (default 1: one all-reduce "
                         "after the backward pass; on 2 GPUs 2 / 4 / 8 ranges took 3.40 / 3.59 / 3.93 ms against 3.29)")
    ap.add_argument("--graph", action="store_true",
                    help="one GPU, model training workloads: record the whole step in a CUDA graph and replay it")
    ap.add_argument("--optimizer", default="adam", choices=["adam", "sgd"],
                    help="model training workloads: Adam as the reference driver uses it, or plain SGD lr 0.02")
    ap.add_argument("--model-global-batch", type=int, default=4096)
    ap.add_argument("--no-model", action="store_true", help="skip the model-level block of the default run")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long back-to-back block")
    ap.add_argument("--sustained-steps", type=int, default=1000)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-variants", action="store_true")
    return ap.parse_args()


def p_value(s):
    return math.inf if s in ("inf", "infinity") else float(s)


def p_family(p):
    if math.isinf(p):
        return "inf"
    if float(p).is_integer() and 1 <= p <= 8:
        return "int"
    return "general"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.samples = []
        self.proc = None
        self.thread = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            self.sel = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            self.sel = str(device_index)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.sel, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [s.strip() for s in line.split(",")]
            if len(parts) >= 7:
                self.samples.append((time.time(), parts))

    def mark(self):
        """Start of the timed region: only samples taken from here on are summarised (if there are any)."""
        self.t_mark = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = [p for (t, p) in self.samples if t >= getattr(self, "t_mark", 0.0)]
        scope = "timed region"
        if not window:
            window = [p for (_, p) in self.samples]
            scope = "warm-up and timed region (no sample fell inside the timed region)"
        self.scope = scope
        for s in window:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
                pw.append(float(s[2]))
            except ValueError:
                continue
            for n, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm),
                "scope": self.scope}


# ------------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------------
def make_host_inputs(args, rank):
    """Synthetic stand-in for a CIFAR-10 batch (3 x 32 x 32 images flattened to 3072 features in [0, 1]),
    N(0, 1) weights as the reference initialises them, N(0, 1) upstream gradient.  CPU generator: weights
    seed 0 on every rank, data seed = rank."""
    gw = torch.Generator().manual_seed(0)
    w = torch.randn(args.co, args.ci, generator=gw)
    gd = torch.Generator().manual_seed(1000 + rank)
    x = torch.rand(args.batch, args.ci, 1, generator=gd)
    g = torch.randn(args.batch, args.co, 1, generator=gd)
    return x, w, g


def event_ms_list(fn, steps, warmup, flush):
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def run_ours(args, rank, world, local_rank, comm_group=None):
    import torch.distributed as dist
    import l_inf_dist_net_v2_b200 as ldn
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    from l_inf_dist_net_v2_b200._lib import lib
    from l_inf_dist_net_v2_b200.parallel import allreduce_mean_

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    p = p_value(args.p)
    fam = p_family(p)
    B, CI, CO = args.batch, args.ci, args.co
    pairs = B * CI * CO
    xh, wh, gh = make_host_inputs(args, rank)
    xh, gh = xh.pin_memory(), gh.pin_memory()
    x, w, g = xh.to(dev), wh.to(dev), gh.to(dev)
    y = torch.empty(B, CO, 1, device=dev)
    pos = torch.empty(B, CO, 1, device=dev, dtype=torch.int32)
    gx = torch.empty_like(x)
    gw = torch.empty_like(w)
    yh = torch.empty(B, CO, 1).pin_memory()
    flush_buf = torch.empty(256 * 1024 * 1024 // 4, device=dev)

    def flush():
        flush_buf.zero_()

    def fwd(pp=p):
        if math.isinf(pp):
            C.inf_dist_forward(x, w, y, pos, 1)
        else:
            C.norm_dist_forward(x, w, y, 1, pp)

    def bwd_x(pp=p):
        if math.isinf(pp):
            C.inf_dist_backward_input(g, pos, gx, 1)
        else:
            C.norm_dist_backward_input(g, x, w, y, gx, 1, pp)

    def bwd_w(pp=p):
        if math.isinf(pp):
            C.inf_dist_backward_input_weight(g, pos, None, gw, 1)
        else:
            C.norm_dist_backward_input_weight(g, x, w, y, None, gw, 1, pp)

    def bwd(pp=p):
        if math.isinf(pp):
            C.inf_dist_backward_input_weight(g, pos, gx, gw, 1)
        else:
            C.norm_dist_backward_input_weight(g, x, w, y, gx, gw, 1, pp)

    # N > 1, finite p: the backward pass runs in ranges of output channels; the all-reduce of one range of grad_weight
    # (on the CTA-limited NCCL group, the distance kernels leaving that many SMs free meanwhile) overlaps the next
    # range's kernels, so only the last range's exchange is exposed.
    chunks = args.bwd_chunks if (world > 1 and not math.isinf(p)) else 1
    if CO % max(chunks, 1) != 0:
        chunks = 1
    sm_total = torch.cuda.get_device_properties(dev).multi_processor_count
    reserve = args.reserve_sms if (comm_group is not None and chunks > 1) else 0

    def step():
        fwd()
        if chunks <= 1:
            bwd()
            if world > 1:
                allreduce_mean_([gw])
            return
        per = CO // chunks
        works = []
        for ci in range(chunks):
            C.norm_dist_backward_channels(g, x, w, y, gx, gw, p, ci * per, per, ci > 0)
            works.append(dist.all_reduce(gw[ci * per:(ci + 1) * per], op=dist.ReduceOp.AVG,
                                         group=comm_group if ci + 1 < chunks else None, async_op=True))
            if reserve and ci == 0:
                lib.ldn_set_max_ctas(sm_total - reserve)
        if reserve:
            lib.ldn_set_max_ctas(0)
        for wk in works:
            wk.wait()

    # public-API step with host buffers
    w_param = w.clone().requires_grad_()
    x_dev = torch.empty_like(x)
    g_dev = torch.empty_like(g)

    # Input pipeline of the end-to-end run: every step's batch and upstream gradient come from pinned host
    # memory and its output goes back to the host; the copies run on their own streams, so the upload of step
    # i + 1 and the download of step i - 1 overlap the kernels of step i (double-buffered device tensors).
    x_buf = [torch.empty_like(x) for _ in range(2)]
    g_buf = [torch.empty_like(g) for _ in range(2)]
    y_keep = [None, None]
    h2d_stream, d2h_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    up_done = [torch.cuda.Event() for _ in range(2)]
    buf_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = torch.cuda.Event()

    def upload(i):
        b = i & 1
        with torch.cuda.stream(h2d_stream):
            h2d_stream.wait_event(buf_free[b])
            x_buf[b].copy_(xh, non_blocking=True)
            g_buf[b].copy_(gh, non_blocking=True)
            up_done[b].record(h2d_stream)

    def run_e2e(steps):
        main = torch.cuda.current_stream()
        for b in range(2):
            buf_free[b].record(main)
        upload(0)
        for i in range(steps):
            b = i & 1
            if i + 1 < steps:
                upload(i + 1)
            flush()
            main.wait_event(up_done[b])
            xin = x_buf[b].detach().requires_grad_()
            w_param.grad = None
            out = ldn.norm_dist(xin, w_param, p)
            out.backward(g_buf[b])
            if world > 1:
                allreduce_mean_([w_param.grad])
            buf_free[b].record(main)
            out_ready.record(main)
            y_keep[b] = out.detach()
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(out_ready)
                yh.copy_(y_keep[b], non_blocking=True)
        main.wait_stream(d2h_stream)
        main.wait_stream(h2d_stream)

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- timed region: device-resident ----------------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        flush()
        step()
    torch.cuda.synchronize()
    barrier()
    sampler.mark()
    launches0 = lib.ldn_kernel_launches()
    torch.cuda.synchronize()
    t_wall0 = time.perf_counter()
    ms = event_ms_list(step, args.steps, 0, flush)
    torch.cuda.synchronize()
    barrier()
    t_wall1 = time.perf_counter()
    launches = int(lib.ldn_kernel_launches() - launches0)
    clocks = sampler.stop()
    total_ms = sum(ms)
    # ---- timed region: end to end ----------------------------------------------------------------
    barrier()
    run_e2e(max(args.warmup, 3))
    torch.cuda.synchronize()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    run_e2e(args.steps)
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    total_e2e = ev0.elapsed_time(ev1)
    C.check_status()

    if world > 1:
        t = torch.tensor([total_ms, total_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, total_e2e = float(t[0]), float(t[1])

    # ---- the same step back to back for seconds: what the clocks settle at under a sustained load ---------------
    sustained = None
    if not args.no_sustained:
        s2 = ClockSampler(local_rank)
        s2.start()
        for _ in range(3):
            flush()
            step()
        torch.cuda.synchronize()
        barrier()
        s2.mark()
        ms_s = event_ms_list(step, args.sustained_steps, 0, flush)
        torch.cuda.synchronize()
        barrier()
        ck = s2.stop()
        tot = sum(ms_s)
        if world > 1:
            t = torch.tensor([tot], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            tot = float(t[0])
        n = args.sustained_steps
        tail = sorted(ms_s[n // 2:])
        sustained = {"steps": n, "seconds": round(tot * 1e-3, 3), "ms_per_step": round(tot / n, 4),
                     "ms_per_step_second_half_median": round(tail[len(tail) // 2], 4),
                     "value": round(world * pairs * n / (tot * 1e-3) / 1e9, 2), "unit": UNIT, "clocks": ck}

    model = None
    if not args.no_model:
        try:
            model = model_block(args, rank, world, local_rank, comm_group)
        except Exception as exc:  # the headline line must survive a failure here
            model = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            lib.ldn_set_max_ctas(0)
        C.check_status()

    if rank != 0:
        return None

    value = world * pairs * args.steps / (total_ms * 1e-3) / 1e9
    e2e_value = world * pairs * args.steps / (total_e2e * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"norm_dist layer fwd+bwd {B}x{CI}->{CO} per rank, p={args.p}, G=1, HW=1",
                   "p": args.p, "batch_per_rank": B, "in_features": CI, "out_features": CO,
                   "pairs_per_step_per_rank": pairs, "passes_per_pair": 3,
                   "exchange": ("none" if world == 1 else "NCCL all-reduce(mean) of grad_weight after the backward pass"
                                if chunks <= 1 else
                                f"NCCL all-reduce(mean) of grad_weight in {chunks} ranges of output channels, each started "
                                f"behind its range's backward kernels ({reserve} SMs left free meanwhile)"),
                   "l2": "256 MiB buffer overwritten before every timed step"},
        "samples_per_s": round(world * B * args.steps / (total_ms * 1e-3), 1),
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "ms_per_step": round(total_e2e / args.steps, 4),
                "h2d_bytes_per_step": xh.numel() * 4 + gh.numel() * 4, "d2h_bytes_per_step": yh.numel() * 4,
                "api": "l_inf_dist_net_v2_b200.norm_dist + autograd backward",
                "pipeline": "uploads / downloads on side streams, double-buffered; L2 flush inside the timed region"},
        "gpu_launches": launches,
        "clocks": clocks,
        "wall_s_timed_region": round(t_wall1 - t_wall0, 3),
    }

    # ---- per-kernel rooflines (rank 0) ------------------------------------------------------------
    props = torch.cuda.get_device_properties(dev)
    sms = props.multi_processor_count
    max_mhz = clocks.get("sm_max_mhz") or 1965.0
    sink = torch.zeros(64, device=dev)
    lane_ops = ctypes.c_ulonglong(0)

    def probe(kind, iters):
        def run():
            lib.ldn_probe_pipe(kind, iters, sink.data_ptr(), ctypes.byref(lane_ops),
                               torch.cuda.current_stream().cuda_stream)
        t = min(event_ms_list(run, 5, 2, lambda: None))
        return lane_ops.value / (t * 1e-3) / 1e12

    ffma_peak = probe(0, 4000)
    mufu_peak = probe(1, 1000)
    # what the general-p instruction streams sustain on register operands (Tpair/s): fused backward, forward sum
    mix_bwd_peak = probe(4, 500)
    mix_fwd_peak = probe(5, 500)
    nominal_fp32 = sms * SM_LANES * max_mhz * 1e6 / 1e12
    nominal_mufu = sms * MUFU_LANES * max_mhz * 1e6 / 1e12

    def kernel_rows(pp, label, steps):
        fam_ = p_family(pp)
        s_f, s_x, s_w = SLOTS["inf" if fam_ == "inf" else ("8" if fam_ == "int" else "general")]
        rows = []
        fwd(pp)
        todo = [("forward", lambda: fwd(pp), s_f), ("grad_input", lambda: bwd_x(pp), s_x),
                ("grad_weight", lambda: bwd_w(pp), s_w)]
        if fam_ != "inf":
            todo.append(("backward_fused", lambda: bwd(pp), SLOTS_FUSED))
        for name, fn, slots in todo:
            t = statistics.median(event_ms_list(fn, steps, 3, flush))
            row = {"p": label, "kernel": name, "ms": round(t, 4), "gpair_per_s": round(pairs / (t * 1e-3) / 1e9, 1)}
            # duration of the tile kernel alone (the call also runs coefficient / fix-up / reduction kernels):
            # CUDA events recorded by the library around that one launch, median of 5 calls
            lib.ldn_enable_kernel_timing(1)
            solo = []
            for _ in range(5):
                flush()
                fn()
                solo.append(lib.ldn_last_tile_kernel_ms())
            lib.ldn_enable_kernel_timing(0)
            t_tile = statistics.median(solo)
            # (a tile kernel is most of its call; anything far below that is not the kernel this row is about)
            if t_tile > 0.2 * t and not (fam_ == "inf" and name != "forward"):
                row["tile_kernel_ms"] = round(t_tile, 4)
            if fam_ == "inf" and name != "forward":
                # scatter kernels: HBM-bound.  bytes: g + pos reads, zero-fill of the gradient, one 8-byte
                # read-modify-write per scattered element
                nb = 8 * B * CO + 4 * (B * CI if name == "grad_input" else CO * CI) + 8 * B * CO
                row.update({"bound": "hbm", "bytes": nb, "gb_per_s": round(nb / (t * 1e-3) / 1e9, 1)})
            else:
                ach = slots * pairs / (t * 1e-3) / 1e12
                row.update({"bound": "fp32", "slots_per_pair": slots, "tlaneop_per_s": round(ach, 2),
                            "frac_of_ffma_probe": round(ach / ffma_peak, 3),
                            "frac_of_nominal": round(ach / nominal_fp32, 3)})
                if "tile_kernel_ms" in row:
                    ach_k = slots * pairs / (row["tile_kernel_ms"] * 1e-3) / 1e12
                    row.update({"tile_kernel_tlaneop_per_s": round(ach_k, 2),
                                "tile_kernel_frac_of_ffma_probe": round(ach_k / ffma_peak, 3)})
                if fam_ == "general" and name != "backward_fused":
                    mu = 2 * pairs / (t * 1e-3) / 1e12
                    row.update({"mufu_top_per_s": round(mu, 3), "frac_of_mufu_probe": round(mu / mufu_peak, 3)})
                if fam_ == "general" and "tile_kernel_ms" in row:
                    # the tile kernel against the register-only loop with the same per-pair instruction stream
                    mix = mix_fwd_peak if name == "forward" else mix_bwd_peak
                    row["tile_kernel_frac_of_mix_probe"] = round(
                        pairs / (row["tile_kernel_ms"] * 1e-3) / 1e12 / mix, 3)
            rows.append(row)
        return rows

    # DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) as captured with ncu: read from
    # profiles/dram_traffic.json, which names the capture command and the source revision; only valid for its shape
    ncu_traffic, traffic_source = {}, None
    try:
        tj = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
        if tj.get("shape") == [B, CI, CO]:
            ncu_traffic = tj.get("p", {}).get(args.p, {})
            traffic_source = f"profiles/dram_traffic.json ({tj.get('captured')}, source revision {tj.get('revision')})"
    except Exception:
        pass
    rows = kernel_rows(p, args.p, max(10, min(args.steps, 30)))
    in_step = [r for r in rows if r["kernel"] in (("forward", "grad_input", "grad_weight") if fam == "inf"
                                                 else ("forward", "backward_fused"))]
    dominant = max(in_step, key=lambda r: r["ms"])
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    if dominant["bound"] == "fp32":
        line["roofline"] = {
            "bound": "fp32", "kernel": f"{dominant['kernel']} (p={args.p})",
            "achieved": dominant.get("tile_kernel_tlaneop_per_s", dominant["tlaneop_per_s"]),
            "peak": round(ffma_peak, 2), "unit": "Tlaneop/s",
            "frac": dominant.get("tile_kernel_frac_of_ffma_probe", dominant["frac_of_ffma_probe"]),
            "kernel_ms": dominant.get("tile_kernel_ms"), "call_ms": dominant["ms"],
            "call_frac": dominant["frac_of_ffma_probe"],
            "note": "achieved / frac use the tile kernel's own duration (CUDA events around that launch); call_* "
                    "include the helper kernels of the same entry point; general p: frac_of_instruction_mix_probe "
                    "compares the kernel with a register-only loop of its MUFU + FMA instruction stream",
            "peak_source": "FFMA-loop probe measured in this run (MEASURED_PEAKS.json holds no FP32 figure)",
            "peak_nominal": round(nominal_fp32, 2), "frac_of_nominal": dominant["frac_of_nominal"],
            "slots_per_pair": dominant["slots_per_pair"], "ms": dominant["ms"],
            "frac_of_instruction_mix_probe": dominant.get("tile_kernel_frac_of_mix_probe"),
            "traffic": ncu_traffic.get(dominant["kernel"]), "traffic_unit": "bytes per launch (ncu)",
            "traffic_source": traffic_source,
            "algorithmic_bytes": (4 * (B * CO + B * CI + CO * CI) + 4 * (B * CI + CO * CI))
            if dominant["kernel"] == "backward_fused" else 4 * (B * CI + CO * CI + B * CO)}
    else:
        line["roofline"] = {
            "bound": "hbm", "kernel": f"{dominant['kernel']} (p={args.p})", "achieved": dominant["gb_per_s"],
            "peak": hbm_peak, "unit": "GB/s", "frac": round(dominant["gb_per_s"] / hbm_peak, 3),
            "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback 6650 GB/s", "ms": dominant["ms"],
            "traffic": None}
    if sustained is not None:
        # whole step (forward + both gradients) in algorithmic lane-instructions, at the clock that held
        fam_slots = {"int": 4 + SLOTS_FUSED, "general": 6 + SLOTS_FUSED, "inf": 2}[fam]
        ach = fam_slots * pairs / (sustained["ms_per_step"] * 1e-3) / 1e12
        mhz = sustained["clocks"].get("sm_mhz")
        sustained.update({"slots_per_pair_per_step": fam_slots, "step_tlaneop_per_s": round(ach, 2),
                          "frac_of_nominal_at_max_clock": round(ach / nominal_fp32, 3),
                          "frac_of_nominal_at_sampled_clock":
                              round(ach / (sms * SM_LANES * mhz * 1e6 / 1e12), 3) if mhz else None,
                          "ms_x_mhz": round(sustained["ms_per_step"] * mhz, 1) if mhz else None,
                          "ffma_probe_tlaneop_per_s": round(ffma_peak, 2),
                          "note": "the FFMA probe ran after this block at whatever clock the GPU then held; "
                                  "frac_of_nominal_at_sampled_clock uses the median SM clock sampled during this block"})
        line["sustained"] = sustained
    if model is not None:
        line["model"] = model
    line["kernels"] = rows
    line["probes"] = {"ffma_tlaneop_per_s": round(ffma_peak, 2), "mufu_top_per_s": round(mufu_peak, 3),
                      "general_p_mix_bwd_tpair_per_s": round(mix_bwd_peak, 3),
                      "general_p_mix_fwd_tpair_per_s": round(mix_fwd_peak, 3),
                      "nominal_fp32_tlaneop_per_s": round(nominal_fp32, 2),
                      "nominal_mufu_top_per_s": round(nominal_mufu, 3), "sms": sms}
    if world == 1 and not args.no_variants:
        extra = []
        for label in ("8", "inf", "37.5"):
            if label != args.p:
                extra += kernel_rows(p_value(label), label, 10)
        # p = inf certification kernels: value without indices, interval bounds at eps = 8/255
        eps = 8.0 / 255.0
        xl, xu = (x - eps).clamp(0, 1), (x + eps).clamp(0, 1)
        yl, yu = torch.empty_like(y), torch.empty_like(y)
        pl, pu = torch.empty_like(pos), torch.empty_like(pos)
        for name, fn, slots in (
                ("forward_nograd", lambda: C.inf_dist_forward_nograd(x, w, y, 1), 2),
                ("bounds_nograd", lambda: C.bound_inf_dist_forward_nograd(xl, xu, w, yl, yu, 1), 4),
                ("bounds_with_indices", lambda: C.bound_inf_dist_forward(xl, xu, w, yl, yu, pl, pu, 1), 4)):
            t = statistics.median(event_ms_list(fn, 10, 3, flush))
            ach = slots * pairs / (t * 1e-3) / 1e12
            extra.append({"p": "inf", "kernel": name, "ms": round(t, 4), "gpair_per_s": round(pairs / (t * 1e-3) / 1e9, 1),
                          "bound": "fp32", "slots_per_pair": slots, "tlaneop_per_s": round(ach, 2),
                          "frac_of_ffma_probe": round(ach / ffma_peak, 3), "frac_of_nominal": round(ach / nominal_fp32, 3)})
        line["variants"] = extra
        fwd()
    C.check_status()

    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args, target_s=12.0)
    return line


# ------------------------------------------------------------------------------------------------
# Model-level workloads: the reference's MLPModel / HybridModel recipes (ell_inf_models.py:16-75) on this package's
# models, losses (main.py:304-318) and optimisers; tests/test_gpu_models.py pins these classes to the reference
# ------------------------------------------------------------------------------------------------
IMAGE = [3, 32, 32]


def build_model(kind, p, device):
    """kind "mlp": MLPModel(depth=6, width=5120, identity_val=10.0); "hybrid": HybridModel(depth=7, width=5120,
    hidden=512, identity_val=10.0); random initial weights (seed 0 on every rank)."""
    import l_inf_dist_net_v2_b200 as ldn
    torch.manual_seed(0)
    with torch.device(device):
        if kind == "mlp":
            net = ldn.MLPModel(depth=6, width=5120, input_dim=IMAGE, identity_val=10.0)
        else:
            net = ldn.HybridModel(depth=7, width=5120, input_dim=IMAGE, hidden=512, identity_val=10.0)
    ldn.set_p_norm(net, p)
    return net


def make_optimizer_factory(name):
    from l_inf_dist_net_v2_b200.optim import FusedAdam, FusedSGD
    if name == "sgd":
        return (lambda params: FusedSGD(params, lr=0.02)), "SGD lr 0.02 (one-kernel update)"
    return (lambda params: FusedAdam(params, lr=0.03, betas=(0.9, 0.99), eps=1e-10)), \
        "Adam lr 0.03 betas (0.9, 0.99) eps 1e-10 as main.py:388-392 (one-kernel update)"


class TrainStep:
    """One training step as the reference's train() runs it (main.py:76-91): batch from pinned host memory, forward
    with targets, loss, backward, gradient exchange, optimiser step; the loss value goes back to the host."""

    def __init__(self, kind, p, batch, rank, world, device, optimizer="adam", reserve_sms=0, comm_group=None,
                 eps=None, shard_updates=False, graph=False):
        import l_inf_dist_net_v2_b200 as ldn
        from l_inf_dist_net_v2_b200.parallel import OverlappedDataParallel
        self.net = build_model(kind, p, device)
        self.net.train()
        self.loss_fn = ldn.losses.hinge(mix=0.25) if kind == "mlp" else ldn.losses.crossentropy(mix=0)
        self.eps = eps if eps is not None else (8.0 / 255.0 if kind == "mlp" else 0.0345)
        factory, self.optimizer_name = make_optimizer_factory(optimizer)
        self.graph = None
        self.graph_launches = 0
        self.use_graph = bool(graph) and world == 1
        if self.use_graph:
            # one GPU: the whole step (copies, forward, loss, backward, Adam with its step count on the device) is
            # recorded once and replayed; nothing is deferred
            from l_inf_dist_net_v2_b200.optim import FusedAdam
            self.opt = FusedAdam(list(self.net.parameters()), lr=0.03, betas=(0.9, 0.99), eps=1e-10, capturable=True)
            self.optimizer_name = "Adam lr 0.03 betas (0.9, 0.99) eps 1e-10 (one-kernel update, step count on the device)"
            self.ddp = None
        # first layer's exchange (exposed) on the default group at full width, the rest on the CTA-limited group
        if not self.use_graph:
            self.ddp = OverlappedDataParallel(
                self.net, factory, group=comm_group,
                first_group=torch.distributed.group.WORLD if comm_group is not None else None,
                reserve_sms=reserve_sms, shard_updates=shard_updates)
        gen = torch.Generator().manual_seed(1000 + rank)
        self.xh = torch.rand(batch, *IMAGE, generator=gen).pin_memory()
        self.th = torch.randint(0, 10, (batch,), generator=gen).pin_memory()
        self.x = torch.empty(batch, *IMAGE, device=device)
        self.t = torch.empty(batch, dtype=torch.long, device=device)
        self.loss_h = torch.zeros(1).pin_memory()
        self.h2d = self.xh.numel() * 4 + self.th.numel() * 8
        self.d2h = 4

    def _eager(self):
        self.x.copy_(self.xh, non_blocking=True)
        self.t.copy_(self.th, non_blocking=True)
        logits, worst = self.net(self.x, targets=self.t, eps=self.eps)
        loss = self.loss_fn(logits, worst, self.t)
        loss.backward()
        if self.ddp is not None:
            self.ddp.step()
        else:
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
        self.loss_h.copy_(loss.detach().view(1), non_blocking=True)

    def capture(self):
        """Warm-up on the capture stream (scratch arenas and optimiser state reach their final size), then record."""
        from l_inf_dist_net_v2_b200._lib import lib
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                self._eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = lib.ldn_kernel_launches()
        with torch.cuda.graph(self.graph, stream=s):
            self._eager()
        self.graph_launches = int(lib.ldn_kernel_launches() - before)

    def __call__(self):
        if self.use_graph:
            if self.graph is None:
                self.capture()
            self.graph.replay()
        else:
            self._eager()

    def finish(self):
        if self.ddp is not None:
            self.ddp.finish()


class CertifySweep:
    """The certification pass of main.py:182-215 over `samples` synthetic test images in batches of `batch`: eval
    mode, p = inf, value and interval bounds (eps = 8/255, box [0, 1]) through every layer, clean and certified
    correct counts accumulated on the device; the last batch may be ragged."""

    def __init__(self, kind, samples, batch, rank, device):
        self.net = build_model(kind, math.inf, device)
        self.net.eval()
        self.samples, self.batch = samples, batch
        gen = torch.Generator().manual_seed(2000 + rank)
        self.xh = torch.rand(batch, *IMAGE, generator=gen).pin_memory()
        self.th = torch.randint(0, 10, (batch,), generator=gen).pin_memory()
        self.x = torch.empty(batch, *IMAGE, device=device)
        self.t = torch.empty(batch, dtype=torch.long, device=device)
        self.up = torch.ones(3, 1, 1, device=device)
        self.down = torch.zeros(3, 1, 1, device=device)
        self.counts = torch.zeros(2, device=device)
        self.counts_h = torch.zeros(2).pin_memory()
        self.batches = (samples + batch - 1) // batch
        self.h2d = self.xh.numel() * 4 + self.th.numel() * 8

    def one_batch(self, n):
        self.x.copy_(self.xh, non_blocking=True)
        self.t.copy_(self.th, non_blocking=True)
        x, t = self.x[:n], self.t[:n]
        with torch.no_grad():
            logits, worst = self.net(x, targets=t, eps=8.0 / 255.0, up=self.up, down=self.down)
            self.counts[0] += (logits.argmax(1) == t).sum()
            self.counts[1] += (worst.argmax(1) == t).sum()

    def __call__(self):
        self.counts.zero_()
        left = self.samples
        for _ in range(self.batches):
            self.one_batch(min(self.batch, left))
            left -= self.batch
        self.counts_h.copy_(self.counts, non_blocking=True)


def _timed(fn, reps, world, dev):
    """reps calls of fn between two CUDA events, bracketed by barriers; max over ranks, in ms."""
    import torch.distributed as dist
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    _timed.host_ms = (time.perf_counter() - t0) * 1e3  # host time to enqueue the work (this rank)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms


def model_block(args, rank, world, local_rank, comm_group):
    """Configuration 5 of the benchmark set: HybridModel(depth=7, width=5120, hidden=512) at p = inf, one training
    step on a global batch of 4096 split over the ranks (main.py:346-348) with the gradient exchange, and the
    50 000-sample certification sweep sharded over the ranks."""
    import torch.distributed as dist
    from l_inf_dist_net_v2_b200._lib import lib
    dev = torch.device("cuda", local_rank)
    out = {}
    gb = args.model_global_batch
    if gb % world != 0:
        return {"error": f"global batch {gb} is not divisible by {world} ranks"}
    step = TrainStep("hybrid", math.inf, gb // world, rank, world, dev, optimizer="adam",
                     reserve_sms=args.reserve_sms if world > 1 else 0, comm_group=comm_group,
                     shard_updates=args.shard_updates)
    reps = 10 if world == 1 else 20
    launches0 = lib.ldn_kernel_launches()
    for _ in range(3):
        step()
    ms = _timed(step, reps, world, dev)
    host_ms = _timed.host_ms
    launches = int(lib.ldn_kernel_launches() - launches0) // (reps + 3)
    row = {"model": "HybridModel(depth=7, width=5120, hidden=512, identity_val=10.0), p=inf, cross-entropy on "
                    "worst-case logits, eps_train 0.0345",
           "global_batch": gb, "batch_per_rank": gb // world, "steps": reps, "ms_per_step": round(ms / reps, 3),
           "samples_per_s": round(gb * reps / (ms * 1e-3), 1), "optimizer": step.optimizer_name,
           "host_enqueue_ms_per_step": round(host_ms / reps, 3),
           "library_kernels_per_step": launches, "h2d_bytes_per_step": step.h2d, "d2h_bytes_per_step": step.d2h,
           "exchange": "none" if world == 1 else
           ("NCCL reduce-scatter (mean) per parameter, update of the rank's 1/N slice, all-gather"
            if args.shard_updates else "NCCL all-reduce (mean) per parameter") +
           f", started after backward in forward order, each layer's update deferred to just before its next forward; "
           f"{args.reserve_sms} SMs left free by the distance kernels while collectives are in flight"}
    if world > 1:
        step.ddp.exchange = False  # same step without the collectives: what the exchange costs
        for _ in range(2):
            step()
        ms0 = _timed(step, reps, world, dev)
        step.ddp.exchange = True
        row["ms_per_step_without_exchange"] = round(ms0 / reps, 3)
        row["exposed_exchange_ms"] = round((ms - ms0) / reps, 3)
    step.finish()
    out["hybrid_train"] = row
    del step
    torch.cuda.empty_cache()
    n_local = args.certify_samples // world
    sweep = CertifySweep("hybrid", n_local, 512, rank, dev)
    sweep.one_batch(512)
    sweep.one_batch(512)
    ms = _timed(sweep, 1, world, dev)
    counts = sweep.counts_h.clone().to(dev)
    if world > 1:
        dist.all_reduce(counts)  # main.py:207
    out["hybrid_certify"] = {
        "model": "HybridModel(depth=7, width=5120, hidden=512), eval mode, p=inf, value + interval bounds, eps=8/255",
        "samples": n_local * world, "samples_per_rank": n_local, "batch": 512, "batches_per_rank": sweep.batches,
        "seconds": round(ms * 1e-3, 4), "samples_per_s": round(n_local * world / (ms * 1e-3), 1),
        "h2d_bytes_per_batch": sweep.h2d, "clean_correct": int(counts[0]), "certified_correct": int(counts[1])}
    del sweep
    torch.cuda.empty_cache()
    return out


def run_model(args, rank, world, local_rank, comm_group):
    """--workload mlp-train | mlp-certify | hybrid-train | hybrid-certify: the model-level step as the headline."""
    import torch.distributed as dist
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    from l_inf_dist_net_v2_b200._lib import lib

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    kind, what = args.workload.split("-")
    train = what == "train"
    B = args.batch
    sampler = ClockSampler(local_rank)
    if train:
        p = p_value(args.p)
        step = TrainStep(kind, p, B, rank, world, dev, optimizer=args.optimizer,
                         reserve_sms=args.reserve_sms if world > 1 else 0, comm_group=comm_group,
                         shard_updates=args.shard_updates, graph=args.graph)
        h2d, d2h = step.h2d, step.d2h
        per_step = B
    else:
        n_local = args.certify_samples // world
        sweep = CertifySweep(kind, n_local, B, rank, dev)
        step = lambda: sweep.one_batch(B)  # noqa: E731
        h2d, d2h = sweep.h2d, 8
        per_step = B
        args.steps = min(args.steps, sweep.batches) if args.steps else sweep.batches
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler.mark()
    launches0 = lib.ldn_kernel_launches()
    ms = _timed(step, args.steps, world, dev)
    host_ms = _timed.host_ms
    launches = int(lib.ldn_kernel_launches() - launches0)
    if train and step.use_graph:
        launches = step.graph_launches * args.steps  # replays launch what the capture recorded
    clocks = sampler.stop()
    if train:
        step.finish()
    C.check_status()
    if rank != 0:
        return None
    value = world * per_step * args.steps / (ms * 1e-3)
    name = args.workload.replace("-", "_") + "_samples_per_s"
    model = ("HybridModel(depth=7, width=5120, hidden=512, identity_val=10.0)" if kind == "hybrid"
             else "MLPModel(depth=6, width=5120, identity_val=10.0)")
    loss_name = "cross-entropy on worst-case logits, eps_train 0.0345" if kind == "hybrid" else "hinge loss"
    return {"metric": name, "value": round(value, 1), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": ("%s training step, p=%s, %s, %s, batch %d per rank"
                                    % (model, args.p, loss_name, step.optimizer_name, B)) if train else
                                   ("%s certification (value + interval bounds, eps=8/255), p=inf, batch %d per rank"
                                    % (model, B)),
                       "batch_per_rank": B, "l2": "working set 560 MB of weights per step, larger than L2"},
            "e2e": {"value": round(value, 1), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "l_inf_dist_net_v2_b200 models + autograd + parallel.OverlappedDataParallel + optim" +
                           (", whole step replayed from a CUDA graph" if (train and step.use_graph) else "")},
            "gpu_launches": launches, "clocks": clocks,
            "host_enqueue_ms_per_step": round(host_ms / args.steps, 3)}


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's CPU torch path (oracle/torch_port.py)
# ------------------------------------------------------------------------------------------------
def _cpu_sample(args, rows, cols):
    gen = torch.Generator().manual_seed(0)
    x = torch.rand(rows, args.ci, 1, generator=gen)
    w = torch.randn(cols, args.ci, generator=gen)
    g = torch.randn(rows, cols, 1, generator=gen)
    return x, w, g


def _cpu_step(x, w, g, p):
    from oracle import torch_port
    t0 = time.perf_counter()
    torch_port.norm_dist_fwd_bwd(x, w, g, p, chunk=256)
    return time.perf_counter() - t0


def _size_sample(args, p, target_s):
    """Chooses (rows, cols) of the workload so that one forward+backward takes about target_s seconds."""
    rows = min(args.batch, 32)
    x, w, g = _cpu_sample(args, rows, 256)
    _cpu_step(x, w, g, p)
    t = _cpu_step(x, w, g, p)
    per_col = t / 256
    cols = int(max(256, min(args.co, (target_s / per_col) // 256 * 256)))
    return rows, cols


def cpu_baseline(args, target_s):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    p = p_value(args.p)
    rows, cols = _size_sample(args, p, target_s)
    x, w, g = _cpu_sample(args, rows, cols)
    t = _cpu_step(x, w, g, p)
    pairs = rows * cols * args.ci
    return {"value": round(pairs / t / 1e9, 4), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{rows} of {args.batch} batch rows x {cols} of {args.co} outputs x {args.ci} inputs, "
                      f"forward + autograd backward, p={args.p}, {t:.1f} s",
            "path": "oracle/torch_port.py (broadcast + vector_norm, the reference's use_custom_cuda_func=False path)"}


def run_reference(args, rank):
    if rank != 0:
        return None
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    p = p_value(args.p)
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows, cols = _size_sample(args, p, min(3.0, budget))
    x, w, g = _cpu_sample(args, rows, cols)
    for _ in range(args.warmup):
        _cpu_step(x, w, g, p)
    times = [_cpu_step(x, w, g, p) for _ in range(args.steps)]
    pairs = rows * cols * args.ci
    total = sum(times)
    value = pairs * args.steps / total / 1e9
    sample = (f"{rows} of {args.batch} batch rows x {cols} of {args.co} outputs x {args.ci} inputs per step, "
              f"forward + autograd backward")
    return {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"norm_dist layer fwd+bwd {args.batch}x{args.ci}->{args.co} per rank, p={args.p}, "
                               f"G=1, HW=1", "p": args.p, "batch_per_rank": args.batch, "in_features": args.ci,
                   "out_features": args.co, "sample": sample},
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def run_reference_cuda(args, rank, local_rank):
    """Extra arm: the reference's own CUDA kernels (oracle/_ref, recompiled for sm_100a) on the same step."""
    if rank != 0:
        return None
    from oracle.build import REF_SO
    if not os.path.exists(REF_SO):
        return {"impl": "reference-cuda", "unavailable": "oracle/_ref/libldn_ref.so was not built"}
    ref = ctypes.CDLL(REF_SO)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    p = p_value(args.p)
    B, CI, CO = args.batch, args.ci, args.co
    xh, wh, gh = make_host_inputs(args, rank)
    x, w, g = xh.to(dev), wh.to(dev), gh.to(dev)
    y = torch.empty(B, CO, 1, device=dev)
    pos = torch.empty(B, CO, 1, device=dev, dtype=torch.int32)
    gx, gw = torch.empty_like(x), torch.empty_like(w)
    flush_buf = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    dims = (B, CO, CI, 1, 1)

    def fwd():
        if math.isinf(p):
            ref.ldn_ref_inf_dist_forward(P(x), P(w), P(y), P(pos), *dims)
        else:
            ref.ldn_ref_norm_dist_forward(P(x), P(w), P(y), *dims, ctypes.c_float(p))

    def bwd():
        if math.isinf(p):
            ref.ldn_ref_inf_dist_backward_input_weight(P(g), P(pos), P(gx), P(gw), *dims)
        else:
            ref.ldn_ref_norm_dist_backward_input_weight(P(g), P(x), P(w), P(y), P(gx), P(gw), *dims, ctypes.c_float(p))

    def step():
        fwd()
        bwd()

    flush = flush_buf.zero_
    ms = event_ms_list(step, args.steps, max(args.warmup, 3), flush)
    t_f = statistics.median(event_ms_list(fwd, 10, 2, flush))
    t_b = statistics.median(event_ms_list(bwd, 10, 2, flush))
    pairs = B * CI * CO
    return {"impl": "reference-cuda", "metric": METRIC, "unit": UNIT,
            "value": round(pairs * args.steps / (sum(ms) * 1e-3) / 1e9, 2), "ms_per_step": round(sum(ms) / args.steps, 4),
            "forward_ms": round(t_f, 4), "backward_ms": round(t_b, 4), "n_gpus": 1, "steps": args.steps,
            "config": {"workload": f"norm_dist layer fwd+bwd {B}x{CI}->{CO}, p={args.p}, reference CUDA kernels "
                                   f"recompiled for sm_100a"}}


def main():
    # Libraries (NCCL among them) may print to stdout; the contract is ONE JSON line there.  Everything else that is
    # written to file descriptor 1 while the benchmark runs goes to stderr.
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        line = run_reference(args, rank)
    elif args.impl == "reference-cuda":
        line = run_reference_cuda(args, rank, local_rank)
    else:
        if world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        comm_group = None
        if world > 1 and args.reserve_sms > 0:
            from l_inf_dist_net_v2_b200.parallel import nccl_group_with_cta_limit
            comm_group = nccl_group_with_cta_limit(args.reserve_sms)
        if args.workload == "layer":
            line = run_ours(args, rank, world, local_rank, comm_group)
        else:
            line = run_model(args, rank, world, local_rank, comm_group)
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
    if line is not None:
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())


if __name__ == "__main__":
    main()
