"""Data-parallel plumbing for the operator: the batch dimension shards with no communication; the only
exchange is the all-reduce (mean) of parameter gradients that follows the grad_weight kernels, as
DistributedDataParallel does in the reference (main.py:357), and the averaging of a few scalar metrics
(main.py:60-64).  Works with any torch.distributed backend (NCCL on GPUs, gloo in CPU tests)."""
import torch
import torch.distributed as dist

__all__ = ["shard_bounds", "shard_batch", "allreduce_mean_", "average_scalars", "OverlappedDataParallel",
           "nccl_group_with_cta_limit"]


def shard_bounds(n, rank, world):
    """Rows [lo, hi) of a global batch of n that rank `rank` of `world` owns: equal contiguous shards of
    n // world rows (main.py:346-348); n must be divisible by world."""
    if n % world != 0:
        raise ValueError(f"global batch {n} is not divisible by world size {world}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_batch(t, rank, world):
    lo, hi = shard_bounds(t.size(0), rank, world)
    return t[lo:hi]


def allreduce_mean_(tensors, group=None, bucket_bytes=64 << 20):
    """In-place mean over ranks of every tensor in `tensors`.  Tensors are packed into flat buckets of at
    most `bucket_bytes` (one collective per bucket; a tensor larger than a bucket travels alone, in place)."""
    world = dist.get_world_size(group)
    if world == 1:
        return
    # NCCL averages inside the collective; other backends (gloo) sum, then one division pass follows
    avg = dist.get_backend(group) == "nccl"
    bucket, size = [], 0

    def reduce_(t):
        if avg:
            dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
        else:
            dist.all_reduce(t, group=group)
            t.div_(world)

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        if len(bucket) == 1 and bucket[0].is_contiguous():
            reduce_(bucket[0])
        else:
            flat = torch.cat([b.reshape(-1) for b in bucket])
            reduce_(flat)
            off = 0
            for b in bucket:
                b.copy_(flat[off:off + b.numel()].view_as(b))
                off += b.numel()
        bucket, size = [], 0

    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if size + nbytes > bucket_bytes:
            flush()
        bucket.append(t)
        size += nbytes
    flush()


def average_scalars(*values, device=None, group=None):
    """Mean over ranks of a few python floats (assumes equal shard sizes, like the reference)."""
    t = torch.tensor(values, dtype=torch.float32, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, group=group)
        t /= dist.get_world_size(group)
    return t.tolist()


class _null_context:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


def nccl_group_with_cta_limit(max_ctas):
    """A second NCCL process group over all ranks whose collectives use at most `max_ctas` CTAs, so that they can run
    on the SMs the distance kernels are told to leave free (OverlappedDataParallel(reserve_sms=...))."""
    opts = dist.ProcessGroupNCCL.Options()
    opts.config.max_ctas = int(max_ctas)
    opts.config.min_ctas = 1
    return dist.new_group(backend="nccl", pg_options=opts)


class OverlappedDataParallel:
    """Data-parallel training with DistributedDataParallel's semantics (main.py:357: every rank applies the mean of all
    ranks' gradients) and most of the gradient exchange hidden behind the next step's forward pass.

    At p = inf a layer's backward pass is a scatter of a few hundred microseconds while its weight gradient is
    60-100 MB, so there is no backward work to hide the all-reduce behind.  Instead:

      * `step()` (after backward) starts the exchange of every parameter in FORWARD order and marks every layer's
        update as due; nothing waits;
      * a layer's own optimiser applies its update in a forward pre-hook, just before that layer is used again, after
        waiting for that layer's collectives only.  So only the first layer's exchange is exposed; the later layers'
        run beside the forward kernels of the layers in front of them.  The values every layer computes with are
        exactly those of the usual "all-reduce everything, then step" order;
      * the first layer's collectives use `first_group` (default: `group`); the others use `group`, which may be a
        CTA-limited NCCL group (nccl_group_with_cta_limit): while those are in flight the persistent distance kernels
        leave `reserve_sms` SMs free (ldn_set_max_ctas) for them -- a kernel that takes every SM would otherwise
        either keep the collective waiting or lose SMs to it in mid-flight;
      * `shard_updates=True`: large parameters are exchanged as reduce-scatter + all-gather instead of one all-reduce
        (the same bytes on the wire), and between the two every rank updates only its 1/world slice of the parameter,
        with optimiser state for that slice only.  The update is an elementwise map, so the parameters are the same
        as with the full update on every rank, but the memory-bound optimiser pass (28 bytes per parameter for Adam)
        shrinks by the world size.  The whole chain (reduce-scatter, slice update, all-gather, layer after layer in
        forward order) is issued on a side stream by `step()`; a layer's forward pre-hook only waits for that layer's
        all-gather.  Off by default: the slice updates then run on the few SMs the distance kernels leave free and the
        two collectives of a layer take longer than its one all-reduce; the step of the hybrid model at p = inf took
        12.5 ms with it against 7.5 ms without on two GPUs, 13.0 against 13.4 ms on four, 8.4 against 7.6 ms on eight.

    `optimizer_factory(params)` builds one optimiser per layer (any torch.optim optimiser, or optim.FusedAdam /
    FusedSGD); with shard_updates its parameters are 1-D slices that alias the layer's parameters.  Call `finish()`
    before evaluating, checkpointing or reading parameters: it applies what is still due and, like
    DistributedDataParallel's buffer broadcast, copies rank 0's buffers (MeanShift running means) to all ranks.
    """

    SMALL = 4 << 20  # pending bytes below which the distance kernels take all SMs again; smallest sharded parameter

    def __init__(self, model, optimizer_factory, group=None, first_group=None, reserve_sms=0, set_max_ctas=None,
                 shard_updates=False):
        self.model = model
        self.group = group
        self.first_group = first_group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.reserve_sms = reserve_sms if self.world > 1 else 0
        self._set_max_ctas = set_max_ctas
        self._sm_count = None
        self._capped = False
        self.units = []
        self.exchange = self.world > 1
        self.shard = bool(shard_updates) and self.world > 1
        self._side = None
        for module in model.modules():
            params = [q for q in module.parameters(recurse=False) if q.requires_grad]
            if not params:
                continue
            unit = {"module": module, "params": params, "pending": [], "bytes": 0, "due": False,
                    "ready": None, "slices": {}}
            opt_params = []
            for q in params:
                n = q.numel()
                if (self.shard and q.is_contiguous() and n % self.world == 0
                        and n * q.element_size() >= self.SMALL):
                    per = n // self.world
                    piece = q.data.view(-1)[self.rank * per:(self.rank + 1) * per]
                    unit["slices"][id(q)] = piece
                    opt_params.append(piece)
                else:
                    opt_params.append(q)
            unit["optimizer"] = optimizer_factory(opt_params)
            self.units.append(unit)
            module.register_forward_pre_hook(lambda mod, args, u=unit: self._apply(u))

    def _cap(self, on):
        if self.reserve_sms <= 0 or on == self._capped:
            return
        if self._set_max_ctas is None:
            from ._lib import lib
            self._set_max_ctas = lib.ldn_set_max_ctas
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self._set_max_ctas(self._sm_count - self.reserve_sms if on else 0)
        self._capped = on

    def _reduce(self, tensor, group, out=None):
        """Starts the mean over ranks of `tensor` (into `out`, this rank's slice of it, if given).  Backends without
        an averaging reduction or a reduce-scatter (gloo) sum with an all-reduce; the division follows the wait."""
        nccl = dist.get_backend(group) == "nccl"
        if nccl and out is not None:
            return dist.reduce_scatter_tensor(out, tensor, op=dist.ReduceOp.AVG, group=group, async_op=True), None
        op = dist.ReduceOp.AVG if nccl else dist.ReduceOp.SUM
        return dist.all_reduce(tensor, op=op, group=group, async_op=True), (None if nccl else tensor)

    def _update(self, unit):
        """On the current stream: wait for the unit's gradient exchange, update, and (sharded parameters) start and
        wait for the all-gather of the updated slices."""
        for work, summed in unit["pending"]:
            work.wait()
            if summed is not None:
                summed.div_(self.world)
        unit["pending"].clear()
        unit["bytes"] = 0
        stream = torch.cuda.current_stream() if torch.cuda.is_available() else None
        for q in unit["params"]:
            piece = unit["slices"].get(id(q))
            if piece is not None and q.grad is not None:
                per = piece.numel()
                piece.grad = q.grad.view(-1)[self.rank * per:(self.rank + 1) * per]
        unit["optimizer"].step()
        for q in unit["params"]:
            piece = unit["slices"].get(id(q))
            if piece is not None and q.grad is not None:
                if self.exchange:
                    work = dist.all_gather_into_tensor(q.data.view(-1), piece, group=unit["group"], async_op=True)
                    work.wait()
                piece.grad = None
            if q.grad is not None and stream is not None and q.grad.is_cuda:
                q.grad.record_stream(stream)  # the update may have run on the side stream
            q.grad = None
        unit["due"] = False

    def _apply(self, unit):
        if unit["ready"] is not None:
            torch.cuda.current_stream().wait_event(unit["ready"])  # exchanged and updated on the side stream
            unit["ready"] = None
            unit["bytes"] = 0
        elif unit["due"]:
            self._update(unit)
        else:
            return
        # kernels launched from here on are ordered behind every collective whose wait is already in the stream
        if self._capped and sum(u["bytes"] for u in self.units) < self.SMALL:
            self._cap(False)

    # -- training-loop interface ------------------------------------------------------------------------------------
    def step(self):
        """After backward: start the exchange (forward order) and make every layer's update due; the update itself
        happens before the layer's next forward, or in finish()."""
        side = None
        if self.shard and self.exchange and torch.cuda.is_available():
            if self._side is None:
                self._side = torch.cuda.Stream()
            side = self._side
            side.wait_stream(torch.cuda.current_stream())  # the gradients are complete
        first = True
        for unit in self.units:
            grads = [q for q in unit["params"] if q.grad is not None]
            if self.exchange and grads:
                group = (self.first_group if first and self.first_group is not None else self.group)
                unit["group"] = group
                ctx = torch.cuda.stream(side) if side is not None else _null_context()
                with ctx:
                    for q in grads:
                        piece = unit["slices"].get(id(q))
                        flat = q.grad.view(-1) if piece is not None else q.grad
                        out = None
                        if piece is not None:
                            per = piece.numel()
                            out = flat[self.rank * per:(self.rank + 1) * per]
                        unit["pending"].append(self._reduce(flat, group, out))
                        unit["bytes"] += q.grad.numel() * q.grad.element_size()
                    if side is not None:
                        # the rest of this layer's chain right behind its reduce-scatter, so that the next layer's
                        # collectives queue behind this layer's all-gather and not in front of it
                        nbytes = unit["bytes"]
                        self._update(unit)
                        unit["bytes"] = nbytes
                        unit["ready"] = torch.cuda.Event()
                        unit["ready"].record(side)
                first = False
            if unit["ready"] is None:
                unit["due"] = True
        if self.exchange and sum(u["bytes"] for u in self.units[1:]) >= self.SMALL:
            self._cap(True)

    def finish(self):
        for unit in self.units:
            self._apply(unit)
        if self._side is not None:
            torch.cuda.current_stream().wait_stream(self._side)
        self._cap(False)
        if self.world > 1:
            bufs = [b for b in self.model.buffers()]
            if bufs:
                flat = torch.cat([b.reshape(-1).float() for b in bufs])
                dist.broadcast(flat, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                               group=self.group)
                off = 0
                for b in bufs:
                    b.copy_(flat[off:off + b.numel()].view_as(b))
                    off += b.numel()
