"""World-size-2 CPU (gloo) test of the data-parallel plumbing: shard the batch, compute each rank's
grad_weight with the CPU checker, all-reduce (mean), compare with the full-batch gradient."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from l_inf_dist_net_v2_b200.parallel import shard_batch, shard_bounds, allreduce_mean_, average_scalars
    rng = np.random.default_rng(0)
    B, CI, CO = 8, 24, 10
    x = rng.random((B, CI, 1), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    g = rng.standard_normal((B, CO, 1)).astype(np.float32)
    lo, hi = shard_bounds(B, rank, world)
    assert (lo, hi) == (rank * 4, rank * 4 + 4)
    xs = shard_batch(torch.from_numpy(x), rank, world).numpy()
    gs = g[lo:hi]
    ys = oracle.norm_dist_forward(xs, w, 8.0)
    _, gw_local = oracle.norm_dist_backward(gs, xs, w, ys, 8.0, want_gx=False)
    gw = torch.from_numpy(gw_local.copy())
    bias_grad = torch.full((CO,), float(rank + 1))
    allreduce_mean_([gw, bias_grad], bucket_bytes=1 << 20)        # both in one bucket
    gw2 = torch.from_numpy(gw_local.copy())
    allreduce_mean_([gw2], bucket_bytes=16)                        # larger than a bucket: travels alone
    y_full = oracle.norm_dist_forward(x, w, 8.0)
    _, gw_full = oracle.norm_dist_backward(g, x, w, y_full, 8.0, want_gx=False)
    ok = np.allclose(gw.numpy(), gw_full / world, rtol=1e-5, atol=1e-6)
    ok = ok and np.allclose(gw2.numpy(), gw_full / world, rtol=1e-5, atol=1e-6)
    ok = ok and torch.allclose(bias_grad, torch.full((CO,), 1.5))
    m = average_scalars(float(rank), 2.0)
    ok = ok and abs(m[0] - 0.5) < 1e-6 and abs(m[1] - 2.0) < 1e-6
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "bad")
    dist.destroy_process_group()


def test_shard_and_allreduce_world2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_shard_bounds_rejects_uneven_batches():
    import pytest
    from l_inf_dist_net_v2_b200.parallel import shard_bounds
    with pytest.raises(ValueError):
        shard_bounds(10, 0, 4)
    assert shard_bounds(4096, 3, 8) == (1536, 2048)


def _overlap_worker(rank, world, port, out_dir, shard=False):
    """Three training steps of a small hybrid model: OverlappedDataParallel (updates applied layer by layer before
    the next forward) against the plain order (backward, all-reduce of every gradient, one optimiser step)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import copy
    import l_inf_dist_net_v2_b200 as ldn
    from l_inf_dist_net_v2_b200 import modules
    from l_inf_dist_net_v2_b200.parallel import OverlappedDataParallel, allreduce_mean_
    from oracle import torch_port
    # CPU ranks: the checker's torch port stands in for the CUDA operator
    modules.norm_dist = lambda x, w, p, groups=1, tag=None: torch_port.norm_dist(x, w, p, groups)
    torch.manual_seed(0)
    net_a = ldn.HybridModel(depth=4, width=32, input_dim=[1, 4, 4], hidden=16, identity_val=None)
    net_b = copy.deepcopy(net_a)
    ldn.set_p_norm(net_a, float("inf"))
    ldn.set_p_norm(net_b, float("inf"))
    loss_fn = ldn.losses.crossentropy()
    make = lambda params: torch.optim.Adam(params, lr=0.03, betas=(0.9, 0.99), eps=1e-10)  # noqa: E731
    if shard:
        OverlappedDataParallel.SMALL = 0  # shard every parameter whose size divides by the world size
    ddp = OverlappedDataParallel(net_a, make, shard_updates=shard)
    if shard:
        assert sum(len(u["slices"]) for u in ddp.units) >= 4
    opt_b = make(list(net_b.parameters()))
    gen = torch.Generator().manual_seed(100 + rank)
    ok = True
    for _ in range(3):
        x = torch.rand(8, 1, 4, 4, generator=gen)
        t = torch.randint(0, 10, (8,), generator=gen)
        for net in (net_a, net_b):
            net.train()
        logits, worst = net_a(x, targets=t, eps=0.03)
        loss_fn(logits, worst, t).backward()
        ddp.step()
        opt_b.zero_grad(set_to_none=True)
        logits_b, worst_b = net_b(x, targets=t, eps=0.03)
        loss_fn(logits_b, worst_b, t).backward()
        allreduce_mean_([q.grad for q in net_b.parameters()])
        opt_b.step()
        ok = ok and torch.equal(logits, logits_b)  # the forward saw the same parameters in both orders
    ddp.finish()
    for qa, qb in zip(net_a.parameters(), net_b.parameters()):
        ok = ok and torch.allclose(qa, qb, rtol=0, atol=1e-7)
    # buffers: rank 0's running means everywhere
    flat = torch.cat([b.reshape(-1) for b in net_a.buffers()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    ok = ok and all(torch.equal(gathered[0], g) for g in gathered)
    ok = ok and all(q.grad is None for q in net_a.parameters())
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "bad")
    dist.destroy_process_group()


def test_overlapped_data_parallel_matches_plain_order_world2(tmp_path):
    port = _free_port()
    mp.spawn(_overlap_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_overlapped_data_parallel_with_sharded_updates_world2(tmp_path):
    """Every rank updates only its slice of each parameter (with optimiser state for that slice) and the slices are
    gathered: the parameters must come out as with the full update on every rank."""
    port = _free_port()
    mp.spawn(_overlap_worker, args=(2, port, str(tmp_path), True), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"
