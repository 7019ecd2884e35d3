"""Data-parallel gradient exchange on gloo ranks (CPU): the bucketed, overlapped all-reduce gives the same
averages as the flat one; ranks whose gradient layouts differ are refused; a rank that leaves between two steps
makes its peer's next exchange fail within the process-group timeout instead of waiting for ever.  Failures are
made on the host only."""
import datetime
import os
import time

import pytest
import torch


def _tiny_model(width=6, seed=3):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(5, width), torch.nn.Tanh(), torch.nn.Linear(width, 4),
                               torch.nn.Tanh(), torch.nn.Linear(4, 3))


def _grads(net, rank):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.rand(7, 5, generator=g)
    for p in net.parameters():
        p.grad = None
    net(x).square().sum().backward()


def _init(rank, world, port, timeout_s=60):
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return dist


def _bucketed_worker(rank, world, port, tmpdir):
    from geo_b200.dp import BucketedGradientAllReduce, GradientAllReduce

    dist = _init(rank, world, port)
    out = {}
    for name in ("flat", "bucketed"):
        net = _tiny_model()
        params = list(net.parameters())
        # 64-byte buckets: the six parameters fall into several buckets, the first two layers' last
        hook = GradientAllReduce(world) if name == "flat" else BucketedGradientAllReduce(params, world, bucket_bytes=64)
        for _ in range(2):          # twice: the hook must re-arm itself
            _grads(net, rank)
            hook(params)
        out[name] = [p.grad.clone() for p in params]
        if name == "bucketed":
            out["buckets"] = len(hook.buckets)
            # a parameter that received no gradient contributes zeros and keeps its None
            _grads(net, rank)
            params[0].grad = None
            hook(params)
            out["none_kept"] = params[0].grad is None
    torch.save(out, os.path.join(tmpdir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_allreduce_equals_flat_allreduce(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, 21000 + os.getpid() % 2000
    mp.spawn(_bucketed_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [torch.load(os.path.join(tmp_path, f"r{i}.pt")) for i in range(world)]
    assert r[0]["buckets"] >= 3 and r[0]["none_kept"]
    # expected averages computed here
    expect = None
    for rank in range(world):
        net = _tiny_model()
        _grads(net, rank)
        gs = [p.grad.clone() for p in net.parameters()]
        expect = gs if expect is None else [a + b for a, b in zip(expect, gs)]
    expect = [e / world for e in expect]
    for rank in range(world):
        for a, b, e in zip(r[rank]["flat"], r[rank]["bucketed"], expect):
            assert torch.allclose(a, e, rtol=0, atol=1e-6) and torch.equal(a, b)


def _mismatch_worker(rank, world, port, tmpdir):
    from geo_b200.dp import BucketedGradientAllReduce, GradientAllReduce

    dist = _init(rank, world, port)
    raised = []
    net = _tiny_model(width=6 + rank)          # rank 1 has a wider hidden layer
    params = list(net.parameters())
    try:
        BucketedGradientAllReduce(params, world, bucket_bytes=1 << 20)
    except ValueError as e:
        raised.append("bucketed:" + str(e)[:40])
    try:
        _grads(net, rank)
        GradientAllReduce(world)(params)
    except ValueError as e:
        raised.append("flat:" + str(e)[:40])
    torch.save(raised, os.path.join(tmpdir, f"m{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_with_different_gradient_layouts_are_refused(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, 23000 + os.getpid() % 2000
    mp.spawn(_mismatch_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        raised = torch.load(os.path.join(tmp_path, f"m{rank}.pt"))
        assert len(raised) == 2 and raised[0].startswith("bucketed:") and raised[1].startswith("flat:")


def _departing_worker(rank, world, port, tmpdir):
    from geo_b200.dp import GradientAllReduce

    dist = _init(rank, world, port, timeout_s=8)
    net = _tiny_model()
    params = list(net.parameters())
    hook = GradientAllReduce(world)
    _grads(net, rank)
    hook(params)                                # step 1: both ranks take part
    if rank == 1:
        return                                  # leaves between steps, nothing in flight
    t0 = time.time()
    err = None
    try:
        _grads(net, rank)
        hook(params)                            # step 2: the peer is gone
    except Exception as e:  # noqa: BLE001  (gloo reports a closed connection or a timeout as RuntimeError)
        err = type(e).__name__
    torch.save({"err": err, "seconds": time.time() - t0}, os.path.join(tmpdir, "departed.pt"))


def test_rank_that_leaves_between_steps_fails_its_peer_in_bounded_time(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, 25000 + os.getpid() % 2000
    ctx = mp.spawn(_departing_worker, args=(world, port, str(tmp_path)), nprocs=world, join=False)
    t0 = time.time()
    while not ctx.join(timeout=5):
        assert time.time() - t0 < 90, "ranks did not finish"
    r = torch.load(os.path.join(tmp_path, "departed.pt"))
    assert r["err"] is not None, "the surviving rank's all-reduce returned although its peer had left"
    assert r["seconds"] < 40
