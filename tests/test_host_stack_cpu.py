"""Host-side mirrors of the reference's layers / network / training step, on the CPU, against a
golden step recorded from the reference's own Python (tests/golden/make_golden.py), and the
data-parallel gradient exchange on two gloo ranks."""
import os
import sys

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cpu_stand_in  # noqa: E402


def _load_reference_state(net, g):
    convs = [net.conv1, net.conv2, net.conv3, net.fc1]
    with torch.no_grad():
        for i, c in enumerate(convs):
            w = torch.from_numpy(g[f"w{i}_levels"].astype(np.float32)) / 128
            c.weight_org.copy_(w)
            c.weight.data.copy_(w)
    return convs


def test_training_step_matches_reference_python(monkeypatch, oracle_lib):
    from geo_b200 import network
    from geo_b200.train import TrainStep

    cpu_stand_in.install(monkeypatch)
    g = np.load(os.path.join(GOLDEN, "ref_tiny_cnn_step.npz"))
    torch.manual_seed(3)
    net = network.CONV_tiny_add_partial()
    net.err, net.z_unit, net.load_unit, net.load_wait = [7] * 4, [3, 3, 4, 4], [8] * 4, [2] * 4
    convs = _load_reference_state(net, g)
    x = torch.from_numpy(g["x_levels"].astype(np.float32)) / 128
    y = torch.from_numpy(g["y"])

    net.train()
    logits = net(x.clone())
    assert torch.allclose(logits, torch.from_numpy(g["logits"]), rtol=1e-5, atol=1e-5)
    loss = torch.nn.functional.cross_entropy(logits, y) * 128.0
    assert abs(loss.item() - float(g["loss"])) <= 1e-4 * abs(float(g["loss"]))
    loss.backward()
    for i, c in enumerate(convs):
        ref = g[f"gw{i}"]
        mine = c.weight.grad.numpy()
        mine = mine if mine.size <= 8000 else mine.reshape(-1)[::16]
        assert np.allclose(mine.reshape(ref.shape), ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max()), f"grad of conv {i}"
    assert np.allclose(net.bn1.weight.grad.numpy(), g["g_bn1_w"], rtol=1e-4, atol=1e-4 * np.abs(g["g_bn1_w"]).max())
    assert np.allclose(net.bn4.bias.grad.numpy(), g["g_bn4_b"], rtol=1e-4, atol=1e-6)

    # one optimiser step through TrainStep == the reference loop body (utils_own.py:98-114)
    torch.manual_seed(3)
    net2 = network.CONV_tiny_add_partial()
    net2.err, net2.z_unit, net2.load_unit, net2.load_wait = [7] * 4, [3, 3, 4, 4], [8] * 4, [2] * 4
    _load_reference_state(net2, g)
    TrainStep(net2, lr=2e-3, optim="SGD")(x.clone(), y)
    assert np.allclose(net2.fc1.weight_org.numpy(), g["fc1_weight_org_after"], rtol=0, atol=2e-7)
    assert np.allclose(net2.conv1.weight_org.numpy(), g["conv1_weight_org_after"], rtol=0, atol=2e-7)


def test_lenet_model_with_sc_linear_layers(monkeypatch, oracle_lib):
    """CONV_minimal_add_partial (two SC convs, three Linear_Or layers): shapes, gradients on every parameter,
    and the linear layer's value against the oracle."""
    from geo_b200 import layers, network

    cpu_stand_in.install(monkeypatch)
    torch.manual_seed(0)
    net = network.CONV_minimal_add_partial()
    x = torch.rand(3, 1, 28, 28)
    out = net(x)
    assert out.shape == (3, 10)
    out.sum().backward()
    for name, p in net.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
    lin = layers.Linear_Or(24, 7, bias=False)
    a = torch.rand(5, 24)
    y = lin(a.clone(), err=6)
    ref = oracle_lib.linear(lin.weight.new_tensor(((a * 128).round().clamp(-127, 127) / 128).numpy()), lin.weight.detach(), 64,
                            z_unit=24)
    assert torch.equal(y.detach() * 64, torch.from_numpy(ref).float())


def test_functional_argument_handling(monkeypatch, oracle_lib):
    from geo_b200 import functional as sc_f

    cpu_stand_in.install(monkeypatch)
    a = sc_f.quantize(torch.rand(2, 3, 6, 6), 7)
    w = sc_f.quantize(torch.rand(4, 3, 3, 3) * 2 - 1, 7)
    with pytest.raises(NotImplementedError):
        sc_f.conv2d_generic(a, w, (1, 1), (1, 1), forward="1d_bin", generator="lfsr", legacy=True)
    with pytest.raises(NotImplementedError):
        sc_f.conv2d_generic(a, w, (1, 1), (1, 1), forward="bin_mult", generator="lfsr")   # simulation-only mode
    with pytest.raises(NotImplementedError):
        sc_f.conv2d_generic(a, w, (1, 1), (1, 1), forward="1d_bin", generator="sobol")   # no such generator
    with pytest.raises(ValueError):
        sc_f.conv2d_generic(a, w, (1, 1), (2, 2), forward="1d_bin", generator="lfsr")
    # padding[0] pads the last dimension, padding[1] dimension 2 (utils_functional.py:492)
    out = sc_f.conv2d_generic(a, w, (2, 0), (1, 1), bit_length=64, forward="1d_bin", generator="lfsr")
    assert out.shape == (2, 4, 4, 8)
    assert torch.equal(out * 64, torch.from_numpy(oracle_lib.conv2d(a, w, 64, "1d_bin", pad_h=0, pad_w=2)).float())
    # defaults: bit_length 128, forward full_or, load_unit 8 (no progressive loading)
    out = sc_f.conv2d_generic(a, w, (0, 0), (1, 1))
    assert torch.equal(out * 128, torch.from_numpy(oracle_lib.conv2d(a, w, 128, "full_or")).float())
    lin = sc_f.linear_generic(a.flatten(1)[:, :24], w.flatten(1)[:, :24], bit_length=128, generator="lfsr")
    assert lin.shape == (2, 4)
    q, scale = sc_f.quantize_shift(torch.tensor([0.3, 0.7, 1.9]))
    assert float(scale) == 4.0 and torch.allclose(q, torch.tensor([0.3125, 0.6875, 1.90625]))


def _dp_worker(rank, world, port, tmpdir):
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_stand_in as stand_in

    class MP:  # minimal monkeypatch stand-in inside the child process
        def setattr(self, obj, name, val):
            setattr(obj, name, val)

    stand_in.install(MP())
    from geo_b200 import network
    from geo_b200.dp import GradientAllReduce, shard_batch
    from geo_b200.train import TrainStep

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.manual_seed(11)
    net = network.CONV_tiny_add_partial()
    net.load_unit = [8] * 4
    g = torch.Generator().manual_seed(5)
    x = torch.rand(4 * world, 3, 32, 32, generator=g)
    y = torch.randint(0, 10, (4 * world,), generator=g)
    xs, ys = shard_batch(x, y, rank, world)
    hook = GradientAllReduce(world)
    step = TrainStep(net, grad_hook=hook)
    step(xs.clone(), ys)
    torch.save({"fc1": net.fc1.weight_org.clone(), "conv2": net.conv2.weight_org.clone(),
                "bytes": hook.bytes_per_step}, os.path.join(tmpdir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_gradient_allreduce_two_gloo_ranks(monkeypatch, oracle_lib, tmp_path):
    import torch.multiprocessing as mp

    from geo_b200 import network
    from geo_b200.dp import shard_batch
    from geo_b200.train import TrainStep

    world, port = 2, 29000 + os.getpid() % 2000
    mp.spawn(_dp_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r0 = torch.load(os.path.join(tmp_path, "rank0.pt"))
    r1 = torch.load(os.path.join(tmp_path, "rank1.pt"))
    assert torch.equal(r0["fc1"], r1["fc1"]) and torch.equal(r0["conv2"], r1["conv2"])  # replicas stay in sync
    assert r0["bytes"] == 4 * sum(p.numel() for p in network.CONV_tiny_add_partial().parameters())

    # expected: average of the two shards' gradients, computed in this process
    cpu_stand_in.install(monkeypatch)
    g = torch.Generator().manual_seed(5)
    x = torch.rand(8, 3, 32, 32, generator=g)
    y = torch.randint(0, 10, (8,), generator=g)
    grads = []
    for rank in range(world):
        torch.manual_seed(11)
        net = network.CONV_tiny_add_partial()
        net.load_unit = [8] * 4
        net.train()
        xs, ys = shard_batch(x, y, rank, world)
        loss = torch.nn.functional.cross_entropy(net(xs.clone()), ys) * 128.0
        loss.backward()
        grads.append([p.grad.clone() for p in net.parameters()])
    torch.manual_seed(11)
    net = network.CONV_tiny_add_partial()
    net.load_unit = [8] * 4
    avg = [(a + b) / 2 for a, b in zip(*grads)]

    def inject(params):
        for p, gavg in zip(params, avg):
            p.grad = gavg.clone()

    xs, ys = shard_batch(x, y, 0, world)
    TrainStep(net, grad_hook=inject)(xs.clone(), ys)
    assert torch.allclose(net.fc1.weight_org, r0["fc1"], rtol=0, atol=1e-7)
    assert torch.allclose(net.conv2.weight_org, r0["conv2"], rtol=0, atol=1e-7)

    with pytest.raises(ValueError):
        shard_batch(x[:7], y[:7], 0, 2)
