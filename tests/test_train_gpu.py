"""Training step on the GPU: the whole-step CUDA graph must reproduce the eagerly launched step,
and the host mirror of the 4-layer CNN must reproduce the reference's recorded CPU step."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _model(device, seed=0):
    from geo_b200 import network

    torch.manual_seed(seed)
    net = network.CONV_tiny_add_partial()
    net.err, net.z_unit, net.load_unit, net.load_wait = [7] * 4, [3, 3, 4, 4], [2] * 4, [2] * 4
    return net.to(device)


def test_graph_replay_equals_eager_steps(cuda_device):
    from geo_b200.train import TrainStep

    g = torch.Generator().manual_seed(3)
    xs = [torch.rand(32, 3, 32, 32, generator=g).to(cuda_device) for _ in range(4)]
    ys = [torch.randint(0, 10, (32,), generator=g).to(cuda_device) for _ in range(4)]

    def run(graph, hook):
        net = _model(cuda_device)
        step = TrainStep(net, graph=graph, grad_hook=hook)
        losses = []
        # the warm-up runs of the capture are undone, so the graph's first call is one step like eager's;
        # the learning rate changes after the second step, as a scheduler would change it
        for i, (x, y) in enumerate(zip(xs, ys)):
            if i == 2:
                step.optimizer.param_groups[0]["lr"] = 5e-4
            loss, _ = step(x.clone(), y)
            losses.append(float(loss))
        stats = [b.detach().clone() for n, b in net.named_buffers() if "running" in n]
        return losses, [p.detach().clone() for p in net.parameters()] + stats

    l_eager, p_eager = run(False, None)
    l_graph, p_graph = run(True, None)
    l_two, p_two = run(True, lambda params: None)   # a gradient hook splits the step into two graphs
    assert l_eager == l_graph == l_two              # every kernel is deterministic: bit-identical
    for a, b, c in zip(p_eager, p_graph, p_two):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_graph_step_with_adam_is_capturable(cuda_device):
    """Adam under graph replay (capturable form, tensor learning rate) follows the eager Adam step."""
    from geo_b200.train import TrainStep

    g = torch.Generator().manual_seed(5)
    x = torch.rand(16, 3, 32, 32, generator=g).to(cuda_device)
    y = torch.randint(0, 10, (16,), generator=g).to(cuda_device)
    out = []
    for graph in (False, True):
        net = _model(cuda_device, seed=2)
        step = TrainStep(net, lr=1e-3, optim="Adam", graph=graph)
        for _ in range(3):
            loss, _ = step(x.clone(), y)
        out.append((float(loss), [p.detach().clone() for p in net.parameters()]))
    assert abs(out[0][0] - out[1][0]) <= 1e-4 * abs(out[0][0])
    for a, b in zip(out[0][1], out[1][1]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)


def test_evaluation_cache_survives_a_change_of_batch_size(cuda_device):
    """Weight streams prepared at one batch size serve any other: the prepared layout (dense streams plus the
    sign-sorted section of long-group layers) does not depend on the batch.  conv3 of the 4-layer CNN at batch 1
    has 64 output positions (dense kernel), at batch 8 it has 512 (sign-sorted kernel)."""
    g = torch.Generator().manual_seed(10)
    x = torch.rand(8, 3, 32, 32, generator=g).to(cuda_device)
    for order in ((1, 8), (8, 1)):
        net = _model(cuda_device).eval()
        with torch.no_grad():
            got = [net(x[:n].clone()) for n in order]          # second call hits the cache of the first
            for c in (net.conv1, net.conv2, net.conv3, net.fc1):
                c.invalidate_stream_cache()
            fresh = net(x[:order[1]].clone())                  # uncached
            assert torch.equal(got[1], fresh)
            big, small = (got[1], got[0]) if order == (1, 8) else (got[0], got[1])
            assert torch.equal(big[:1], small)                 # and the result does not depend on the batch split


def test_evaluation_keeps_weight_streams_until_the_weights_change(cuda_device):
    """In evaluation mode a layer quantises its weights and packs their streams once; the result must
    equal the uncached computation, fewer kernels are launched from the second call on, and an
    in-place change of ``weight_org`` (optimiser step, checkpoint load) drops the cache."""
    from geo_b200 import ops

    net = _model(cuda_device).eval()
    g = torch.Generator().manual_seed(9)
    x = torch.rand(8, 3, 32, 32, generator=g).to(cuda_device)
    with torch.no_grad():
        ops.STATS.reset()
        y1 = net(x.clone())
        first = ops.STATS.launches
        ops.STATS.reset()
        y2 = net(x.clone())
        second = ops.STATS.launches
        assert torch.equal(y1, y2)
        assert second < first                       # no weight quantisation, no weight-stream kernels
        # same weights through the training-mode path (no cache) with frozen statistics
        net.train()
        for m in net.modules():
            if hasattr(m, "running_mean"):
                m.eval()
        y3 = net(x.clone())
        assert torch.equal(y1, y3)
        net.eval()
        # an in-place weight change must be seen
        net.conv2.weight_org.mul_(0.5)
        y4 = net(x.clone())
        assert not torch.equal(y1, y4)
        for c in (net.conv1, net.conv2, net.conv3, net.fc1):
            c.invalidate_stream_cache()
        assert torch.equal(net(x.clone()), y4)
        # a write through .data bypasses the version counter: the cache has to be dropped by hand
        net.conv2.weight_org.data.mul_(2.0)
        net.conv2.invalidate_stream_cache()
        assert torch.equal(net(x.clone()), y1)


def test_vgg16_and_lenet_models_train_one_step(cuda_device):
    """The two other models of the reference's network.py: one eager training step each runs on the native
    kernels and leaves finite losses, gradients and parameters."""
    from geo_b200 import network
    from geo_b200.train import TrainStep

    g = torch.Generator().manual_seed(21)
    for net, x in ((network.VGG16_add_partial(), torch.rand(8, 3, 32, 32, generator=g)),
                   (network.CONV_minimal_add_partial(), torch.rand(16, 1, 28, 28, generator=g))):
        net = net.to(cuda_device)
        y = torch.randint(0, 10, (x.shape[0],), generator=g).to(cuda_device)
        step = TrainStep(net)
        before = [p.detach().clone() for p in net.parameters()]
        loss, out = step(x.to(cuda_device), y)
        assert out.shape == (x.shape[0], 10) and torch.isfinite(loss)
        changed = sum(int(not torch.equal(a, b)) for a, b in zip(before, net.parameters()))
        assert changed > 0 and all(torch.isfinite(p).all() for p in net.parameters())


def test_two_graph_step_with_packed_gradient_exchange(cuda_device):
    """The data-parallel hook's pack / unpack phases live inside the two graphs and only the
    collective runs between them; with a one-rank process group the result must equal the
    hook-free step exactly."""
    import torch.distributed as dist

    from geo_b200.dp import GradientAllReduce
    from geo_b200.train import TrainStep

    created = False
    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{29600 + os.getpid() % 300}", rank=0, world_size=1)
        created = True
    try:
        g = torch.Generator().manual_seed(4)
        x = torch.rand(16, 3, 32, 32, generator=g).to(cuda_device)
        y = torch.randint(0, 10, (16,), generator=g).to(cuda_device)
        results = []
        for hook in (None, GradientAllReduce(1)):
            net = _model(cuda_device, seed=1)
            step = TrainStep(net, graph=True, grad_hook=hook)
            for _ in range(3):
                loss, _ = step(x.clone(), y)
            torch.cuda.synchronize()
            results.append((float(loss), [p.detach().clone() for p in net.parameters()]))
        assert results[0][0] == results[1][0]
        for a, b in zip(results[0][1], results[1][1]):
            assert torch.equal(a, b)
    finally:
        if created:
            dist.destroy_process_group()


def test_gpu_step_matches_reference_cpu_step(cuda_device):
    """Same check as the CPU host-stack test, but through the CUDA kernels (load_unit 8, as the
    reference's CPU kernel has no progressive loading)."""
    from geo_b200 import network

    g = np.load(os.path.join(GOLDEN, "ref_tiny_cnn_step.npz"))
    torch.manual_seed(3)
    net = network.CONV_tiny_add_partial()
    net.err, net.z_unit, net.load_unit, net.load_wait = [7] * 4, [3, 3, 4, 4], [8] * 4, [2] * 4
    convs = [net.conv1, net.conv2, net.conv3, net.fc1]
    with torch.no_grad():
        for i, c in enumerate(convs):
            w = torch.from_numpy(g[f"w{i}_levels"].astype(np.float32)) / 128
            c.weight_org.copy_(w)
            c.weight.data.copy_(w)
    net = net.to(cuda_device)
    x = (torch.from_numpy(g["x_levels"].astype(np.float32)) / 128).to(cuda_device)
    y = torch.from_numpy(g["y"]).to(cuda_device)
    net.train()
    logits = net(x.clone())
    ref = torch.from_numpy(g["logits"])
    assert torch.allclose(logits.detach().cpu(), ref, rtol=1e-4, atol=1e-4)
    loss = torch.nn.functional.cross_entropy(logits, y) * 128.0
    loss.backward()
    for i, c in enumerate(convs):
        refg = g[f"gw{i}"]
        mine = c.weight.grad.detach().cpu().numpy()
        mine = mine if mine.size <= 8000 else mine.reshape(-1)[::16]
        assert np.allclose(mine.reshape(refg.shape), refg, rtol=1e-3, atol=2e-5 * np.abs(refg).max()), f"grad of conv {i}"
