"""Native quantised batch norm against a PyTorch restatement of utils_class.py:37-93 (CPU, fp32)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def reference_bn_fixed(x, weight, bias, running_mean, running_var, training, eps=1e-5, momentum=0.1):
    """utils_class.py:43-65: graph of F.batch_norm, value x * w_q + b_q."""
    out = F.batch_norm(x, running_mean, running_var, weight, bias, training=training, momentum=momentum, eps=eps)
    dims = (0, 2, 3) if x.dim() == 4 else (0,)
    shape = (-1, 1, 1) if x.dim() == 4 else (-1,)
    if training:
        mean, var = x.mean(dim=dims), x.var(dim=dims, unbiased=False)
    else:
        mean, var = running_mean, running_var
    w = weight.data if weight is not None else 1
    b = bias.data if bias is not None else 0
    w_n = (w / torch.sqrt(var + eps)).detach()
    b_n = (b - mean * w / torch.sqrt(var + eps)).detach()
    scale = 2 ** torch.ceil(torch.log2(torch.mean(w_n) * 3))
    q = lambda t: ((t / scale) * 128).round().clamp(-127, 127) / 128 * scale  # noqa: E731
    out.data = (x.data * q(w_n).reshape(shape) + q(b_n).reshape(shape)).to(out.dtype)
    return out, scale


@pytest.mark.parametrize("shape", [(16, 32, 8, 8), (5, 7, 3, 5), (64, 10), (256, 64, 4, 4)])
@pytest.mark.parametrize("training", [True, False])
@pytest.mark.parametrize("affine", [True, False])
def test_bn_fixed_matches_reference_formulation(cuda_device, shape, training, affine):
    from geo_b200 import layers

    g = torch.Generator().manual_seed(sum(shape) + training)
    C = shape[1]
    x = torch.rand(*shape, generator=g) * 2 - 0.3
    cls = layers.BatchNorm2d_fixed if len(shape) == 4 else layers.BatchNorm1d_fixed
    m = cls(C, affine=affine)
    with torch.no_grad():
        if affine:
            m.weight.copy_(torch.rand(C, generator=g) + 0.5)
            m.bias.copy_(torch.rand(C, generator=g) - 0.5)
        m.running_mean.copy_(torch.rand(C, generator=g) * 0.2 + 0.5)
        m.running_var.copy_(torch.rand(C, generator=g) * 0.2 + 0.2)
    rm, rv = m.running_mean.clone(), m.running_var.clone()
    w_ref = m.weight.detach().clone().requires_grad_(True) if affine else None
    b_ref = m.bias.detach().clone().requires_grad_(True) if affine else None
    x_ref = x.clone().requires_grad_(True)
    out_ref, scale_ref = reference_bn_fixed(x_ref, w_ref, b_ref, rm, rv, training)
    go = torch.randn(*shape, generator=g)
    out_ref.backward(go)

    m = m.to(cuda_device)
    m.train(training)
    xd = x.to(cuda_device).requires_grad_(True)
    out = m(xd)
    out.backward(go.to(cuda_device))

    assert float(m.scale) == float(scale_ref)
    # a folded coefficient that lands within rounding error of a quantisation boundary may fall on
    # the other side; everything else must agree to fp32 accuracy
    diff = (out.detach().cpu() - out_ref.detach()).abs()
    tol = 1e-5 * out_ref.detach().abs().max().item()
    assert (diff <= tol).float().mean().item() > 0.97
    assert torch.allclose(xd.grad.cpu(), x_ref.grad, rtol=1e-4, atol=1e-5 * x_ref.grad.abs().max().item())
    if affine:
        assert torch.allclose(m.weight.grad.cpu(), w_ref.grad, rtol=1e-4, atol=1e-5 * w_ref.grad.abs().max().item())
        assert torch.allclose(m.bias.grad.cpu(), b_ref.grad, rtol=1e-4, atol=1e-5 * b_ref.grad.abs().max().item())
    assert torch.allclose(m.running_mean.cpu(), rm, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m.running_var.cpu(), rv, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("shape", [(8, 5, 12, 12), (3, 4, 7, 9), (2, 3, 6, 10), (256, 32, 32, 32)])
def test_pool_hardtanh_matches_pytorch(cuda_device, shape):
    from geo_b200 import layers

    g = torch.Generator().manual_seed(shape[2])
    x = torch.rand(*shape, generator=g) * 2.4 - 0.7
    go = torch.randn(shape[0], shape[1], shape[2] // 2, shape[3] // 2, generator=g)
    xr = x.clone().requires_grad_(True)
    yr = F.hardtanh(F.avg_pool2d(xr, 2), 0, 1)
    yr.backward(go)
    xd = x.to(cuda_device).requires_grad_(True)
    y = layers.AvgPool2Hardtanh()(xd)
    y.backward(go.to(cuda_device))
    assert torch.allclose(y.detach().cpu(), yr.detach(), rtol=0, atol=1e-7)
    assert torch.allclose(xd.grad.cpu(), xr.grad, rtol=0, atol=1e-7)


def test_native_quantize_equals_the_elementwise_formula(cuda_device):
    """geo_sc_quantize against (x * 2^p).round().clamp(...) / 2^p (utils_functional.py:33-39), bit for bit:
    ties (round half to even), values beyond the clamp, negative zero, infinities, NaN, ragged sizes."""
    from geo_b200 import functional as sc_f
    from geo_b200 import ops

    g = torch.Generator().manual_seed(3)
    for prec in (0, 1, 7, 8, 12):
        levels = 2 ** prec
        x = torch.cat([
            (torch.rand(100003, generator=g) * 4 - 2),
            (torch.arange(-3 * levels, 3 * levels + 1, dtype=torch.float32) + 0.5) / levels,   # every tie
            torch.tensor([0.0, -0.0, 1.0, -1.0, float("inf"), float("-inf"), float("nan"), 1e-30, -1e-30, 3e38]),
        ]).to(cuda_device)
        want = (x * levels).round().clamp(-levels + 1, levels - 1) / levels
        got = ops.quantize(x, prec)
        assert torch.equal(torch.nan_to_num(got, nan=123.0), torch.nan_to_num(want, nan=123.0)), prec
        assert torch.equal(torch.isnan(got), torch.isnan(want))
        assert torch.equal(sc_f.quantize(x, prec=prec).isnan(), want.isnan())
    assert ops.quantize(torch.empty(0, device=cuda_device), 7).numel() == 0


def test_counts_to_float_is_exact(cuda_device):
    from geo_b200 import ops

    g = torch.Generator().manual_seed(11)
    for shape in ((256, 32, 16, 16), (3, 5, 7), (0,)):
        c = torch.randint(-5 * 256, 5 * 256, shape, generator=g, dtype=torch.int32).to(cuda_device)
        for L in (8, 128, 256):
            assert torch.equal(ops.counts_to_float(c, L), c.to(torch.float32) / L)


@pytest.mark.parametrize("shape", [(16, 32, 8, 8), (256, 32, 32, 32), (3, 5, 6, 12), (8, 64, 2, 4)])
@pytest.mark.parametrize("training", [True, False])
def test_fused_bn_pool_hardtanh_equals_the_two_layers(cuda_device, shape, training):
    """layers.bn_pool_hardtanh against AvgPool2Hardtanh()(BatchNorm2d_fixed(x)): same value (bit for bit),
    same running statistics and scale buffer, gradients within fp32 summation-order tolerance."""
    from geo_b200 import layers

    g = torch.Generator().manual_seed(sum(shape))
    C = shape[1]
    x0 = (torch.rand(*shape, generator=g) * 1.6 - 0.3).to(cuda_device)
    go = torch.randn(shape[0], C, shape[2] // 2, shape[3] // 2, generator=g).to(cuda_device)
    results = []
    for fused in (False, True):
        torch.manual_seed(1)
        bn = layers.BatchNorm2d_fixed(C).to(cuda_device)
        with torch.no_grad():
            bn.weight.fill_(1.3)
            bn.bias.fill_(0.2)
            bn.running_mean.fill_(0.4)
            bn.running_var.fill_(0.3)
        bn.train(training)
        x = x0.clone().requires_grad_(True)
        y = layers.bn_pool_hardtanh(bn, x) if fused else layers.AvgPool2Hardtanh()(bn(x))
        y.backward(go)
        results.append((y.detach(), x.grad, bn.weight.grad, bn.bias.grad, bn.running_mean.clone(), bn.running_var.clone(),
                        bn.scale.clone()))
    a, b = results
    assert torch.equal(a[0], b[0])
    assert torch.equal(a[4], b[4]) and torch.equal(a[5], b[5]) and torch.equal(a[6], b[6])
    for i, name in ((1, "grad_x"), (2, "grad_weight"), (3, "grad_bias")):
        scale = a[i].abs().max().item() + 1e-30
        assert (a[i] - b[i]).abs().max().item() <= 2e-5 * scale, name


def test_fused_bn_pool_hardtanh_falls_back_for_other_shapes(cuda_device):
    from geo_b200 import layers, ops

    x = torch.rand(2, 3, 7, 9).to(cuda_device)
    assert not ops.bn_pool_act_supported(x)
    bn = layers.BatchNorm2d_fixed(3).to(cuda_device)
    y = layers.bn_pool_hardtanh(bn, x)
    assert y.shape == (2, 3, 3, 4)


@pytest.mark.parametrize("training", [True, False])
def test_fused_epilogue_equals_the_separate_kernels(cuda_device, training):
    """Bit counts -> batch norm -> pool -> hardtanh -> rounding -> next layer's streams in one pass
    (geo_sc_epilogue_forward) against the chain of separate entry points, bit for bit: the rounded activation, the
    stream image including its zero border, the saved statistics and the running statistics; and the backward
    pass reading counts against the one reading the float value."""
    from geo_b200 import _lib, ops

    g = torch.Generator().manual_seed(12)
    cases = [
        # counts shape, L of the counts, next layer: (c_out, k, pad, L, mode, z_unit, load_unit, load_wait)
        ((6, 8, 12, 16), 128, (5, 3, 1, 128, "1d_bin", 4, 2, 2)),
        ((3, 5, 8, 8), 64, (7, 5, 2, 256, "yz_bin", 2, 8, 1)),
        ((4, 16, 4, 8), 256, (9, 2, 0, 32, "z_bin", 4, 3, 4)),
        ((2, 3, 6, 4), 32, (4, 1, 0, 16, "full_or", 4, 8, 1)),
        # next layers with >= 64 channels take the batch-innermost stream image (batch padded to a multiple of 4)
        ((6, 64, 8, 8), 128, (32, 3, 1, 128, "1d_bin", 4, 2, 2)),
        ((5, 72, 4, 8), 64, (40, 3, 1, 256, "full_or", 4, 8, 1)),
        ((9, 64, 12, 8), 128, (33, 3, 0, 64, "2d_bin", 4, 8, 1)),
    ]
    for shape, L_in, (O2, k, pad, L2, mode, z, lu, lw) in cases:
        B, C, H, W = shape
        counts = torch.randint(-L_in * 3, L_in * 3, shape, generator=g, dtype=torch.int32).to(cuda_device)
        bw = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
        bb = (torch.rand(C, generator=g) - 0.5).to(cuda_device)
        rm = [torch.rand(C, generator=g).to(cuda_device) for _ in range(1)] * 1
        rm1, rv1 = rm[0].clone(), (torch.rand(C, generator=g) + 0.5).to(cuda_device)
        rm2, rv2 = rm1.clone(), rv1.clone()
        nd = ops.make_desc(B, C, H // 2, W // 2, O2, k, k, L2, mode, pad_h=pad, pad_w=pad, z_unit=z, total_width=7,
                           load_width=lu, load_wait_w=lw, load_wait_a=lw)
        if C >= 64:
            assert _lib.act_stream_layout(nd) == (True, (B + 3) // 4 * 4)
        act, streams, mean, invstd, scale, wq, bq = ops.epilogue_forward(counts, L_in, nd, bw, bb, rm1, rv1, training, 0.1, 1e-5)
        x = ops.counts_to_float(counts, L_in)
        y, mean2, invstd2, scale2, wq2, bq2 = ops.bn_pool_act_forward(x, bw, bb, rm2, rv2, training, 0.1, 1e-5)
        yq = ops.quantize(y, 7)
        streams2 = ops.generate_act_streams(yq, nd)
        assert torch.equal(act, yq)
        # the buffers are rounded up to 256 bytes: compare the stream words, not the slack behind them
        assert torch.equal(ops.act_streams_canonical(streams, nd), ops.act_streams_canonical(streams2, nd))
        for a, b in ((mean, mean2), (invstd, invstd2), (scale, scale2), (wq, wq2), (bq, bq2), (rm1, rm2), (rv1, rv2)):
            assert torch.equal(a, b)
        go = torch.randn(act.shape, generator=g).to(cuda_device)
        gx, gw, gb = ops.epilogue_backward(counts, L_in, go, bw, mean, invstd, wq, bq, training)
        gx2, gw2, gb2 = ops.bn_pool_act_backward(x, go, bw, mean2, invstd2, wq2, bq2, training)
        assert torch.equal(gx, gx2) and torch.equal(gw, gw2) and torch.equal(gb, gb2)


def test_network_with_fused_blocks_equals_network_of_separate_layers(cuda_device):
    """The 4-layer CNN and the VGG-11-style network, forward and backward, with the SC blocks fused (one pass from
    bit counts to the next layer's streams) and as separate layers: logits, running statistics and every gradient
    are identical."""
    from geo_b200 import layers, network

    g = torch.Generator().manual_seed(31)
    for make, batch in ((network.CONV_tiny_add_partial, 16), (network.VGG11_add_partial, 8)):
        x = torch.rand(batch, 3, 32, 32, generator=g).to(cuda_device)
        y = torch.randint(0, 10, (batch,), generator=g).to(cuda_device)
        results = []
        for fuse in (True, False):
            layers.FUSE_EPILOGUE = fuse
            try:
                torch.manual_seed(5)
                net = make().to(cuda_device).train()
                out = net(x.clone())
                torch.nn.functional.cross_entropy(out, y).backward()
                stats = [b.detach().clone() for n, b in net.named_buffers() if "running" in n]
                results.append((out.detach().clone(), [p.grad.detach().clone() for p in net.parameters()], stats))
            finally:
                layers.FUSE_EPILOGUE = True
        assert torch.equal(results[0][0], results[1][0])
        for a, b in zip(results[0][1] + results[0][2], results[1][1] + results[1][2]):
            assert torch.equal(a, b)
        # evaluation mode: weight-stream cache and running statistics
        outs = []
        for fuse in (True, False):
            layers.FUSE_EPILOGUE = fuse
            try:
                net.eval()
                with torch.no_grad():
                    outs.append(net(x.clone()))
                    outs.append(net(x.clone()))      # second call: cached weight streams
            finally:
                layers.FUSE_EPILOGUE = True
        assert all(torch.equal(outs[0], o) for o in outs[1:])
