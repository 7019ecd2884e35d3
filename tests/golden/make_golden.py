"""Generate the committed golden vectors from the reference itself.

Run in a container where the reference tree is mounted and ``oracle/build_ref.py`` has been
run:   python tests/golden/make_golden.py

Two files are written next to this script:

* ``ref_cpu_1d.npz``     -- outputs of the reference's CPU kernel ``sc_extension.conv2d_add_partial_new``
  (torch_c/sc-extension/sc.cpp, built unmodified) for a list of small cases.
* ``ref_legacy_L128.npz`` -- outputs of the reference's bit-serial PyTorch simulation
  (``utils_functional.conv2d_generic(..., legacy=True)``, utils_functional.py:516-609) at L=128
  for 1d_bin and full_or, and of ``linear_generic`` (utils_functional.py:302-404) for full_or.

Inputs are stored with the outputs so that the vectors do not depend on any RNG.
(The vectors for progressive loading and the z/yz modes come from the reference's CUDA
kernels and are generated on a GPU by ``make_golden_cuda.py``.)
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


CPU_CASES = [
    # (L, act shape, weight shape, (pad0, pad1) as passed to the reference, quantised?)
    (8, (2, 3, 7, 6), (3, 3, 3, 2), (0, 0), True),
    (16, (2, 3, 7, 6), (3, 3, 3, 2), (0, 0), True),
    (32, (2, 3, 7, 6), (3, 3, 3, 2), (1, 0), True),
    (64, (3, 5, 9, 8), (7, 5, 2, 4), (0, 0), True),
    (64, (2, 3, 8, 8), (4, 3, 5, 5), (2, 2), False),
    (128, (2, 3, 8, 8), (4, 3, 3, 3), (1, 2), False),
    (128, (1, 6, 6, 10), (17, 6, 3, 3), (1, 1), True),
    (256, (2, 4, 6, 6), (5, 4, 3, 3), (1, 1), True),
    (256, (1, 1, 5, 5), (1, 1, 1, 1), (0, 0), False),
    (128, (3, 8, 4, 4), (10, 8, 4, 4), (0, 0), True),
]


def main():
    ext = ref_loader.ref_sc_extension()
    assert ext is not None, "run oracle/build_ref.py first"
    torch.manual_seed(20240)
    out = {}
    for i, (L, ashape, wshape, pad, quant) in enumerate(CPU_CASES):
        a = torch.rand(*ashape)
        w = torch.rand(*wshape) * 2 - 1
        if quant:
            a, w = q7(a), q7(w)
        # exercise the clamps as well
        if i % 3 == 0:
            a.view(-1)[0] = 1.5
            a.view(-1)[1] = -0.25
            w.view(-1)[0] = 1.0
            w.view(-1)[1] = -1.0
        y = ext.conv2d_add_partial_new(a, w, L, pad, (1, 1))
        out[f"c{i}_a"] = a.numpy()
        out[f"c{i}_w"] = w.numpy()
        out[f"c{i}_meta"] = np.array([L, pad[0], pad[1]], np.int32)
        out[f"c{i}_y"] = y.numpy().astype(np.int32)
    out["n"] = np.array(len(CPU_CASES))
    np.savez_compressed(os.path.join(HERE, "ref_cpu_1d.npz"), **out)

    uf = ref_loader.reference_python()
    out = {}
    cases = [("1d_bin", (2, 3, 8, 8), (4, 3, 3, 3), (1, 1)), ("full_or", (2, 3, 8, 8), (4, 3, 3, 3), (1, 1)),
             ("1d_bin", (1, 4, 6, 7), (3, 4, 2, 5), (0, 0)), ("full_or", (2, 2, 5, 5), (6, 2, 3, 2), (0, 1))]
    for i, (fwd, ashape, wshape, pad) in enumerate(cases):
        a = q7(torch.rand(*ashape))
        w = q7(torch.rand(*wshape) * 2 - 1)
        y = uf.conv2d_generic(a.clone(), w.clone(), pad, (1, 1), bit_length=128, forward=fwd, generator="lfsr",
                              legacy=True)
        out[f"c{i}_a"] = a.numpy()
        out[f"c{i}_w"] = w.numpy()
        out[f"c{i}_meta"] = np.array([128, pad[0], pad[1], 0 if fwd == "1d_bin" else 3], np.int32)
        out[f"c{i}_y"] = (y.detach() * 128).round().numpy().astype(np.int32)
    out["n"] = np.array(len(cases))
    # linear_generic full_or, shared generators (seed index = input feature)
    a = q7(torch.rand(5, 24))
    w = q7(torch.rand(7, 24) * 2 - 1)
    y = uf.linear_generic(a.clone(), w.clone(), bit_length=128, generator="lfsr", forward="full_or")
    out["lin_a"], out["lin_w"] = a.numpy(), w.numpy()
    out["lin_y"] = (y.detach() * 128).round().numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "ref_legacy_L128.npz"), **out)
    print("wrote", sorted(os.listdir(HERE)))


def make_2d_golden():
    """``ref_legacy_2d_L128.npz``: the reference's bit-serial simulation with forward='2d_bin' (OR over the
    channels, binary accumulation over the filter taps; utils_functional.py:528-541,597-601) at L=128."""
    uf = ref_loader.reference_python()
    torch.manual_seed(4242)
    out = {}
    cases = [((2, 3, 8, 8), (4, 3, 3, 3), (1, 1)), ((1, 5, 6, 7), (3, 5, 2, 4), (0, 0)), ((2, 8, 5, 5), (6, 8, 3, 2), (0, 1)),
             ((3, 2, 4, 4), (5, 2, 1, 1), (0, 0))]
    for i, (ashape, wshape, pad) in enumerate(cases):
        a = q7(torch.rand(*ashape))
        w = q7(torch.rand(*wshape) * 2 - 1)
        y = uf.conv2d_generic(a.clone(), w.clone(), pad, (1, 1), bit_length=128, forward="2d_bin", generator="lfsr",
                              legacy=True)
        out[f"c{i}_a"] = a.numpy()
        out[f"c{i}_w"] = w.numpy()
        out[f"c{i}_meta"] = np.array([128, pad[0], pad[1], 4], np.int32)
        out[f"c{i}_y"] = (y.detach() * 128).round().numpy().astype(np.int32)
    out["n"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "ref_legacy_2d_L128.npz"), **out)
    print("wrote ref_legacy_2d_L128.npz")


def make_full_bin_golden():
    """``ref_legacy_full_bin_L128.npz``: the reference's bit-serial simulation with forward='full_bin' (every
    product bit counted, no OR; utils_functional.py:593-595,607-609 and :379-384 for the linear layer) at L=128."""
    uf = ref_loader.reference_python()
    torch.manual_seed(777)
    out = {}
    cases = [((2, 3, 8, 8), (4, 3, 3, 3), (1, 1)), ((1, 5, 6, 7), (3, 5, 2, 4), (0, 0)), ((2, 8, 5, 5), (6, 8, 3, 2), (0, 1))]
    for i, (ashape, wshape, pad) in enumerate(cases):
        a = q7(torch.rand(*ashape))
        w = q7(torch.rand(*wshape) * 2 - 1)
        y = uf.conv2d_generic(a.clone(), w.clone(), pad, (1, 1), bit_length=128, forward="full_bin", generator="lfsr",
                              legacy=True)
        out[f"c{i}_a"] = a.numpy()
        out[f"c{i}_w"] = w.numpy()
        out[f"c{i}_meta"] = np.array([128, pad[0], pad[1], 5], np.int32)
        out[f"c{i}_y"] = (y.detach() * 128).round().numpy().astype(np.int32)
    out["n"] = np.array(len(cases))
    a = q7(torch.rand(5, 24))
    w = q7(torch.rand(7, 24) * 2 - 1)
    y = uf.linear_generic(a.clone(), w.clone(), bit_length=128, generator="lfsr", forward="full_bin")
    out["lin_a"], out["lin_w"] = a.numpy(), w.numpy()
    out["lin_y"] = (y.detach() * 128).round().numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "ref_legacy_full_bin_L128.npz"), **out)
    print("wrote ref_legacy_full_bin_L128.npz")


def make_acc_golden(generator="acc"):
    """``ref_legacy_acc_stats.npz`` / ``ref_legacy_rand_stats.npz``: mean and standard deviation, over 200 runs,
    of the outputs of the reference's bit-serial simulation with generator='acc' (random sampling without
    replacement, utils_functional.py:157-176) or 'rand' (independent bits, :92-102) for one small 1d_bin conv
    at L=128 -- the target of a statistical check."""
    uf = ref_loader.reference_python()
    torch.manual_seed(99)
    a = q7(torch.rand(2, 4, 6, 6))
    w = q7((torch.rand(5, 4, 3, 3) * 2 - 1) * 0.6)
    runs = []
    for _ in range(200):
        y = uf.conv2d_generic(a.clone(), w.clone(), (1, 1), (1, 1), bit_length=128, forward="1d_bin",
                              generator=generator, legacy=True)
        runs.append((y.detach() * 128).round())
    r = torch.stack(runs)
    np.savez_compressed(os.path.join(HERE, f"ref_legacy_{generator}_stats.npz"), a=a.numpy(), w=w.numpy(),
                        mean=r.mean(0).numpy().astype(np.float32), std=r.std(0).numpy().astype(np.float32),
                        runs=np.array(200))
    print(f"wrote ref_legacy_{generator}_stats.npz")


def make_training_step_golden():
    """One forward/backward/SGD step of the reference's own 4-layer CNN on the CPU
    (network.CONV_tiny_add_partial + utils_class + utils_own.forward, reference files unmodified),
    batch 4.  Weights are stored as the int8 levels the layers quantise to, inputs as uint8 levels."""
    import sys
    import types

    uf = ref_loader.reference_python()
    from oracle import REFERENCE_ROOT as ref_root
    for name in ("bokeh", "bokeh.io", "bokeh.plotting", "bokeh.layouts"):   # utils.py imports them, unused here
        m = types.ModuleType(name)
        m.output_file = m.save = m.show = m.figure = m.column = None
        sys.modules.setdefault(name, m)
    sys.modules["utils_functional"] = uf
    sys.modules["sc_extension"] = ref_loader.ref_sc_extension()
    sys.path.insert(0, ref_root)
    try:
        import network
        import utils_own
    finally:
        sys.path.remove(ref_root)
    torch.manual_seed(3)
    net = network.CONV_tiny_add_partial()
    net.err, net.z_unit, net.load_unit, net.load_wait = [7] * 4, [3, 3, 4, 4], [8] * 4, [2] * 4
    convs = [net.conv1, net.conv2, net.conv3, net.fc1]
    for c in convs:       # put the master weights on the 7-bit grid so that they can be stored as int8
        c.weight_org.copy_(q7(c.weight_org * 3))
        c.weight.data.copy_(c.weight_org)
    x_lv = torch.randint(0, 128, (4, 3, 32, 32), dtype=torch.uint8)
    y = torch.tensor([3, 1, 4, 1])
    out = {"x_levels": x_lv.numpy(), "y": y.numpy()}
    for i, c in enumerate(convs):
        out[f"w{i}_levels"] = (c.weight_org * 128).round().to(torch.int8).numpy()
    param_copy = [p.clone().float().detach().requires_grad_(True) for p in net.parameters()]
    opt = torch.optim.SGD(param_copy, lr=2e-3, weight_decay=0, momentum=0.01)
    net.train()
    # forward/backward once by hand to record logits and gradients ...
    logits = net(x_lv.float() / 128)
    loss = torch.nn.functional.cross_entropy(logits, y) * 128.0
    for p in net.parameters():
        p.grad = None
    loss.backward()
    out["logits"] = logits.detach().numpy()
    out["loss"] = np.array(loss.item(), np.float32)
    for i, c in enumerate(convs):
        g = c.weight.grad.detach().numpy()
        out[f"gw{i}"] = g if g.size <= 8000 else g.reshape(-1)[::16].copy()
    out["g_bn1_w"] = net.bn1.weight.grad.numpy()
    out["g_bn4_b"] = net.bn4.bias.grad.numpy()
    # ... then the reference's own loop body (utils_own.forward) for the optimiser step; it only
    # steps once 128 samples have been seen, so feed the same 4 images 32 times.
    loader = [(x_lv.float() / 128, y)] * 32
    # the reference's accuracy() helper (utils.py:142-155) fails on this torch version (.view of a
    # non-contiguous tensor); it only feeds the printed metrics, so it is stubbed out here
    utils_own.accuracy = lambda output, target, topk=(1,): [torch.zeros(1) for _ in topk]
    utils_own.forward(loader, net, torch.nn.CrossEntropyLoss(), 0, training=True, optimizer=opt,
                      param_copy=param_copy, modules=net)
    out["fc1_weight_org_after"] = net.fc1.weight_org.numpy()
    out["conv1_weight_org_after"] = net.conv1.weight_org.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_tiny_cnn_step.npz"), **out)
    print("wrote ref_tiny_cnn_step.npz")


def make_guide_golden():
    """Gradients of the reference's own float guide functions (utils_functional.py:189-296), called with the weight
    split of conv2d_generic (:611-613) and differentiated by autograd on the CPU in fp32, for every accumulation
    mode and three small shapes each.  A fifth of the weights are exactly zero (both clamps have a kink there)
    and the upstream gradient is random.  Inputs are stored as levels (uint8 / int8, k/128)."""
    uf = ref_loader.reference_python()
    g = torch.Generator().manual_seed(77)
    shapes = [((2, 3, 7, 6), (4, 3, 3, 2), (1, 1), 2), ((1, 8, 6, 6), (5, 8, 3, 3), (0, 1), 4),
              ((3, 6, 5, 8), (9, 6, 2, 4), (2, 0), 3)]
    out, n = {}, 0
    for mode in ("full_or", "1d_bin", "z_bin", "yz_bin", "2d_bin", "full_bin"):
        for ashape, wshape, (pad_h, pad_w), z in shapes:
            a_lv = torch.randint(0, 128, ashape, generator=g, dtype=torch.int32)
            w_lv = torch.randint(-127, 128, wshape, generator=g, dtype=torch.int32)
            w_lv[torch.rand(wshape, generator=g) < 0.2] = 0
            a = (a_lv.float() / 128).requires_grad_(True)
            w = (w_lv.float() / 128 * 0.5).requires_grad_(True)          # multiples of 1/256: still exact in bf16
            ap = torch.nn.functional.pad(a, (pad_w, pad_w, pad_h, pad_h))
            w_pos, w_neg = w.clamp(0, 100), -(w.clamp(-100, 0))          # utils_functional.py:611-612
            if mode == "full_or":
                pos, neg = uf.conv2d_or_approx(ap, w_pos, (0, 0), (1, 1)), uf.conv2d_or_approx(ap, w_neg, (0, 0), (1, 1))
            elif mode == "full_bin":
                pos = torch.nn.functional.conv2d(ap, w_pos, padding=(0, 0), stride=(1, 1))
                neg = torch.nn.functional.conv2d(ap, w_neg, padding=(0, 0), stride=(1, 1))
            elif mode == "2d_bin":
                pos, neg = uf.conv2d_or_bin_2d(ap, w_pos, w_neg, (0, 0), (1, 1))
            elif mode == "1d_bin":
                pos, neg = uf.conv2d_or_bin_1d(ap, w_pos, w_neg, (0, 0), (1, 1))
            elif mode == "z_bin":
                pos, neg = uf.conv2d_or_bin_z(ap, w_pos, w_neg, (0, 0), (1, 1))
            else:
                pos, neg = uf.conv2d_or_bin_yz(ap, w_pos, w_neg, (0, 0), (1, 1), z)
            y = pos - neg
            go = torch.randn(y.shape, generator=g)
            ga, gw = torch.autograd.grad(y, (a, w), go)
            out[f"g{n}_meta"] = np.array([MODE_IDS[mode], pad_h, pad_w, z], np.int32)
            out[f"g{n}_a"] = a_lv.to(torch.uint8).numpy()
            out[f"g{n}_w2"] = w_lv.to(torch.int8).numpy()               # weight = level / 256
            out[f"g{n}_go"] = go.numpy()
            out[f"g{n}_ga"] = ga.numpy()
            out[f"g{n}_gw"] = gw.numpy()
            n += 1
    out["n"] = np.array(n)
    np.savez_compressed(os.path.join(HERE, "ref_guide_grads.npz"), **out)
    print(f"wrote ref_guide_grads.npz ({n} cases)")


MODE_IDS = {"1d_bin": 0, "z_bin": 1, "yz_bin": 2, "full_or": 3, "2d_bin": 4, "full_bin": 5}


if __name__ == "__main__":
    # python tests/golden/make_golden.py [all|forward|2d|full_bin|acc|rand|step|guide]: each part writes only its own fixture files
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("all", "forward"):
        main()
    if which in ("all", "2d"):
        make_2d_golden()
    if which in ("all", "full_bin"):
        make_full_bin_golden()
    if which in ("all", "acc"):
        make_acc_golden("acc")
    if which in ("all", "rand"):
        make_acc_golden("rand")
    if which in ("all", "step"):
        make_training_step_golden()
    if which in ("all", "guide"):
        make_guide_golden()
