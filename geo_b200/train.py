"""One optimiser step of SC-CNN training, mirroring the loop body of the reference's
``utils_own.forward`` (utils_own.py:57-114): scaled cross-entropy loss, backward through the
guide, gradients copied to an fp32 master copy of the parameters, optimiser step on the master
copy, parameters copied back and ``weight_org`` refreshed (clamped to [-1, 0.999])."""
from __future__ import annotations

import torch
import torch.nn as nn

SCALE_FACTOR = 128.0  # loss scale (utils_own.py:15,81)


class TrainStep:
    """Holds the model, the master parameter copy and the optimiser; ``__call__`` runs one step
    on a device batch and returns the (scaled) loss tensor.

    ``grad_hook`` is called with the list of parameters after backward and before the gradients
    are copied to the master copy: the data-parallel wrapper all-reduces them there."""

    def __init__(self, model, lr=2e-3, optim="SGD", grad_hook=None, graph=False):
        self.model = model
        self.criterion = nn.CrossEntropyLoss()
        self.param_copy = [p.clone().float().detach().requires_grad_(True) for p in model.parameters()]
        if optim == "SGD":      # main_conv.py:216-217
            self.optimizer = torch.optim.SGD(self.param_copy, lr=lr, weight_decay=0, momentum=0.01)
        elif optim == "Adam":   # main_conv.py:212-213
            self.optimizer = torch.optim.Adam(self.param_copy, lr=lr, weight_decay=0)
        else:
            raise ValueError(optim)
        self.grad_hook = grad_hook
        self.params = list(model.parameters())
        self.sc_modules = [m for m in model.modules() if hasattr(m, "weight_org")]
        # graph=True: the whole step (forward, backward, gradient exchange, optimiser) is captured
        # into one CUDA graph on first use and replayed afterwards; shapes must then stay fixed.
        self.use_graph = graph
        self._graph = None
        self._graph_update = None
        self._split_hook = False
        self._static = None

    def __call__(self, inputs, targets):
        if not self.use_graph:
            return self._step(inputs, targets)
        if self._graph is None:
            self._capture(inputs, targets)
        sx, sy, sloss, sout = self._static
        sx.copy_(inputs, non_blocking=True)
        sy.copy_(targets, non_blocking=True)
        self._graph.replay()
        if self._graph_update is not None:
            # the gradient exchange runs between the two graphs, outside any capture: collectives
            # inside a capture depend on the communication library's capture support and a rank
            # that fails to capture leaves its peers waiting
            if self._split_hook:
                self.grad_hook.reduce()
            else:
                self.grad_hook(self.params)
            self._graph_update.replay()
        return sloss, sout

    def _capture(self, inputs, targets):
        sx, sy = inputs.detach().clone(), targets.detach().clone()
        side = torch.cuda.Stream(device=sx.device)
        side.wait_stream(torch.cuda.current_stream(sx.device))
        with torch.cuda.stream(side):
            for _ in range(3):  # warm-up: lazy initialisation, optimiser state, allocator pools
                self._step(sx.clone(), sy)
        torch.cuda.current_stream(sx.device).wait_stream(side)
        torch.cuda.synchronize(sx.device)
        graph = torch.cuda.CUDAGraph()
        self._graph_update = None
        if self.grad_hook is None:
            with torch.cuda.graph(graph):
                sloss, sout = self._step(sx.clone(), sy)
        else:
            # a hook that offers pack / reduce / unpack keeps its copies inside the graphs
            hook = self.grad_hook
            self._split_hook = all(hasattr(hook, n) for n in ("pack", "reduce", "unpack"))
            with torch.cuda.graph(graph):
                sloss, sout = self._forward_backward(sx.clone(), sy)
                if self._split_hook:
                    hook.pack(self.params)
            if self._split_hook:
                hook.reduce()
            else:
                hook(self.params)
            update = torch.cuda.CUDAGraph()
            with torch.cuda.graph(update, pool=graph.pool()):
                if self._split_hook:
                    hook.unpack(self.params)
                self._update()
            self._graph_update = update
        self._graph = graph
        self._static = (sx, sy, sloss, sout)

    def _step(self, inputs, targets):
        out = self._forward_backward(inputs, targets)
        if self.grad_hook is not None:
            self.grad_hook(self.params)
        self._update()
        return out

    def _forward_backward(self, inputs, targets):
        model = self.model
        model.train()
        output = model(inputs)
        loss = self.criterion(output, targets) * SCALE_FACTOR
        for p in self.params:
            p.grad = None
        loss.backward()
        return loss.detach(), output.detach()

    def _update(self):
        with torch.no_grad():
            for m in self.sc_modules:
                m.weight.data.copy_(m.weight_org)
            for master, p in zip(self.param_copy, self.params):
                if p.grad is not None:
                    master.grad = p.grad.detach().to(torch.float32) / SCALE_FACTOR
            self.optimizer.step()
            for master, p in zip(self.param_copy, self.params):
                p.data.copy_(master.data)
            for m in self.sc_modules:
                m.weight_org.copy_(m.weight.data.clamp(-1, 0.999))
            self.optimizer.zero_grad(set_to_none=True)
