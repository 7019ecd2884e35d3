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
    are copied to the master copy: the data-parallel wrapper all-reduces them there.

    ``graph=True`` captures the step into CUDA graphs on the first call and replays them afterwards:
    * shapes must stay fixed, and the loss / output tensors returned are the graph's own buffers,
      overwritten by the next call (clone them to keep them);
    * the warm-up runs that capture needs are undone (parameters, master copy, optimiser state,
      ``weight_org`` and the batch-norm statistics are put back), so the first call applies exactly one
      step, as an eager call does;
    * the learning rate is read from a device scalar that is refreshed from
      ``optimizer.param_groups[0]['lr']`` before every replay, so schedulers keep working (SGD: the
      update is written out with that scalar; Adam is built with ``capturable=True`` and a tensor lr)."""

    def __init__(self, model, lr=2e-3, optim="SGD", grad_hook=None, graph=False):
        self.model = model
        self.criterion = nn.CrossEntropyLoss()
        self.param_copy = [p.clone().float().detach().requires_grad_(True) for p in model.parameters()]
        if optim == "SGD":      # main_conv.py:216-217
            self.optimizer = torch.optim.SGD(self.param_copy, lr=lr, weight_decay=0, momentum=0.01)
        elif optim == "Adam":   # main_conv.py:212-213
            if graph:   # the stock Adam reads its step count on the host; the capturable form does not
                dev = self.param_copy[0].device
                self.optimizer = torch.optim.Adam(self.param_copy, lr=torch.tensor(float(lr), device=dev),
                                                  weight_decay=0, capturable=True)
            else:
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
        self._lr_dev = None       # graph mode, SGD: the learning rate the captured update reads
        self._captured = False    # inside graph capture or its warm-up: SGD update written out

    def __call__(self, inputs, targets):
        if not self.use_graph:
            return self._step(inputs, targets)
        if self._graph is None:
            self._capture(inputs, targets)
        sx, sy, sloss, sout = self._static
        sx.copy_(inputs, non_blocking=True)
        sy.copy_(targets, non_blocking=True)
        self._refresh_lr()
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

    def _refresh_lr(self):
        """Copies the host learning rate into the device scalar of the captured SGD update."""
        if self._lr_dev is not None:
            lr = self.optimizer.param_groups[0]["lr"]
            if float(lr) != self._lr_host:
                self._lr_host = float(lr)
                self._lr_dev.fill_(self._lr_host)

    def _snapshot(self):
        model_state = {k: v.detach().clone() for k, v in list(self.model.named_parameters()) + list(self.model.named_buffers())
                       if v is not None}
        return model_state, [p.detach().clone() for p in self.param_copy]

    def _restore(self, snap):
        model_state, masters = snap
        with torch.no_grad():
            for k, v in list(self.model.named_parameters()) + list(self.model.named_buffers()):
                if v is not None and k in model_state:
                    v.copy_(model_state[k])
            for p, m in zip(self.param_copy, masters):
                p.copy_(m)
            # a fresh optimiser state: zero moments and step counts act exactly like no state at all
            for st in self.optimizer.state.values():
                for v in st.values():
                    if torch.is_tensor(v):
                        v.zero_()

    def _capture(self, inputs, targets):
        sx, sy = inputs.detach().clone(), targets.detach().clone()
        if isinstance(self.optimizer, torch.optim.SGD):
            self._lr_host = float(self.optimizer.param_groups[0]["lr"])
            self._lr_dev = torch.full((), self._lr_host, dtype=torch.float32, device=sx.device)
        self._captured = True
        snap = self._snapshot()
        side = torch.cuda.Stream(device=sx.device)
        side.wait_stream(torch.cuda.current_stream(sx.device))
        with torch.cuda.stream(side):
            for _ in range(3):  # warm-up: lazy initialisation, optimiser state, allocator pools
                self._step(sx.clone(), sy)
        torch.cuda.current_stream(sx.device).wait_stream(side)
        torch.cuda.synchronize(sx.device)
        self._restore(snap)     # the warm-up steps must not count as training
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
        # the loop body of utils_own.py:98-114, with the per-tensor copies, divisions and clamps batched into
        # multi-tensor calls (a handful of kernels instead of one per parameter)
        with torch.no_grad():
            if self.sc_modules:
                torch._foreach_copy_([m.weight.data for m in self.sc_modules], [m.weight_org for m in self.sc_modules])
            have = [(master, p.grad.detach()) for master, p in zip(self.param_copy, self.params) if p.grad is not None]
            if have:
                grads = [g if g.dtype == torch.float32 else g.to(torch.float32) for _, g in have]
                for (master, _), g in zip(have, torch._foreach_div(grads, SCALE_FACTOR)):
                    master.grad = g
            if self._plain_sgd():
                self._sgd_step(self._lr_dev if self._captured else float(self.optimizer.param_groups[0]["lr"]))
            else:
                self.optimizer.step()
            torch._foreach_copy_([p.data for p in self.params], [m.data for m in self.param_copy])
            if self.sc_modules:
                clamped = torch._foreach_clamp_min([m.weight.data for m in self.sc_modules], -1.0)
                torch._foreach_clamp_max_(clamped, 0.999)
                torch._foreach_copy_([m.weight_org for m in self.sc_modules], clamped)
                for m in self.sc_modules:
                    if hasattr(m, "invalidate_stream_cache"):
                        m.invalidate_stream_cache()
            self.optimizer.zero_grad(set_to_none=True)

    def _plain_sgd(self):
        if not isinstance(self.optimizer, torch.optim.SGD) or len(self.optimizer.param_groups) != 1:
            return False
        group = self.optimizer.param_groups[0]
        plain = group["weight_decay"] == 0 and group["dampening"] == 0 and not group["nesterov"] and not group.get("maximize")
        if self.use_graph and not plain:
            raise NotImplementedError("graph=True with SGD: plain momentum only (no weight decay, dampening, Nesterov)")
        return plain

    def _sgd_step(self, lr):
        """torch.optim.SGD's update for plain momentum (the settings of main_conv.py:216-217), written out so that
        the learning rate can be a device scalar: a captured graph then follows later changes of
        ``param_groups['lr']``.  Eager steps use the same arithmetic with the host value, so both launch modes
        give bit-identical parameters.  The momentum buffers live in ``optimizer.state`` as usual."""
        group = self.optimizer.param_groups[0]
        params = [p for p in self.param_copy if p.grad is not None]
        grads = [p.grad for p in params]
        momentum = group["momentum"]
        if momentum != 0:
            bufs = []
            for p in params:
                st = self.optimizer.state[p]
                if "momentum_buffer" not in st or st["momentum_buffer"] is None:
                    st["momentum_buffer"] = torch.zeros_like(p)   # zero buffer: first step gives buf = grad
                bufs.append(st["momentum_buffer"])
            torch._foreach_mul_(bufs, momentum)
            torch._foreach_add_(bufs, grads)
            grads = bufs
        torch._foreach_sub_(params, torch._foreach_mul(grads, lr))
