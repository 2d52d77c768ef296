"""CUDA-graph replay of one stage's forward and backward for one micro-batch slot.

A pipeline stage runs a few thousand small kernels per micro-batch; launched eagerly from Python the stage is
bound by the host, not by the GPU, and the more stages a model is cut into the worse that gets (the work per
stage shrinks, the launch cost per kernel does not). ``GraphedFn`` captures ``outs = fn(*inputs)`` and the
matching backward as two CUDA graphs over static buffers and exposes them as ONE autograd node: forward copies
the inputs into the static inputs and replays the first graph, backward copies the incoming gradients and
replays the second, which also hands every parameter gradient to ``grad_sink`` INSIDE the graph (for the LM
stages: an in-place add into the flat fp32 gradient buffer), so a micro-batch costs two graph launches.

A 1F1B stage has several micro-batches in flight (forward done, backward pending); each needs its own saved
activations, so the schedule owns one ``GraphedFn`` per in-flight SLOT, each with a private memory pool, and
uses slot ``mb % slots``. A slot is only reused after its backward has run, which also makes it safe to send
straight out of the static output / input-gradient buffers: the neighbour has consumed a buffer long before the
slot's next replay overwrites it.

The torch helper ``torch.cuda.make_graphed_callables`` does the same for modules whose parameter gradients are
returned to autograd; it shares one pool between callables on the assumption that they run in capture order,
which a pipeline schedule does not do. Architecture-free: nothing here knows about language models.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch


class _Replay(torch.autograd.Function):
    @staticmethod
    def forward(ctx, graphed: "GraphedFn", _anchor, *inputs):
        for static, given in zip(graphed.static_in, inputs):
            if static.data_ptr() != given.data_ptr():
                static.copy_(given)
        graphed.fwd.replay()
        ctx.graphed = graphed
        return tuple(o.detach() for o in graphed.static_out)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *grads):
        g = ctx.graphed
        for static, given in zip(g.static_gout, grads):
            if static is None:
                continue
            if given is None:
                static.zero_()
            elif static.data_ptr() != given.data_ptr():
                static.copy_(given)
        g.bwd.replay()
        gins = iter(g.static_gin)
        return (None, None) + tuple(next(gins).detach() if s.requires_grad else None for s in g.static_in)


class GraphedFn:
    """``fn(*inputs) -> tensor or tuple of tensors`` captured for replay. ``params``: the parameters ``fn`` reads
    (their gradients go to ``grad_sink(param, grad)``, called once per parameter whose gradient autograd
    returns, inside the captured backward). Floating-point inputs are differentiable, others are not."""

    def __init__(self, fn: Callable, sample_inputs: Sequence[torch.Tensor], params: Sequence[torch.nn.Parameter],
                 grad_sink: Callable[[torch.nn.Parameter, torch.Tensor], None], warmup: int = 2):
        self.params = [p for p in params if p.requires_grad]
        self.static_in = [t.detach().clone().requires_grad_(t.is_floating_point()) for t in sample_inputs]
        device = self.params[0].device if self.params else self.static_in[0].device
        # the node needs one differentiable input even when the stage takes none (the first stage reads tokens)
        self.anchor = torch.zeros(1, device=device, requires_grad=True)
        diff_in = [t for t in self.static_in if t.requires_grad]
        targets = diff_in + self.params

        def run():
            out = fn(*self.static_in)
            return tuple(out) if isinstance(out, (tuple, list)) else (out,)

        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                outs = run()
                live = [o for o in outs if o.requires_grad]
                grads = torch.autograd.grad(live, targets, [torch.zeros_like(o) for o in live], allow_unused=True)
                for p, g in zip(self.params, grads[len(diff_in):]):
                    if g is not None:
                        grad_sink(p, g)
                del outs, live, grads
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)

        pool = torch.cuda.graph_pool_handle()
        self.fwd, self.bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.fwd, pool=pool):
            self.static_out = run()
        live = [o for o in self.static_out if o.requires_grad]
        self.static_gout = [torch.zeros_like(o) if o.requires_grad else None for o in self.static_out]
        with torch.cuda.graph(self.bwd, pool=pool):
            grads = torch.autograd.grad(live, targets, [g for g in self.static_gout if g is not None],
                                        allow_unused=True)
            for p, g in zip(self.params, grads[len(diff_in):]):
                if g is not None:
                    grad_sink(p, g)
        self.static_gin = [g if g is not None else torch.zeros_like(t) for g, t in zip(grads[:len(diff_in)], diff_in)]

    def __call__(self, *inputs: torch.Tensor):
        return _Replay.apply(self, self.anchor, *inputs)
