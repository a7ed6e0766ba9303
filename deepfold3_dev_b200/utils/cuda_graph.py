"""Capture-once / replay-many execution of shape-stable functions: autograd-free ones (``GraphCache``) and, for
training, a forward graph plus a backward graph behind one autograd node (``TrainGraphCache``).

``GraphCache.run(fn, inputs)`` evaluates ``fn(**inputs)`` (a tree of tensors in, a tree of tensors out). The first
call for a given shape signature runs ``fn`` eagerly once (lazy set-up inside kernels happens there), captures a
second run into a CUDA graph on private placeholder copies of the inputs and keeps it; later calls copy the new
inputs into the placeholders, replay, and return clones of the captured outputs. A few graphs are kept (least
recently used first out) in one shared memory pool.

What makes a function capturable here: no host reads of device values, no data-dependent shapes, parameters read in
place (the bf16 weight mirror of the flat optimizer is persistent memory), weight-cast caches bypassed while
capturing, and dropout seeds taken from a device-resident base seed (``GraphSeed``) that is refreshed before every
replay, so each replay draws new masks.
"""

from __future__ import annotations

import collections
import dataclasses

import torch


def tree_map(fn, obj):
    """Apply ``fn`` to every tensor of a tree of dataclasses / dicts / lists / tuples; other leaves pass through."""
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return dataclasses.replace(obj, **{f.name: tree_map(fn, getattr(obj, f.name)) for f in dataclasses.fields(obj)})
    if isinstance(obj, dict):
        return {k: tree_map(fn, v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(tree_map(fn, v) for v in obj)
    return obj


def tree_tensors(obj) -> list:
    out: list = []
    tree_map(lambda t: out.append(t) or t, obj)
    return out


def tree_signature(obj) -> tuple:
    sig: list = []

    def visit(o):
        if isinstance(o, torch.Tensor):
            sig.append((tuple(o.shape), o.dtype))
        elif dataclasses.is_dataclass(o) and not isinstance(o, type):
            for f in dataclasses.fields(o):
                visit(getattr(o, f.name))
        elif isinstance(o, dict):
            for k in sorted(o):
                sig.append(k)
                visit(o[k])
        elif isinstance(o, (list, tuple)):
            for v in o:
                visit(v)
        else:
            sig.append(o if isinstance(o, (int, float, bool, str, type(None))) else type(o).__name__)

    visit(obj)
    return tuple(sig)


class GraphSeed:
    """Device-resident base seed for dropout inside a captured region; ``offset()`` numbers the draws in call order."""

    current: "GraphSeed | None" = None

    def __init__(self, device):
        self.tensor = torch.zeros(1, dtype=torch.int64, device=device)
        self.count = 0

    def offset(self) -> int:
        self.count += 1
        return self.count * 0x9E3779B1

    def refresh(self) -> None:
        self.tensor.fill_(int(torch.randint(0, 2**31 - 1, (1,)).item()))

    def __enter__(self):
        self._prev, GraphSeed.current = GraphSeed.current, self
        self.count = 0
        return self

    def __exit__(self, *exc):
        GraphSeed.current = self._prev
        return False


class CapturedCall:
    def __init__(self, fn, inputs: dict, pool):
        self.inputs = tree_map(lambda t: t.clone(), inputs)
        self._in = tree_tensors(self.inputs)
        self.seed = GraphSeed(self._in[0].device)
        amp = torch.is_autocast_enabled("cuda")

        def call():
            with self.seed:
                if amp:
                    with torch.autocast("cuda", dtype=torch.get_autocast_dtype("cuda"), cache_enabled=False):
                        return fn(**self.inputs)
                return fn(**self.inputs)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.seed.refresh()
            call()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool):
            self.outputs = call()

    def __call__(self, inputs: dict):
        for dst, src in zip(self._in, tree_tensors(inputs)):
            dst.copy_(src)
        self.seed.refresh()
        self.graph.replay()
        return tree_map(lambda t: t.clone(), self.outputs)


class GraphCache:
    def __init__(self, max_graphs: int = 3):
        self.max_graphs = max_graphs
        self._graphs: collections.OrderedDict = collections.OrderedDict()
        self._pool = None
        self.failed = False
        self.error: Exception | None = None

    def run(self, fn, inputs: dict, mode=None):
        """``mode``: anything else the captured work depends on (for a module: its training flag)."""
        if self.failed:
            return fn(**inputs)
        key = (mode, torch.is_autocast_enabled("cuda"), tree_signature(inputs))
        g = self._graphs.get(key)
        if g is None:
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            while len(self._graphs) >= self.max_graphs:
                self._graphs.popitem(last=False)
            try:
                g = CapturedCall(fn, inputs, self._pool)
            except Exception as exc:  # noqa: BLE001 - something in fn cannot be captured: stay eager from now on
                torch.cuda.synchronize()
                self.failed, self.error = True, exc
                import logging

                logging.getLogger(__name__).warning("CUDA graph capture failed, running eagerly: %r", exc)
                return fn(**inputs)
            self._graphs[key] = g
        else:
            self._graphs.move_to_end(key)
        return g(inputs)


class GraphedTrainCall:
    """``fn(**inputs) -> dict`` with autograd, executed as two CUDA graphs.

    The forward of ``fn`` is captured once with autograd recording, then ``torch.autograd.grad`` of its outputs with
    respect to the inputs that require grad and to ``params`` is captured as a second graph (the scheme of
    ``torch.cuda.make_graphed_callables``). Inside the backward graph the parameter gradients are added to
    ``param.grad`` (views of the flat gradient buffer), so a step costs two graph launches instead of tens of
    thousands of kernel launches and autograd-node dispatches. Activations live in the graph's memory pool between
    the two replays. Dropout masks follow a device-resident seed that is refreshed before each forward replay; the
    backward replay regenerates the same masks from it.
    """

    def __init__(self, fn, inputs: dict, params, pool):
        dev = next(t for t in inputs.values() if isinstance(t, torch.Tensor)).device
        self.params = [p for p in params if p.requires_grad]
        for p in self.params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        self.static_in = {}
        for k, v in inputs.items():
            if isinstance(v, torch.Tensor):
                c = v.detach().clone()
                if v.requires_grad:
                    c.requires_grad_(True)
                self.static_in[k] = c
            else:
                self.static_in[k] = v
        self.tensor_keys = [k for k, v in inputs.items() if isinstance(v, torch.Tensor)]
        self.grad_keys = [k for k in self.tensor_keys if inputs[k].requires_grad]
        self.seed = GraphSeed(dev)
        amp = torch.is_autocast_enabled("cuda")
        amp_dtype = torch.get_autocast_dtype("cuda") if amp else None

        def call():
            with self.seed:
                if amp:
                    with torch.autocast("cuda", dtype=amp_dtype, cache_enabled=False):
                        return fn(**self.static_in)
                return fn(**self.static_in)

        def split(out):
            passthrough = {k: next(ik for ik in self.tensor_keys if self.static_in[ik] is v) for k, v in out.items()
                           if isinstance(v, torch.Tensor) and any(self.static_in[ik] is v for ik in self.tensor_keys)}  # fmt: skip
            req = [k for k, v in out.items() if isinstance(v, torch.Tensor) and k not in passthrough and v.requires_grad]
            return passthrough, req

        grad_targets = [self.static_in[k] for k in self.grad_keys] + self.params
        # one eager forward + backward first: lazy set-up inside kernels (function attributes, caches) happens here
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.seed.refresh()
            out = call()
            _, req = split(out)
            g = torch.autograd.grad([out[k] for k in req], grad_targets, [torch.zeros_like(out[k]) for k in req], allow_unused=True)
            del out, g
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()  # the eager activations go back to the driver before the graph pool takes as much again
        self.fwd_graph, self.bwd_graph = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.fwd_graph, pool=pool):
            self.static_out = call()
        self.passthrough, self.out_req = split(self.static_out)
        self.static_gout = [torch.zeros_like(self.static_out[k]) for k in self.out_req]
        with torch.cuda.graph(self.bwd_graph, pool=pool if pool is not None else self.fwd_graph.pool()):
            grads = torch.autograd.grad([self.static_out[k] for k in self.out_req], grad_targets, self.static_gout, allow_unused=True)
            n_in = len(self.grad_keys)
            self.static_gin = list(grads[:n_in])
            dst = [p.grad for p, g in zip(self.params, grads[n_in:]) if g is not None]
            src = [g for g in grads[n_in:] if g is not None]
            if dst:
                torch._foreach_add_(dst, src)
        self.param_grad_ptrs = [p.grad.data_ptr() for p in self.params]

    def stale(self) -> bool:
        """The gradient buffers the backward graph writes moved (optimizer rebuilt, gradients adopted elsewhere)."""
        return any(p.grad is None or p.grad.data_ptr() != ptr for p, ptr in zip(self.params, self.param_grad_ptrs))

    def __call__(self, inputs: dict) -> dict:
        outs = _GraphedReplay.apply(self, inputs, *[inputs[k] for k in self.grad_keys])
        result = {}
        it = iter(outs)
        for k, v in self.static_out.items():
            if k in self.passthrough:
                result[k] = inputs[self.passthrough[k]]
            elif k in self.out_req:
                result[k] = next(it)
            else:
                result[k] = v.detach() if isinstance(v, torch.Tensor) else v
        return result


class _GraphedReplay(torch.autograd.Function):
    @staticmethod
    def forward(ctx, call: GraphedTrainCall, inputs: dict, *grad_inputs):
        for k in call.tensor_keys:
            call.static_in[k].detach().copy_(inputs[k])
        call.seed.refresh()
        call.fwd_graph.replay()
        ctx.call = call
        return tuple(call.static_out[k].detach() for k in call.out_req)

    @staticmethod
    def backward(ctx, *gouts):
        call = ctx.call
        for buf, g in zip(call.static_gout, gouts):
            if g is None:
                buf.zero_()
            else:
                buf.copy_(g)
        call.bwd_graph.replay()
        gin = [None if g is None else g.detach().clone() for g in call.static_gin]
        return (None, None, *gin)


class TrainGraphCache:
    """Graphed forward + backward of one module call per input signature (see ``GraphedTrainCall``); falls back to
    eager execution for good if a capture fails."""

    def __init__(self, max_graphs: int = 1):
        self.max_graphs = max_graphs
        self._graphs: collections.OrderedDict = collections.OrderedDict()
        self._pool = None
        self.failed = False
        self.error: Exception | None = None

    def run(self, fn, inputs: dict, params, mode=None):
        if self.failed:
            return fn(**inputs)
        # shapes, not dtypes: replay copies the inputs into the captured placeholders, which converts (the recycling
        # inputs arrive as fp32 zeros on a step without recycles and as bf16 activations otherwise)
        shapes = tuple((k, tuple(v.shape)) if isinstance(v, torch.Tensor) else (k, v if isinstance(v, (int, float, bool, str, type(None))) else type(v).__name__)
                       for k, v in sorted(inputs.items()))  # fmt: skip
        key = (mode, torch.is_autocast_enabled("cuda"), tuple(sorted(k for k, v in inputs.items() if isinstance(v, torch.Tensor) and v.requires_grad)),
               shapes)  # fmt: skip
        g = self._graphs.get(key)
        if g is not None and g.stale():
            del self._graphs[key]
            g = None
        if g is None:
            while len(self._graphs) >= self.max_graphs:
                self._graphs.popitem(last=False)
            try:
                # a pool of its own per capture: a pool whose last graph was dropped above cannot take new captures
                g = GraphedTrainCall(fn, inputs, list(params), torch.cuda.graph_pool_handle())
            except Exception as exc:  # noqa: BLE001 - something in fn cannot be captured: stay eager from now on
                import logging
                import traceback

                # keep the text only: the exception's traceback would pin every tensor of the failed attempt
                self.failed, self.error = True, "".join(traceback.format_exception(type(exc), exc, exc.__traceback__)[-6:])
                logging.getLogger(__name__).warning("CUDA graph capture of the training pass failed, running eagerly:\n%s", self.error)
                g = None
            if self.failed:  # outside the handler: the exception and the frames it holds are gone by now
                import gc

                torch.cuda.synchronize()
                gc.collect()
                torch.cuda.empty_cache()
                return fn(**inputs)
            self._graphs[key] = g
        else:
            self._graphs.move_to_end(key)
        return g(inputs)
