"""Capture-once / replay-many execution of shape-stable, autograd-free functions.

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
