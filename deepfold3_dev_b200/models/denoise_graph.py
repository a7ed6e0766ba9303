"""CUDA-graph replay of the denoiser inside the sampling loops.

The EDM sampler evaluates the denoiser hundreds of times on tensors of one
fixed shape while everything it conditions on stays put. Eagerly each
evaluation is a few thousand launches of small kernels, so the loop is bound by
launch latency. A ``GraphedDenoiser`` owns placeholder copies of the noisy
positions, the noise level and the whole conditioning state
(``DiffusionStatic``, a tree of dataclasses and tensors), runs the denoiser
once eagerly on them (lazy set-up inside the kernels happens there), captures a
second run into a CUDA graph and from then on replays it: new values are copied
into the placeholders, the graph runs, the result is read from the captured
output.

Graphs are kept per shape signature (a few, least recently used first out) in
one shared memory pool, so a training run with a fixed crop size captures once
and replays in every later step; the parameters are read in place, and the
bf16 casts of the weights are part of the graph (weight-cast caches are
bypassed while capturing, a cached cast would be a dangling pointer in later
replays). Used only without autograd; ``DF3_GRAPH_SAMPLER=0`` switches it off.
"""

from __future__ import annotations

import collections
import os

import torch

from ..utils.cuda_graph import tree_map, tree_signature, tree_tensors

MAX_GRAPHS = 3


def enabled(example: torch.Tensor) -> bool:
    return example.is_cuda and not torch.is_grad_enabled() and os.environ.get("DF3_GRAPH_SAMPLER", "1") != "0"


class GraphedDenoiser:
    """``fn(pos, noise_level, static)`` captured once on placeholder inputs and replayed."""

    def __init__(self, fn, pos, noise_level, static, pool):
        self.fn = fn
        self.pos, self.noise_level = pos.clone(), noise_level.clone()
        self.static = tree_map(lambda t: t.clone(), static)
        self._static_tensors = tree_tensors(self.static)
        self.graph, self.out = None, None
        amp = torch.is_autocast_enabled("cuda")
        ctx = (lambda: torch.autocast("cuda", dtype=torch.get_autocast_dtype("cuda"), cache_enabled=False)) if amp else None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if ctx:
                with ctx():
                    fn(self.pos, self.noise_level, self.static)
            else:
                fn(self.pos, self.noise_level, self.static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=pool):
            if ctx:
                with ctx():
                    self.out = fn(self.pos, self.noise_level, self.static)
            else:
                self.out = fn(self.pos, self.noise_level, self.static)
        self.graph = graph

    def load_static(self, static) -> None:
        for dst, src in zip(self._static_tensors, tree_tensors(static)):
            dst.copy_(src)

    def __call__(self, pos, noise_level):
        self.pos.copy_(pos)
        self.noise_level.copy_(noise_level)
        self.graph.replay()
        return self.out.clone()


class DenoiserGraphs:
    """Per-module cache of captured denoisers, keyed by the shapes of everything they read."""

    def __init__(self):
        self._graphs: collections.OrderedDict = collections.OrderedDict()
        self._pool = None
        self.failed = False

    def get(self, fn, pos, noise_level, static):
        """A callable ``(pos, noise_level) -> denoised`` bound to ``static``; eager if capture is not possible."""
        if self.failed:
            return lambda p, n: fn(p, n, static)
        key = (tuple(pos.shape), pos.dtype, tuple(noise_level.shape), torch.is_autocast_enabled("cuda"),
               tree_signature(static))  # fmt: skip
        g = self._graphs.get(key)
        if g is None:
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            while len(self._graphs) >= MAX_GRAPHS:
                self._graphs.popitem(last=False)
            try:
                g = GraphedDenoiser(fn, pos, noise_level, static, self._pool)
            except Exception:  # noqa: BLE001 - something in the denoiser cannot be captured: stay eager from now on
                torch.cuda.synchronize()
                self.failed = True
                return lambda p, n: fn(p, n, static)
            self._graphs[key] = g
        else:
            self._graphs.move_to_end(key)
            g.load_static(static)
        return g
