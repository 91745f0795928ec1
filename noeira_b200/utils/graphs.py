"""Whole-step CUDA-graph capture.

A training step of the convolutional / transformer models issues thousands of small kernels (3875 for ACT at
batch 8); launched one by one from Python the step is bounded by launch issue, not by the GPU.  ``GraphedStep``
runs a static-shape step function a few times eagerly on one private stream (lazy allocations, kernel attribute
set-up, workspaces), captures it once on that same stream and afterwards replays it: one launch per step.
The reference captures its update step the same way (noeira/nn/core/cuda_graph.mojo; ``capture_recast`` /
``rng_stream`` attributes of noeira/nn/core/module.mojo:135-152 exist to make its modules capturable).

Requirements on ``fn``: static shapes, no host synchronisation (``.item()``, ``.cpu()``), random numbers only
from counter-hash kernels (``nn.Dropout``, ``nn.advance_rng``) or from ``torch.Generator`` objects passed in
``generators`` (their offsets are then advanced per replay by the graph).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .. import _native


class GraphedStep:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], generators: Sequence[torch.Generator] = (),
                 warmup: int = 2):
        self.fn = fn
        self.static_inputs = [t.clone() for t in example_inputs]
        self.stream = torch.cuda.Stream(device=self.static_inputs[0].device if self.static_inputs else None)
        self.graph = None
        self.generators = list(generators)
        self.warmup = warmup
        self.launches = 0
        self.outputs = None
        self._calls = 0

    def _copy_in(self, inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if src is not dst:
                dst.copy_(src, non_blocking=True)

    def __call__(self, *inputs):
        assert len(inputs) == len(self.static_inputs)
        self._copy_in(inputs)
        if self.graph is not None:
            self.graph.replay()
            _native.add_launches(self.launches)
            return self.outputs
        s = self.stream
        s.wait_stream(torch.cuda.current_stream())
        if self._calls < self.warmup:
            with torch.cuda.stream(s):
                self.outputs = self.fn(*self.static_inputs)
            torch.cuda.current_stream().wait_stream(s)
            self._calls += 1
            return self.outputs
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        for gen in self.generators:
            g.register_generator_state(gen)
        n0 = _native.launch_count()
        with torch.cuda.graph(g, stream=s):
            self.outputs = self.fn(*self.static_inputs)
        self.launches = _native.launch_count() - n0
        _native.add_launches(-self.launches)      # the capture pass itself launched nothing
        self.graph = g
        g.replay()
        _native.add_launches(self.launches)
        return self.outputs
