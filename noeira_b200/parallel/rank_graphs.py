"""Captured multi-rank steps.

With one process per GPU every rank captures ITS OWN step graph (``utils.graphs.GraphedStep``); the collectives inside
are kernels that meet on device-side signals with monotone counters, so replays need no host rendezvous.  What must be
common across ranks is the *moment* of capture (a rank replaying a graph while its peer still runs eagerly would
interleave differently sized kernels on the signal pads): ``RankGraph`` puts a barrier before the capture call and
exposes ``captured`` so that drivers can assert that all ranks switched together.
(Reference: ``RankGraphs`` opens a capture on every GPU's stream at once inside one process and replays all graphs
back-to-back, noeira/nn/distributed/rank_graphs.mojo:17-21,50-129.)
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from ..utils.graphs import GraphedStep


class RankGraph:
    def __init__(self, step_fn: Callable, example_inputs: Sequence[torch.Tensor], comm=None, generators=(), warmup: int = 2):
        self.comm = comm
        self.step = GraphedStep(step_fn, example_inputs, generators=generators, warmup=warmup)

    @property
    def captured(self) -> bool:
        return self.step.graph is not None

    def __call__(self, *inputs):
        about_to_capture = (not self.captured) and self.step._calls >= self.step.warmup
        if about_to_capture and self.comm is not None:
            self.comm.barrier()
        out = self.step(*inputs)
        if about_to_capture and self.comm is not None:
            self.comm.barrier()
        return out
