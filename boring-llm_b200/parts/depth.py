"""What the next layer reads when it is not simply the stream the last layer left."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights import TensorSpec, NORM
from .base import Part


class DepthWeightedAverage(Part):
    """out = sum_{j < n} weight[j] * X_j over the streams so far: X_0 the embedding rows, X_(i+1) what layer i left.
    One such part stands behind every layer (n = i + 2 behind layer i); the sum is 32-bit, in ascending j."""

    def __init__(self, n_inputs: int, names: Dict[str, str]):
        super().__init__(names)
        self.n = int(n_inputs)
        self.weight = None

    def local_specs(self):
        return {"weight": TensorSpec((self.n,), NORM)}

    def forward(self, ctx, streams: torch.Tensor, out: torch.Tensor) -> None:
        ops.depth_mix(streams, self.weight, self.n, out)


class AfterBlock:
    """What a model with a `DepthWeightedAverage` behind every block wants done once a block has left its stream: the
    average of the streams so far into `out`, and (if the next block begins with a norm) that norm's rows. A block whose
    last kernel works row by row may do both there and set `done`; else the model calls `run_unfused`."""

    def __init__(self, mix: DepthWeightedAverage, streams: torch.Tensor, out: torch.Tensor, next_norm=None):
        self.mix, self.streams, self.out, self.next_norm = mix, streams, out, next_norm
        self.done = False

    def run_unfused(self, ctx) -> None:
        if not self.done:
            self.mix.forward(ctx, self.streams, self.out)
            self.done = True
