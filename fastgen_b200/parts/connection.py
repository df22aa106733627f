"""Connections: how a sub-layer reads from and writes to the residual stream(s)."""

from __future__ import annotations

from typing import List

import torch

from .base import Connection, StreamUpdate, WeightSpec, register_connection
from .params import HyperConnectionParams


class HyperConnection(Connection):
    """Several residual streams instead of one ("hyper-connections").

    With streams ``x_0 .. x_{S-1}`` (all equal to the embedding at the start), a sub-layer ``f``
    with tensors ``in`` [S], ``out`` [S] and ``mix`` [S, S] (indexed [from, to]) does

        u = sum_s in[s] x_s;  y = f(norm(u));  x_t <- sum_s mix[s, t] x_s + out[t] y

    for all ``t`` at once from the old streams.  The coefficients are float32 and so is all of the
    arithmetic.  ``read`` is one kernel: the update the sub-layer before left pending, ``u`` and
    its norm (the norm must offer ``streams_forward``, as the layer norm does).
    """

    params: HyperConnectionParams

    def weight_specs(self) -> List[WeightSpec]:
        s = self.params.streams
        return [
            WeightSpec(self.names["in"], (s,), ("uniform", 0.3, 0.9)),
            WeightSpec(self.names["out"], (s,), ("uniform", 0.5, 1.0)),
            WeightSpec(self.names["mix"], (s, s), ("uniform", 0.1, 0.7)),
        ]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        self.in_coef = tensors["in"].float().contiguous()
        self.out_coef = tensors["out"].float().contiguous()
        self.mix = tensors["mix"].float().contiguous()

    def read(self, h, pending, norm):
        if pending is not None and not isinstance(pending, StreamUpdate):
            raise TypeError("a hyper-connection follows sub-layers that write to the streams through one")
        return norm.streams_forward(h, update=pending, in_coef=self.in_coef)

    def write(self, delta: torch.Tensor) -> StreamUpdate:
        return StreamUpdate(delta, self.mix, self.out_coef)


register_connection("hyper", HyperConnection)
