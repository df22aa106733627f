"""Embedders: from token ids to the first residual stream."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Embedder, StateSpec, WeightSpec, register_embedder
from .params import BigramHashParams, TableEmbeddingParams


class TableEmbedding(Embedder):
    """``x = table[token] * scale`` (F.embedding of fastgen/forward.py:403-410; the scale is a
    float32 product).  An output of [T, S, dim] receives the row S times."""

    params: TableEmbeddingParams

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        return [WeightSpec(self.names["table"], (p.vocab_size, p.dim))]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        self.weight = tensors["table"].to(ops.act_dtype).contiguous()

    def table(self) -> torch.Tensor:
        return self.weight

    def forward(self, ctx, state, out):
        return self.ops.embedding(self.weight, ctx.tokens, out, scale=self.params.scale)


class BigramHashEmbedding(Embedder):
    """``x = table[token] + bigram[hash(previous token, token)]``.

    The hash is ``(previous * mul_prev + token * mul_cur) mod buckets``; a sequence's first
    token takes the bigram table's last row.  The previous token of a token that opens a step
    is the request's state: one int32 per slot, kept on the device, read and then advanced by
    the kernel, so that it follows decode graphs and runs of steps whose tokens never visit
    the host.  A request that is preempted and recomputed starts again at position 0, where
    the state is not read.
    """

    params: BigramHashParams

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        return [
            WeightSpec(self.names["table"], (p.vocab_size, p.dim)),
            WeightSpec(self.names["bigram"], (p.buckets + 1, p.dim)),
        ]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((1,), torch.int32)

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        self.weight = tensors["table"].to(ops.act_dtype).contiguous()
        self.bigram = tensors["bigram"].to(ops.act_dtype).contiguous()

    def table(self) -> torch.Tensor:
        return self.weight

    def forward(self, ctx, state, out):
        p = self.params
        return self.ops.embedding_bigram(self.weight, self.bigram, ctx.tokens, ctx.pos, ctx.req, state.view(-1), out,
                                         p.buckets, p.mul_prev, p.mul_cur)


register_embedder("table", TableEmbedding)
register_embedder("bigram_hash", BigramHashEmbedding)
