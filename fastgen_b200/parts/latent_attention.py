"""Attention whose keys and values are linear maps of a cached latent."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import CacheSpec, Mixer, WeightSpec, make_position, register_mixer
from .params import LatentAttentionParams


class LatentAttention(Mixer):
    """Causal softmax attention over a compressed cache.

    Per token ``c = rmsnorm(w_dkv[:R] x) * dkv_norm`` (``R = kv_rank``) and ``k_t = turn(w_dkv[R:] x)``
    (``rot_dim`` numbers, shared by all heads) are all that is cached: one pool, one entry a token.
    Queries: ``q = w_uq (rmsnorm(w_dq x) * dq_norm)``, per head ``[head_dim plain | rot_dim turned]``.
    Head ``h`` has keys ``[w_uk,h c | k_t]`` and values ``w_uv,h c``; its output is multiplied by
    ``sigmoid(w_g x)_h`` before ``wo``.

    Computed with the key map folded into the query: ``qa_h = w_uk,h^T q_plain,h`` makes the score
    ``(qa_h . c + q_turned,h . k_t) * scale``, the attention kernel sums latents instead of values
    and ``w_uv,h`` maps a head's summed latent to its output afterwards.  Nothing per head is ever
    made for a cached token, in prompts or in decoding.  The down projections (``w_dq``, ``w_dkv``,
    ``w_g``) run as one product.

    A layer with ``own_cache`` false has no ``w_dkv``: its run of the schedule reads the entries of
    the run it names (``ScheduleEntry.kv_from``), with its own ``w_uk`` and ``w_uv``.
    """

    params: LatentAttentionParams
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.position = make_position(p.position)
        self.qk = p.head_dim + p.rot_dim
        # entries are padded to 16 bytes in both compute types
        self.entry = -(-(p.kv_rank + p.rot_dim) // 8) * 8

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self.names
        specs = [
            WeightSpec(n["w_dq"], (p.q_rank, p.dim)),
            WeightSpec(n["dq_norm"], (p.q_rank,), ("ones",)),
            WeightSpec(n["w_uq"], (p.n_heads * self.qk, p.q_rank)),
        ]
        if p.own_cache:
            specs += [
                WeightSpec(n["w_dkv"], (p.kv_rank + p.rot_dim, p.dim)),
                WeightSpec(n["dkv_norm"], (p.kv_rank,), ("ones",)),
            ]
        specs += [
            WeightSpec(n["w_uk"], (p.n_heads * p.head_dim, p.kv_rank)),
            WeightSpec(n["w_uv"], (p.n_heads * p.v_head_dim, p.kv_rank)),
        ]
        if p.gate:
            specs.append(WeightSpec(n["w_g"], (p.n_heads, p.dim)))
        specs.append(WeightSpec(n["wo"], (p.dim, p.n_heads * p.v_head_dim)))
        return specs

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(1, self.entry, None, n_pools=1)

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        # one down projection: [w_dq; w_g; w_dkv] (the gate's rows padded to a multiple of 8 so that
        # the parts start on 16 bytes)
        self.gate_rows = -(-p.n_heads // 8) * 8 if p.gate else 0
        parts = [tensors["w_dq"]]
        if p.gate:
            g = tensors["w_g"]
            parts.append(torch.cat([g, g.new_zeros((self.gate_rows - p.n_heads, p.dim))], dim=0))
        if p.own_cache:
            parts.append(tensors["w_dkv"])
        self.w_down = torch.cat(parts, dim=0).to(dt).contiguous()
        self.dq_norm = tensors["dq_norm"].float().contiguous()
        self.dkv_norm = tensors["dkv_norm"].float().contiguous() if p.own_cache else None
        self.w_uq = tensors["w_uq"].to(dt).contiguous()
        self.w_uk = tensors["w_uk"].to(dt).reshape(p.n_heads, p.head_dim, p.kv_rank).contiguous()
        self.w_uv = tensors["w_uv"].to(dt).reshape(p.n_heads, p.v_head_dim, p.kv_rank).contiguous()
        # the float32 product takes [out, in] operands: the key map transposed per head
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous() if dt == torch.float32 else None
        self.w_uv_t = self.w_uv.transpose(1, 2).contiguous() if dt == torch.bfloat16 else None
        self.wo = tensors["wo"].to(dt).contiguous()
        self.freqs = self.position.table(ops.device)
        if self.freqs is None:
            self.freqs = torch.zeros(max(1, p.rot_dim // 2), dtype=torch.float32, device=ops.device)
        self.magnitude = float(getattr(self.position, "magnitude", lambda: 1.0)())

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        t, H, R = x.shape[0], p.n_heads, p.kv_rank
        down = ops.linear(x, self.w_down)
        o0 = p.q_rank
        gate = down[:, o0 : o0 + H] if p.gate else None
        o0 += self.gate_rows
        if memory.writes:
            ops.latent_entry_write(down[:, o0 : o0 + R + p.rot_dim], self.dkv_norm, p.eps, self.freqs,
                                   self.magnitude, memory, ctx, R, p.rot_dim)
        cq = ops.rms_rows(down[:, : p.q_rank], self.dq_norm, p.eps)
        q = ops.linear(cq, self.w_uq).view(t, H, self.qk)
        ops.rotate_part(q.view(t, H * self.qk), ctx, self.freqs, self.magnitude, H, self.qk, p.head_dim, p.rot_dim)
        # the key map folded into the queries: qa[h] = q_plain[h] @ w_uk[h]
        qa = ops.head_products(q[:, :, : p.head_dim], self.w_uk, self.w_uk_t)  # [H, T, R]
        lat = torch.empty((H, t, R), dtype=x.dtype, device=x.device)
        ops.latent_attention(qa, q[:, :, p.head_dim :], lat, gate, memory, ctx, H, R, p.rot_dim, p.softmax_scale)
        # a head's summed latent through its value map, heads side by side for wo
        o = torch.empty((t, H, p.v_head_dim), dtype=x.dtype, device=x.device)
        ops.head_products_out(lat, self.w_uv, self.w_uv_t, o)
        return ops.linear(o.view(t, H * p.v_head_dim), self.wo)


register_mixer("latent_attention", LatentAttention)
