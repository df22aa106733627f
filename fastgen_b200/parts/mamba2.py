"""The state-space mixer in the Mamba-2 form."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, StateSpec, WeightSpec, register_mixer
from .params import Mamba2Params


class Mamba2(Mixer):
    """``wo(norm(y * silu(z)))`` with ``y`` the output of a linear recurrence over a matrix state.

    One projection ``w_in`` gives, per token, ``[z | x | B | C | dt]`` (``inner``, ``inner``,
    ``groups * state``, ``groups * state``, ``heads`` columns, ``inner = heads * head_dim``).
    x, B and C pass a causal convolution per channel (``conv`` taps, the last one on the current
    token, a bias) and SiLU.  Per head ``h`` of group ``h // (heads / groups)``, in float32:

        dt = softplus(dt + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x

    ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts of its columns and multiplied by
    ``norm``.  The request's state is fixed-size: S of every head and the convolution's last
    ``conv - 1`` inputs, one float32 row per slot that the cache manager zeroes on admission.
    The recurrence runs token by token in float32, so prompt portions, single tokens and mixed
    batches take the same kernels and give the same numbers however a prompt is cut.
    """

    params: Mamba2Params
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.ssm_floats = p.n_heads * p.state * p.head_dim
        self.conv_floats = (p.conv - 1) * p.channels

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self.names
        return [
            WeightSpec(n["w_in"], (2 * p.inner + 2 * p.groups * p.state + p.n_heads, p.dim)),
            WeightSpec(n["conv"], (p.channels, p.conv), ("normal", 0.3)),
            WeightSpec(n["conv_bias"], (p.channels,), ("normal", 0.1)),
            WeightSpec(n["dt_bias"], (p.n_heads,), ("uniform", -3.0, 0.5)),
            WeightSpec(n["a_log"], (p.n_heads,), ("uniform", -1.0, 1.5)),
            WeightSpec(n["d"], (p.n_heads,), ("ones",)),
            WeightSpec(n["norm"], (p.inner,), ("ones",)),
            WeightSpec(n["wo"], (p.dim, p.inner)),
        ]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.ssm_floats + self.conv_floats,))

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        dt = ops.act_dtype
        self.w_in = tensors["w_in"].to(dt).contiguous()
        self.wo = tensors["wo"].to(dt).contiguous()
        # small vectors enter float32 arithmetic: float32 whatever they were stored in
        self.conv_w = tensors["conv"].float().contiguous()
        self.conv_b = tensors["conv_bias"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.a_log = tensors["a_log"].float().contiguous()
        self.d = tensors["d"].float().contiguous()
        self.norm_w = tensors["norm"].float().contiguous()

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        state = memory.state
        proj = ops.linear(x, self.w_in)  # [T, z | x B C | dt]
        xbc = ops.mamba2_conv(proj, p.inner, p.channels, self.conv_w, self.conv_b, state, self.ssm_floats, p.conv, ctx)
        y = ops.mamba2_scan(xbc, proj, p.inner + p.channels, self.dt_bias, self.a_log, self.d, state, ctx,
                            p.n_heads, p.groups, p.state, p.head_dim)
        g = ops.gated_part_norm(y, proj[:, : p.inner], self.norm_w, p.norm_groups, p.eps, ctx)
        return ops.linear(g, self.wo)


register_mixer("mamba2", Mamba2)
