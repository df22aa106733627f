"""Position encodings: rotary (with llama3 frequency scaling) and none."""

from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, register_position
from .params import NoPositionParams, RopeParams, YarnScaling


def rope_frequencies(params: RopeParams) -> torch.Tensor:
    """Float32 table of ``head_dim/2`` rotation frequencies.

    ``freq_j = theta ** -(2j / head_dim)``; with llama3 scaling a frequency whose
    wavelength ``2*pi/freq`` exceeds ``old_ctx/low`` is divided by ``factor``, one
    between ``old_ctx/high`` and ``old_ctx/low`` is blended
    ``(1-x)*freq/factor + x*freq`` with ``x = (old_ctx/wavelen - low)/(high - low)``,
    and shorter wavelengths are kept (fastgen/forward.py:609-635).  All
    arithmetic is float32 tensor arithmetic, as there.
    """
    hd = params.rot_dims or params.head_dim
    pows = torch.arange(0, hd, 2, dtype=torch.float32) / hd
    freqs = 1.0 / (params.theta ** pows)
    if params.linear_factor is not None:
        freqs = freqs / params.linear_factor
    sc = params.scaling
    if sc is None:
        return freqs
    if isinstance(sc, YarnScaling):
        def turn_dim(turns: float) -> float:
            return hd * math.log(sc.original_max_positions / (2 * math.pi * turns)) / (2 * math.log(params.theta))

        lo = max(math.floor(turn_dim(sc.fast)), 0)
        hi = min(math.ceil(turn_dim(sc.slow)), hd - 1)
        ramp = ((torch.arange(hd // 2, dtype=torch.float32) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return freqs / sc.factor * ramp + freqs * (1.0 - ramp)
    wavelen = (2 * math.pi) / freqs
    low_wavelen = sc.original_max_positions / sc.low_freq_factor
    high_wavelen = sc.original_max_positions / sc.high_freq_factor
    x = sc.original_max_positions / wavelen - sc.low_freq_factor
    x = x / (sc.high_freq_factor - sc.low_freq_factor)
    blended = (1 - x) * freqs / sc.factor + x * freqs
    out = torch.where(wavelen > low_wavelen, freqs / sc.factor, freqs)
    mid = (wavelen >= high_wavelen) & (wavelen <= low_wavelen)
    return torch.where(mid, blended, out)


class Rope(PositionEncoding):
    """Rotation of adjacent pairs ``(x[2j], x[2j+1])`` by ``pos * freq_j``
    (fastgen/kernels/rope.py:57-89).  The kernels are table-driven, so another
    frequency law is another ``table()``.  ``magnitude()`` is the number cosine and sine are
    both multiplied by (1 unless the scaling says otherwise)."""

    params: RopeParams

    def magnitude(self) -> float:
        sc = self.params.scaling
        if isinstance(sc, YarnScaling):
            return 0.1 * math.log(sc.factor) + 1.0
        return 1.0

    def __init__(self, spec) -> None:
        super().__init__(spec)
        self._table: Optional[torch.Tensor] = None

    def table(self, device) -> Optional[torch.Tensor]:
        if self._table is None or self._table.device != torch.device(device):
            freqs = rope_frequencies(self.params)
            # pairs that do not turn have frequency zero
            pairs = self.params.head_dim // 2
            if freqs.numel() < pairs:
                freqs = torch.cat([freqs, torch.zeros(pairs - freqs.numel(), dtype=torch.float32)])
            self._table = freqs.to(device).contiguous()
        return self._table


class NoPosition(PositionEncoding):
    params: NoPositionParams

    def table(self, device) -> Optional[torch.Tensor]:
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
