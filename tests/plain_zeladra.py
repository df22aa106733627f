"""A plain, slow implementation of the Zeladra design: whole sequences, no cache, float64 by default.

One function per mechanism, written from the design's equations in this file's own notation
and sharing no code with the package.  ``forward(config, tensors, tokens)`` runs one sequence
and returns the logits of every position (and, on request, the residual stream after every
layer).  ``tensors`` maps checkpoint names to torch tensors.

Notation: ``T`` tokens, positions ``0 .. T-1``; linear weights are stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

DT = torch.float64


def _w(tensors, name):
    return tensors[name].to(DT)


# -- small pieces ---------------------------------------------------------------------------


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotary_frequencies(base: float, dims: int, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """Frequencies of the ``dims/2`` pairs and the factor that multiplies cos and sin."""
    i = torch.arange(dims // 2, dtype=DT)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    f = f / factor * ramp + f * (1 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude=1.0):
    """``x`` [T, ..., 2P]: pair ``(x[2i], x[2i+1])`` of position ``p`` turns by ``p * freqs[i]``."""
    shape = x.shape
    pairs = x.reshape(*shape[:-1], shape[-1] // 2, 2)
    ang = positions.to(DT).reshape(-1, *([1] * (x.dim() - 2)), 1) * freqs
    c, s = torch.cos(ang) * magnitude, torch.sin(ang) * magnitude
    a, b = pairs[..., 0], pairs[..., 1]
    return torch.stack([a * c - b * s, b * c + a * s], dim=-1).reshape(shape)


def visible(n: int, window: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """[n, n] bool: row i sees column j."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, scale, mask):
    """``q`` [T, H, d], ``k`` [T, H, d], ``v`` [T, H, e] -> [T, H, e]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], -math.inf)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhe->ihe", p, v)


# -- mixers ---------------------------------------------------------------------------------


def gqa_mixer(h, tensors, prefix, m):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ _w(tensors, prefix + "q").T).reshape(T, H, d)
    k = (h @ _w(tensors, prefix + "k").T).reshape(T, G, d)
    v = (h @ _w(tensors, prefix + "v").T).reshape(T, G, e)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        f, mag = rotary_frequencies(float(rot["base"]), rot["dims"], rot.get("scaling"))
        r = rot["dims"]
        q = torch.cat([rotate_pairs(q[..., :r], pos, f, mag), q[..., r:]], dim=-1)
        k = torch.cat([rotate_pairs(k[..., :r], pos, f, mag), k[..., r:]], dim=-1)
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    mask = m.get("mask") or {}
    o = softmax_attention(q, k, v, m["scale"], visible(T, mask.get("size"), mask.get("keep_first", 0)))
    return o.reshape(T, H * e) @ _w(tensors, prefix + "o").T


def latent_entries(h, tensors, prefix, m, eps):
    """What a latent-attention layer caches per token: the normed latent and the turned shared key part."""
    T = h.shape[0]
    R, r = m["kv_rank"], m["rot_dim"]
    ckr = h @ _w(tensors, prefix + "dkv").T
    c = unit_rms(ckr[:, :R], eps) * _w(tensors, prefix + "dkv.norm")
    rot = m["rot"]
    f, mag = rotary_frequencies(float(rot["base"]), rot["dims"], rot.get("scaling"))
    kr = rotate_pairs(ckr[:, R:], torch.arange(T), f, mag)
    return c, kr


def latent_mixer(h, tensors, prefix, m, eps, entries):
    """``entries``: (latent [T, R], turned key part [T, r]) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = entries
    cq = unit_rms(h @ _w(tensors, prefix + "dq").T, eps) * _w(tensors, prefix + "dq.norm")
    q = (cq @ _w(tensors, prefix + "uq").T).reshape(T, H, d + r)
    rot = m["rot"]
    f, mag = rotary_frequencies(float(rot["base"]), rot["dims"], rot.get("scaling"))
    q_plain, q_turn = q[..., :d], rotate_pairs(q[..., d:], torch.arange(T), f, mag)
    k_plain = (c @ _w(tensors, prefix + "uk").T).reshape(T, H, d)
    v = (c @ _w(tensors, prefix + "uv").T).reshape(T, H, e)
    qq = torch.cat([q_plain, q_turn], dim=-1)
    kk = torch.cat([k_plain, kr[:, None, :].expand(T, H, r)], dim=-1)
    o = softmax_attention(qq, kk, v, m["scale"], visible(T))
    gate = torch.sigmoid(h @ _w(tensors, prefix + "g").T)  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * e) @ _w(tensors, prefix + "o").T


def mamba2_mixer(h, tensors, prefix, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    taps, parts = m["conv"], m["norm_groups"]
    inner = H * P
    proj = h @ _w(tensors, prefix + "in").T
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N :]
    # causal convolution per channel: the last column of the kernel meets the current token
    kern, kb = _w(tensors, prefix + "conv"), _w(tensors, prefix + "conv.b")
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=DT), xbc], dim=0)
    conv = torch.zeros_like(xbc)
    for t in range(taps):
        conv = conv + padded[t : t + T] * kern[:, t]
    xbc = silu(conv + kb)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner : inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N :].reshape(T, G, N)
    dt = softplus(dt + _w(tensors, prefix + "dt_bias"))  # [T, H]
    decay = torch.exp(-torch.exp(_w(tensors, prefix + "A_log")) * dt)  # [T, H]
    D = _w(tensors, prefix + "D")
    S = torch.zeros(H, N, P, dtype=DT)
    y = torch.zeros(T, H, P, dtype=DT)
    per = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + D[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * _w(tensors, prefix + "norm")
    return y @ _w(tensors, prefix + "o").T


def gated_mlp(h, tensors, prefix):
    g = silu(h @ _w(tensors, prefix + "gate").T)
    return (g * (h @ _w(tensors, prefix + "up").T)) @ _w(tensors, prefix + "down").T


# -- the model ------------------------------------------------------------------------------


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, layer_outputs: Optional[List] = None):
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = _w(tensors, "embed")[tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    n_streams = config.get("streams")
    streams = [x0.clone() for _ in range(n_streams or 1)]
    cached = {}

    def sublayer(i, q, fn):
        nonlocal streams
        p = f"l{i}."
        norm = lambda u: layer_norm(u, _w(tensors, p + f"norm{q}"), _w(tensors, p + f"norm{q}.b"), eps)
        if n_streams is None:
            streams = [streams[0] + fn(norm(streams[0]))]
            return
        a, b, mix = (_w(tensors, p + f"hc{q}.{n}") for n in ("in", "out", "mix"))
        u = sum(a[s] * streams[s] for s in range(n_streams))
        y = fn(norm(u))
        streams = [sum(mix[s, t] * streams[s] for s in range(n_streams)) + b[t] * y for t in range(n_streams)]

    for i, layer in enumerate(config["layers"]):
        m, kind, p = layer["mixer"], layer["type"], f"l{i}.mix."
        if kind == "attention":
            fn = lambda u: gqa_mixer(u, tensors, p, m)
        elif kind == "mamba2":
            fn = lambda u: mamba2_mixer(u, tensors, p, m, eps)
        elif kind == "latent_attention":
            def fn(u):
                src = m.get("kv_from")
                if src is None:
                    cached[i] = latent_entries(u, tensors, p, m, eps)
                    src = i
                return latent_mixer(u, tensors, p, m, eps, cached[src])
        else:
            raise ValueError(kind)
        sublayer(i, 1, fn)
        if layer.get("mlp") is not None:
            sublayer(i, 2, lambda u: gated_mlp(u, tensors, f"l{i}.mlp."))
        if layer_outputs is not None:
            layer_outputs.append(sum(streams))
    x = sum(streams)
    x = layer_norm(x, _w(tensors, "final.norm"), _w(tensors, "final.norm.b"), eps)
    return x @ _w(tensors, "head").T


def read_model(model_dir, dtype=DT):
    """``(config, tensors)`` of a model folder."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    with open(Path(model_dir) / "config.json") as f:
        config = json.load(f)
    tensors = {k: v.to(dtype) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return config, tensors


def greedy(config, tensors, prompt, n_new: int):
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(forward(config, tensors, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
