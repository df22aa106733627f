"""A plain, slow Sinorax on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing
no code with the package.  A whole sequence is run at once: no cache, no
portions, no batches.  ``forward`` takes the parsed ``config.json`` and a dict
of tensors by checkpoint name, and computes in their dtype (float64 in the tests).
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the bigram table for every token: a hash of (previous, current), or the
    table's last row (number ``buckets``) for a sequence's first token."""
    rows = []
    for i, tok in enumerate(tokens):
        if i == 0:
            rows.append(buckets)
        else:
            rows.append((tokens[i - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(tokens: List[int], cfg: Mapping, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    x = w["embed"][torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
        x = x + w["bigram"][torch.tensor(rows)]
    return x


def dyt(x: torch.Tensor, w: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    """Dynamic Tanh: ``tanh(alpha x) * weight + bias``, no statistics of ``x``."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return gelu_erf(h @ w[prefix + "up"].T) @ w[prefix + "down"].T


def rotate_half_pairs(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float, divide: float = 1.0,
                      sign: float = 1.0) -> torch.Tensor:
    """Rotate the first ``dims`` dimensions of ``x`` [T, heads, size]: dimension ``i`` is
    paired with ``i + dims/2`` and the pair turns by ``sign * pos * base^(-2i/dims) / divide``."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = (base ** (-2.0 * i / dims) / divide).to(x.dtype)  # the table is float32, as the design computes it
    ang = sign * pos.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def softmax_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None,
                 pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i, h] = sum_j softmax_j(q_i . k_j * scale) v_j`` over the keys ``j`` with ``pos_j <= pos_i``
    (and ``pos_i - pos_j < window``).  q [T, H, d], k [S, G, d], v [S, G, dv]; ``pos`` gives the
    queries' positions among the keys (default: query i is key i)."""
    t, nh, _ = q.shape
    ng = k.shape[1]
    pos = torch.arange(t) if pos is None else pos
    out = torch.zeros(t, nh, v.shape[2], dtype=q.dtype)
    for head in range(nh):
        g = head // (nh // ng)
        for i in range(t):
            p = int(pos[i])
            lo = 0 if window is None else max(0, p - window + 1)
            s = (k[lo : p + 1, g] @ q[i, head]) * scale
            out[i, head] = torch.softmax(s, dim=0) @ v[lo : p + 1, g]
    return out


def sigmoid_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
                 gate: Optional[torch.Tensor], r1: Optional[torch.Tensor], r2: Optional[torch.Tensor],
                 pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i, h] = sum_j sigmoid(q_i . k_j * scale + gate_h - r1_h ln(1 + r2_h (pos_i - j))) v_j`` over
    the visible keys; the weights are not normalised."""
    t, nh, _ = q.shape
    ng = k.shape[1]
    pos = torch.arange(t) if pos is None else pos
    out = torch.zeros(t, nh, v.shape[2], dtype=q.dtype)
    for head in range(nh):
        g = head // (nh // ng)
        for i in range(t):
            p = int(pos[i])
            lo = 0 if window is None else max(0, p - window + 1)
            s = (k[lo : p + 1, g] @ q[i, head]) * scale
            if r1 is not None:
                dist = (p - torch.arange(lo, p + 1)).to(q.dtype)
                s = s - r1[head] * torch.log(1.0 + r2[head] * dist)
            if gate is not None:
                s = s + gate[head]
            out[i, head] = torch.sigmoid(s) @ v[lo : p + 1, g]
    return out


def softmax_attention(h: torch.Tensor, m: Mapping, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    """The mixer 'attention': grouped heads, biases, partial rotation of queries and keys with
    linear scaling, values rotated by their own position and the sum turned back by the
    query's, causal softmax."""
    t = h.shape[0]
    nh, ng, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(t, nh, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(t, ng, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(t, ng, dv)
    pos = torch.arange(t)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_half_pairs(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_half_pairs(k, pos, rot["dims"], rot["base"], factor)
        v = rotate_half_pairs(v, pos, dv, rot["base"])
    out = softmax_core(q, k, v, m["scale"], (m.get("mask") or {}).get("size"))
    if rot:
        out = rotate_half_pairs(out, pos, dv, rot["base"], sign=-1.0)
    return out.reshape(t, nh * dv) @ w[p + "o"].T + w[p + "o.b"]


def sigmoid_attention(h: torch.Tensor, m: Mapping, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    """The mixer 'attention_2': no rotation, a logarithmic distance bias taken off the score,
    a sliding window, and sigmoid weights that are not normalised over the keys."""
    t = h.shape[0]
    nh, ng, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(t, nh, d)
    k = (h @ w[p + "k"].T).view(t, ng, d)
    v = (h @ w[p + "v"].T).view(t, ng, dv)
    out = sigmoid_core(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), w[p + "pb"], w[p + "r1"], w[p + "r2"])
    return out.reshape(t, nh * dv) @ w[p + "o"].T


MIXERS = {"attention": softmax_attention, "attention_2": sigmoid_attention}


def read_model(model_dir, dtype=torch.float64):
    """``(config, tensors)`` of a model folder, the tensors in ``dtype``."""
    import json
    from pathlib import Path

    from safetensors import safe_open

    with open(Path(model_dir) / "config.json") as f:
        cfg = json.load(f)
    w = {}
    with safe_open(str(Path(model_dir) / "model.safetensors"), "pt") as f:
        for key in f.keys():
            w[key] = f.get_tensor(key).to(dtype)
    return cfg, w


def greedy(cfg: Mapping, w: Mapping[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the residual stream after
    every layer."""
    x = embed(tokens, cfg, w)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixed = MIXERS[layer["type"]](dyt(x, w, p + "norm1"), layer["mixer"], w, p + "mix.")
        x = x + dyt(mixed, w, p + "norm1b")
        if layer.get("mlp") is not None:
            x = x + dyt(dense_ff(dyt(x, w, p + "norm2"), w, p + "mlp."), w, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = dyt(x, w, "final.norm") @ w["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
