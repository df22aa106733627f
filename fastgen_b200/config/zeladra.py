"""``Zeladra``: config.json keys -> model description.

A decoder whose layers are listed one by one under ``layers``, each with one of three mixers and
an optional gated feed-forward, pre-norm with layer norms (weight and bias), on one residual
stream or on several that every sub-layer mixes (``streams``).

Keys read: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (optional),
``streams`` (optional), and per layer ``type``, ``mixer`` and ``mlp{kind, ff}`` (or null):

* ``attention``: ``heads, kv_heads, dim, vdim, scale, rot{dims, base}, mask{size, keep_first}``:
  grouped-query softmax attention, rotary positions on a head's first ``rot.dims`` dimensions
  (adjacent pairs), a sliding window of ``mask.size`` keys plus the sequence's first
  ``mask.keep_first`` positions, which stay visible at their true positions;
* ``latent_attention``: ``heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot{dims, base,
  scaling{factor, original, fast, slow}}, kv_from``: causal attention over a cached latent (see
  ``parts/latent_attention.py``); with ``kv_from: j`` the layer reads layer ``j``'s cache;
* ``mamba2``: ``heads, vdim, state, groups, conv, norm_groups``: the state-space mixer.

Tensors: ``embed``, ``l<i>.norm1|norm2`` (each with ``.b``), ``l<i>.hc1|hc2.{in,out,mix}`` (with
``streams``), ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``, ``final.norm`` (+ ``.b``), ``head``.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..parts.params import (
    AttentionParams,
    HyperConnectionParams,
    LatentAttentionParams,
    LayerNormParams,
    Mamba2Params,
    NoPositionParams,
    RopeParams,
    SwiGLUParams,
    TableEmbeddingParams,
    YarnScaling,
)
from .model_args import ConfigError, LayerSpec, ModelArgs, PartSpec, ScheduleEntry, positive_int, require
from .registry import register_architecture

#: the design sets no limit on positions; the engine's own limits (cache size) apply
MAX_POSITIONS = 1 << 30


def _norm(dim: int, eps: float, name: str) -> PartSpec:
    return PartSpec("layernorm", LayerNormParams(dim, eps), {"weight": name, "bias": name + ".b"})


def _rope(rot: Optional[Mapping[str, Any]], head_dim: int, where: str) -> PartSpec:
    if not rot:
        return PartSpec("none", NoPositionParams())
    require(rot, ("dims", "base"), f"{where}.rot")
    scaling = None
    sc = rot.get("scaling")
    if sc:
        require(sc, ("factor", "original", "fast", "slow"), f"{where}.rot.scaling")
        scaling = YarnScaling(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    return PartSpec("rope", RopeParams(head_dim=head_dim, theta=float(rot["base"]), scaling=scaling,
                                       rot_dims=positive_int(rot, "dims")))


def _attention(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    head_dim = positive_int(m, "dim")
    mask = m.get("mask") or {}
    window = None
    keep_first = 0
    if mask:
        require(mask, ("size",), f"{where}.mask")
        window = positive_int(mask, "size")
        keep_first = int(mask.get("keep_first", 0))
    params = AttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=head_dim,
        v_head_dim=positive_int(m, "vdim"),
        position=_rope(m.get("rot"), head_dim, where),
        window=window,
        keep_first=keep_first,
        softmax_scale=float(m["scale"]),
        qk_layout="adjacent",
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "wo": "o"}
    return PartSpec("gqa_attention", params, {k: prefix + v for k, v in names.items()})


def _latent_attention(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"), where)
    rot_dim = positive_int(m, "rot_dim")
    if int(m["rot"].get("dims", rot_dim)) != rot_dim:
        raise ConfigError(f"{where}: rot.dims must equal rot_dim")
    own = m.get("kv_from") is None
    params = LatentAttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        head_dim=positive_int(m, "dim"),
        rot_dim=rot_dim,
        v_head_dim=positive_int(m, "vdim"),
        q_rank=positive_int(m, "q_rank"),
        kv_rank=positive_int(m, "kv_rank"),
        softmax_scale=float(m["scale"]),
        eps=eps,
        position=_rope(m["rot"], rot_dim, where),
        own_cache=own,
        gate=True,
    )
    names = {"w_dq": "dq", "dq_norm": "dq.norm", "w_uq": "uq", "w_uk": "uk", "w_uv": "uv", "w_g": "g", "wo": "o"}
    if own:
        names.update({"w_dkv": "dkv", "dkv_norm": "dkv.norm"})
    return PartSpec("latent_attention", params, {k: prefix + v for k, v in names.items()})


def _mamba2(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where)
    params = Mamba2Params(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        head_dim=positive_int(m, "vdim"),
        state=positive_int(m, "state"),
        groups=positive_int(m, "groups"),
        conv=positive_int(m, "conv"),
        norm_groups=positive_int(m, "norm_groups"),
        eps=eps,
    )
    names = {"w_in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D",
             "norm": "norm", "wo": "o"}
    return PartSpec("mamba2", params, {k: prefix + v for k, v in names.items()})


_MIXERS = {"attention": _attention, "latent_attention": _latent_attention, "mamba2": _mamba2}


def zeladra_model_args(config: Mapping[str, Any]) -> ModelArgs:
    require(config, ("vocab", "width", "layers", "norm"), "Zeladra config.json")
    require(config["norm"], ("eps",), "Zeladra config.json: norm")
    dim = positive_int(config, "width")
    vocab = positive_int(config, "vocab")
    eps = float(config["norm"]["eps"])
    if not isinstance(config["layers"], (list, tuple)) or not config["layers"]:
        raise ConfigError("Zeladra config.json: 'layers' must be a non-empty list")
    streams = config.get("streams")
    if streams is not None:
        streams = positive_int(config, "streams")

    def connection(name: str) -> PartSpec:
        return PartSpec("hyper", HyperConnectionParams(streams),
                        {"in": name + ".in", "out": name + ".out", "mix": name + ".mix"})

    layers, schedule = [], []
    for i, layer in enumerate(config["layers"]):
        where = f"layers[{i}]"
        require(layer, ("type", "mixer"), where)
        kind = layer["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
        p = f"l{i}."
        try:
            mixer = _MIXERS[kind](dim, eps, layer["mixer"], p + "mix.", f"{where}.mixer")
        except ValueError as e:
            raise ConfigError(f"{where}: {e}") from None
        kv_from = layer["mixer"].get("kv_from") if kind == "latent_attention" else None
        if kv_from is not None:
            src = config["layers"][kv_from] if isinstance(kv_from, int) and 0 <= kv_from < i else None
            if src is None or src["type"] != "latent_attention" or src["mixer"].get("kv_from") is not None:
                raise ConfigError(f"{where}: kv_from must name an earlier latent_attention layer with a cache of its own")
            for key in ("kv_rank", "rot_dim"):
                if src["mixer"].get(key) != layer["mixer"].get(key):
                    raise ConfigError(f"{where}: {key} differs from that of layer {kv_from}, whose cache it reads")
        extra = []
        if streams is not None:
            extra.append(("mixer_connection", "connection", connection(p + "hc1")))
        mlp = layer.get("mlp")
        ffn = ffn_norm = None
        if mlp is not None:
            require(mlp, ("kind", "ff"), f"{where}.mlp")
            if mlp["kind"] != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
            ffn = PartSpec("swiglu", SwiGLUParams(dim, positive_int(mlp, "ff")),
                           {"w1": p + "mlp.gate", "w3": p + "mlp.up", "w2": p + "mlp.down"})
            ffn_norm = _norm(dim, eps, p + "norm2")
            if streams is not None:
                extra.append(("ffn_connection", "connection", connection(p + "hc2")))
        layers.append(LayerSpec(block="prenorm" if streams is None else "streams", mixer=mixer,
                                mixer_norm=_norm(dim, eps, p + "norm1"), ffn=ffn, ffn_norm=ffn_norm,
                                extra=tuple(extra)))
        schedule.append(ScheduleEntry(i, kv_from))

    scale = float((config.get("embedding") or {}).get("scale", 1.0))
    return ModelArgs(
        architecture="Zeladra",
        dim=dim,
        vocab_size=vocab,
        max_positions=MAX_POSITIONS,
        tie_embeddings=False,
        embedding_name="embed",
        output_name="head",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(dim, eps, "final.norm"),
        embedder=PartSpec("table", TableEmbeddingParams(vocab, dim, scale), {"table": "embed"}),
        streams=streams,
    )


register_architecture("Zeladra", zeladra_model_args)
