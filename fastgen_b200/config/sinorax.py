"""``Sinorax``: config.json keys -> model description.

A decoder whose layers are listed one by one under ``layers`` (each with its own mixer and
sizes), with a hashed bigram embedding beside the token embedding, Dynamic Tanh norms before
and after every sub-layer, dense GELU feed-forwards and scaled, soft-capped logits.

Keys read: ``architecture``, ``vocab``, ``width``, ``norm.eps`` (accepted; the Dynamic Tanh
norm has no use for it), ``embedding.bigram{buckets, mul_prev, mul_cur}`` (optional),
``logit_scale``, ``logit_softcap`` (optional), and per layer ``type``, ``mixer{heads,
kv_heads, dim, vdim, scale, rot{dims, base, scaling{factor}}, mask{size}}`` and
``mlp{kind, ff}`` (or null).  Tensors: ``embed``, ``bigram``, ``l<i>.norm1|norm1b|norm2|
norm2b`` (each with ``.b`` and ``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``final.norm``, ``head``.

Two mixers:

* ``attention``: grouped-query causal softmax attention with biases on its four projections,
  rotary positions on the first ``rot.dims`` dimensions of queries and keys (pairs ``(i, i +
  dims/2)``, frequencies divided by ``rot.scaling.factor``), and values turned by their own
  position over all of ``vdim`` (same pairing, no scaling) with each head's output turned back
  by the query's position;
* ``attention_2``: no biases and no rotation; a sliding window of ``mask.size`` keys; the score
  has ``r1_h ln(1 + r2_h distance)`` taken off and the weight of a key is ``sigmoid(score +
  pb_h)``, not normalised over the keys.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..parts.params import (
    AttentionParams,
    BigramHashParams,
    DenseMLPParams,
    DynamicTanhParams,
    NoPositionParams,
    RopeParams,
    SigmoidAttentionParams,
)
from .model_args import (
    ConfigError,
    LayerSpec,
    ModelArgs,
    PartSpec,
    ScheduleEntry,
    positive_int,
    require,
)
from .registry import register_architecture

#: the design sets no limit on positions; the engine's own limits (cache size) apply
MAX_POSITIONS = 1 << 30


def _norm(dim: int, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", DynamicTanhParams(dim), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _window(mixer: Mapping[str, Any], where: str) -> Optional[int]:
    mask = mixer.get("mask")
    if not mask:
        return None
    require(mask, ("size",), f"{where}.mask")
    return positive_int(mask, "size")


def _softmax_attention(dim: int, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    head_dim, v_head_dim = positive_int(m, "dim"), positive_int(m, "vdim")
    position = PartSpec("none", NoPositionParams())
    value_position = None
    rot = m.get("rot")
    if rot:
        require(rot, ("dims", "base"), f"{where}.rot")
        factor = (rot.get("scaling") or {}).get("factor")
        position = PartSpec(
            "rope",
            RopeParams(
                head_dim=head_dim,
                theta=float(rot["base"]),
                rot_dims=positive_int(rot, "dims"),
                linear_factor=float(factor) if factor is not None else None,
            ),
        )
        value_position = PartSpec("rope", RopeParams(head_dim=v_head_dim, theta=float(rot["base"])))
    params = AttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=head_dim,
        v_head_dim=v_head_dim,
        position=position,
        window=_window(m, where),
        softmax_scale=float(m["scale"]),
        qk_layout="half_split",
        v_layout="half_split",
        bias=True,
        value_position=value_position,
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "wo": "o", "bq": "q.b", "bk": "k.b", "bv": "v.b", "bo": "o.b"}
    return PartSpec("gqa_attention", params, {k: prefix + v for k, v in names.items()})


def _sigmoid_attention(dim: int, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    params = SigmoidAttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=positive_int(m, "dim"),
        v_head_dim=positive_int(m, "vdim"),
        position=PartSpec("none", NoPositionParams()),
        window=_window(m, where),
        softmax_scale=float(m["scale"]),
        gate=True,
        distance_bias=True,
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "wo": "o", "r1": "r1", "r2": "r2", "gate": "pb"}
    return PartSpec("sigmoid_attention", params, {k: prefix + v for k, v in names.items()})


_MIXERS = {"attention": _softmax_attention, "attention_2": _sigmoid_attention}


def sinorax_model_args(config: Mapping[str, Any]) -> ModelArgs:
    require(config, ("vocab", "width", "layers"), "Sinorax config.json")
    dim = positive_int(config, "width")
    vocab = positive_int(config, "vocab")
    if not isinstance(config["layers"], (list, tuple)) or not config["layers"]:
        raise ConfigError("Sinorax config.json: 'layers' must be a non-empty list")

    layers, optional = [], []
    for i, layer in enumerate(config["layers"]):
        where = f"layers[{i}]"
        require(layer, ("type", "mixer"), where)
        kind = layer["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
        m = layer["mixer"]
        require(m, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}.mixer")
        p = f"l{i}."
        try:
            mixer = _MIXERS[kind](dim, m, p + "mix.", f"{where}.mixer")
        except ValueError as e:
            raise ConfigError(f"{where}: {e}") from None
        extra = [("post_mixer_norm", "norm", _norm(dim, p + "norm1b"))]
        mlp = layer.get("mlp")
        ffn = ffn_norm = None
        if mlp is not None:
            require(mlp, ("kind", "ff"), f"{where}.mlp")
            if mlp["kind"] != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
            ffn = PartSpec(
                "dense_mlp",
                DenseMLPParams(dim, positive_int(mlp, "ff"), "gelu_erf"),
                {"up": p + "mlp.up", "down": p + "mlp.down"},
            )
            ffn_norm = _norm(dim, p + "norm2")
            extra.append(("post_ffn_norm", "norm", _norm(dim, p + "norm2b")))
        else:
            # a layer without a feed-forward has no use for its second pair of norms
            for name in (p + "norm2", p + "norm2b"):
                optional += [name, name + ".b", name + ".alpha"]
        layers.append(
            LayerSpec(
                block="sandwich",
                mixer=mixer,
                mixer_norm=_norm(dim, p + "norm1"),
                ffn=ffn,
                ffn_norm=ffn_norm,
                extra=tuple(extra),
            )
        )

    embedder = None
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        require(bigram, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
        embedder = PartSpec(
            "bigram_hash",
            BigramHashParams(vocab, dim, positive_int(bigram, "buckets"), int(bigram["mul_prev"]), int(bigram["mul_cur"])),
            {"table": "embed", "bigram": "bigram"},
        )
    cap = config.get("logit_softcap")
    return ModelArgs(
        architecture="Sinorax",
        dim=dim,
        vocab_size=vocab,
        max_positions=MAX_POSITIONS,
        tie_embeddings=False,
        embedding_name="embed",
        output_name="head",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(dim, "final.norm"),
        embedder=embedder,
        logit_scale=float(config.get("logit_scale", 1.0)),
        logit_softcap=float(cap) if cap else None,
        optional_tensors=tuple(optional),
    )


register_architecture("Sinorax", sinorax_model_args)
