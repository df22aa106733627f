"""Zeladra through the engine against the plain implementation of ``plain_zeladra.py``: each
mechanism alone, whole prompts against token-by-token decoding, portions down to two tokens,
unequal batches, pages and slots used again, keys far away and at the edges of windows, kept
first positions and pages, sizes that pad or equal one, and greedy generation through
``Fastgen.generate``."""

import math
import queue
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_zeladra as pz
from fastgen_b200.config import ConfigError, PartSpec, model_args_from_config
from fastgen_b200.weights import write_random_model

DEV = "cuda:0"


def _rot(dims, base=10000.0, scaling=None):
    rot = dict(dims=dims, base=base)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _attn(heads, kv, dim, vdim, scale, dims=None, base=10000.0, mask=None, keep=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if dims:
        m["rot"] = _rot(dims, base)
    if mask:
        m["mask"] = dict(size=mask)
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return m


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
             rot=_rot(rot_dim, base, scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def _layer(kind, mixer, ff):
    return dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ff) if ff else None)


# two streams; a latent layer that a later one reads; a window shorter than a page with kept first
# positions, one longer than a page that keeps more than a page; a state-space layer without a
# feed-forward; value heads smaller and larger than query heads; frequencies scaled by parts
ZA = dict(
    architecture="Zeladra", vocab=211, width=96, norm=dict(eps=1e-5), embedding=dict(scale=0.7), streams=2,
    layers=[
        _layer("latent_attention", _latent(4, 16, 8, 24, 40, 48, 0.2, 5000.0, (4.0, 64, 8.0, 1.0)), 160),
        _layer("mamba2", _ssm(4, 24, 12, 2, 4, 2), None),
        _layer("attention", _attn(6, 2, 32, 16, 0.3, dims=16, base=1000.0, mask=11, keep=3), 72),
        _layer("latent_attention", _latent(4, 16, 8, 24, 40, 48, 0.2, 5000.0, (4.0, 64, 8.0, 1.0), kv_from=0), 120),
        _layer("attention", _attn(2, 1, 16, 32, 0.25, dims=16, base=300.0, mask=37, keep=20), None),
    ],
)
# three streams; no frequency scaling; every head a group of its own and one norm part; a window
# that keeps nothing and a layer that sees everything; two latent caches of different sizes
ZB = dict(
    architecture="Zeladra", vocab=300, width=128, norm=dict(eps=1e-6), embedding=dict(scale=1.7), streams=3,
    layers=[
        _layer("mamba2", _ssm(3, 16, 40, 3, 2, 1), 200),
        _layer("latent_attention", _latent(3, 24, 16, 40, 64, 80, 0.15, 777.0), 256),
        _layer("attention", _attn(4, 4, 64, 64, 0.2, dims=32, base=50000.0, mask=70), 256),
        _layer("latent_attention", _latent(2, 8, 4, 8, 16, 24, 0.3, 100.0, (2.0, 32, 4.0, 0.5)), None),
        _layer("latent_attention", _latent(5, 24, 16, 16, 32, 80, 0.1, 777.0, kv_from=1), 64),
        _layer("attention", _attn(3, 1, 48, 48, 0.15, dims=48, base=10000.0), 200),
    ],
)
# the one ordinary residual stream; no latent layer; one tap (no convolution state), a state of
# nine rows, heads of 40 values, one group, three norm parts; a window of one key that keeps one
ZC = dict(
    architecture="Zeladra", vocab=331, width=120, norm=dict(eps=1e-5),
    layers=[
        _layer("mamba2", _ssm(3, 40, 9, 1, 1, 3), 328),
        _layer("attention", _attn(5, 5, 16, 16, 0.3, dims=8, base=777.0, mask=1, keep=1), 328),
        _layer("mamba2", _ssm(2, 8, 64, 2, 3, 1), None),
        _layer("attention", _attn(4, 2, 32, 32, 0.2, dims=32, base=2000.0, mask=24, keep=2), 100),
    ],
)
# one stream, but with connections of its own
ZD = dict(
    architecture="Zeladra", vocab=97, width=64, norm=dict(eps=1e-5), streams=1,
    layers=[
        _layer("latent_attention", _latent(2, 16, 16, 16, 24, 32, 0.2, 1000.0), 96),
        _layer("mamba2", _ssm(2, 16, 16, 1, 2, 2), 96),
    ],
)
CONFIGS = {"za": (ZA, 3), "zb": (ZB, 5), "zc": (ZC, 8), "zd": (ZD, 9)}


def make_dir(tmp_path, name, std=0.1):
    cfg, seed = CONFIGS[name]
    return write_random_model(Path(tmp_path) / name, cfg, seed, dtype=torch.bfloat16, norm_jitter=0.3, std=std)


_plain = {}


def plain_logits(model_dir, tokens):
    key = (str(model_dir), tuple(tokens))
    if key not in _plain:
        cfg, w = pz.read_model(model_dir)
        _plain[key] = pz.forward(cfg, w, list(tokens)).numpy()
    return _plain[key]


# The bfloat16 rule of this design's models: a row of logits may differ from the plain one by
# Z_L2 of the row's l2 norm and, in its worst entry, by Z_MAX of the row's largest logit.  A layer
# here rounds to bfloat16 more often than a layer of the dense decoder whose tiny models set the
# bounds of ``helpers.check_row`` (two more products in a latent layer, the streams' sums pass every
# rounding on to all later sub-layers); the worst ratios these tests have shown are 0.034 and 0.043.
# float32 rows are held to ``helpers.check_row``'s 1e-4.
Z_L2, Z_MAX = 0.045, 0.055


def check_row(row, ref, dtype, what):
    if dtype == torch.float32:
        return H.check_row(row, ref, dtype, what)
    l2 = float(np.linalg.norm(row - ref) / max(np.linalg.norm(ref), 1e-30))
    mx = float(np.abs(row - ref).max()) / max(float(np.abs(ref).max()), 1e-30)
    assert l2 <= Z_L2, f"{what}: l2 error {l2:.4f} of the row's norm (allowed {Z_L2})"
    assert mx <= Z_MAX, f"{what}: worst entry off by {mx:.4f} of the largest logit (allowed {Z_MAX})"


def compare(model_dir, requests, got, dtype):
    for rid, toks in requests.items():
        ref = plain_logits(model_dir, toks)
        assert set(got[rid]) == set(range(len(toks))), f"{rid}: positions missing"
        for p, row in got[rid].items():
            check_row(row, ref[p], dtype, f"{rid} pos {p}")


def compare_most(model_dir, requests, got, dtype):
    """For models drawn at random, whose rounding noise nobody has looked at row by row: float32 as
    ``compare``; in bfloat16 a row's error is taken relative to the larger of its own norm and the
    request's typical row norm (rounding errors do not shrink with the row they land in), no row may
    be over one and a half times ``Z_L2`` and at most one row in fifty over ``Z_L2`` itself."""
    if dtype == torch.float32:
        return compare(model_dir, requests, got, dtype)
    errs = []
    for rid, toks in requests.items():
        ref = plain_logits(model_dir, toks)
        assert set(got[rid]) == set(range(len(toks))), f"{rid}: positions missing"
        typical = float(np.median(np.linalg.norm(ref, axis=1)))
        for p, row in got[rid].items():
            errs.append(float(np.linalg.norm(row - ref[p])) / max(typical, float(np.linalg.norm(ref[p]))))
    errs = np.array(errs)
    assert errs.max() <= 1.5 * Z_L2, f"worst row off by {errs.max():.4f} (allowed {1.5 * Z_L2})"
    assert (errs > Z_L2).mean() <= 0.02, f"{(errs > Z_L2).sum()} of {errs.size} rows over {Z_L2}"


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------
# the description and the cache bookkeeping (no GPU)
# ---------------------------------------------------------------------------------
def test_description_reads_every_size_from_the_configuration():
    args = model_args_from_config(ZA)
    assert (args.dim, args.vocab_size, args.streams, len(args.layers)) == (96, 211, 2, 5)
    assert args.embedder.params.scale == 0.7
    lat, ssm, att = args.layers[0].mixer.params, args.layers[1].mixer.params, args.layers[2].mixer.params
    assert (lat.n_heads, lat.head_dim, lat.rot_dim, lat.v_head_dim, lat.q_rank, lat.kv_rank) == (4, 16, 8, 24, 40, 48)
    assert lat.own_cache and not args.layers[3].mixer.params.own_cache
    assert lat.position.params.scaling.factor == 4.0 and lat.position.params.theta == 5000.0
    assert (ssm.n_heads, ssm.head_dim, ssm.state, ssm.groups, ssm.conv, ssm.norm_groups) == (4, 24, 12, 2, 4, 2)
    assert (att.window, att.keep_first, att.n_kv_heads, att.v_head_dim, att.softmax_scale) == (11, 3, 2, 16, 0.3)
    assert args.layers[1].ffn is None and args.layers[0].ffn.params.ffn_dim == 160
    assert [e.kv_from for e in args.schedule] == [None, None, None, 0, None]
    assert args.layers[0].block == "streams" and model_args_from_config(ZC).layers[0].block == "prenorm"
    assert model_args_from_config(ZC).streams is None and model_args_from_config(ZD).streams == 1
    assert model_args_from_config(ZB).layers[2].mixer.params.keep_first == 0


def test_description_errors_name_the_place():
    import copy

    bad = copy.deepcopy(ZA)
    bad["layers"][3]["mixer"]["kv_from"] = 1  # not a latent layer
    with pytest.raises(ConfigError, match=r"layers\[3\]"):
        model_args_from_config(bad)
    bad = copy.deepcopy(ZA)
    bad["layers"][3]["mixer"]["kv_rank"] = 56
    with pytest.raises(ConfigError, match="kv_rank"):
        model_args_from_config(bad)
    bad = copy.deepcopy(ZA)
    del bad["layers"][1]["mixer"]["state"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer.*state"):
        model_args_from_config(bad)
    bad = copy.deepcopy(ZA)
    bad["layers"][2]["type"] = "attention_9"
    with pytest.raises(ConfigError, match="attention_9"):
        model_args_from_config(bad)


def test_random_folder_holds_exactly_the_tensors_of_the_description(tmp_path):
    from safetensors.torch import load_file

    d = make_dir(tmp_path, "za")
    names = set(load_file(str(d / "model.safetensors")))
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.hc1.mix", "l0.hc2.in", "l1.hc1.out", "l0.mix.dkv",
            "l0.mix.dq.norm", "l0.mix.g", "l1.mix.A_log", "l1.mix.conv.b", "l1.mix.dt_bias", "l2.mix.q"} <= names
    assert not {"l3.mix.dkv", "l3.mix.dkv.norm", "l1.norm2", "l1.hc2.in", "l4.mlp.up"} & names
    assert "l0.hc1.in" not in set(load_file(str(make_dir(tmp_path, "zc") / "model.safetensors")))


def test_frequencies_scaled_by_parts():
    from fastgen_b200.parts import RopeParams, YarnScaling, make_position

    for dims, base, sc in ((8, 5000.0, (4.0, 64, 8.0, 1.0)), (16, 100.0, (2.0, 32, 4.0, 0.5)), (4, 1e6, (3.0, 1024, 32.0, 1.0))):
        part = make_position(PartSpec("rope", RopeParams(dims, base, scaling=YarnScaling(*map(float, sc)), rot_dims=dims)))
        want, mag = pz.rotary_frequencies(base, dims, dict(zip(("factor", "original", "fast", "slow"), sc)))
        assert torch.allclose(part.table("cpu").double(), want, rtol=2e-6)
        assert abs(part.magnitude() - mag) < 1e-12 and mag == 0.1 * math.log(sc[0]) + 1.0


def test_a_window_keeps_the_pages_of_the_first_positions():
    """Pages that hold kept first positions stay with the request while its window gives the pages
    behind it back; they return when the request ends and are taken again."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.parts import CacheSpec

    cache = CacheManager([CacheSpec(1, 16, window=10, keep_first=9)], [None], [None], page_size=4, n_pages=24,
                         max_requests=2, max_length=200)
    a = cache.admit("a")
    for new in (3, 30, 31, 64, 65, 100):
        cache.reserve(a, new)
        cache.advance(a, new)
        cache.check()
        last = (new - 1) // 4
        kept = set(range(min(3, last + 1)))  # positions 0..8 lie on pages 0..2
        assert sorted(a.pages[0]) == sorted(kept | set(range(max(0, new - 10 + 1) // 4, last + 1)))
    assert cache.free_pages() == [24 - len(a.pages[0])]
    b = cache.admit("b")
    cache.reserve(b, 20)
    cache.release("a")
    cache.check()
    c = cache.admit("c")
    cache.reserve(c, 6)  # position 0's page among them, on pages that a held
    cache.advance(c, 6)
    cache.check()
    cache.release("b")
    cache.release("c")
    assert cache.free_pages() == [24]
    # no kept positions: the first page goes with the window
    plain = CacheManager([CacheSpec(1, 16, window=10)], [None], [None], page_size=4, n_pages=12, max_requests=1,
                         max_length=200)
    r = plain.admit("r")
    plain.reserve(r, 40)
    plain.advance(r, 40)
    assert 0 not in r.pages[0]


# ---------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------
def _ops(dtype):
    from fastgen_b200.csrc.ops import Ops

    return Ops(dtype, DEV)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams", [1, 2, 3])
def test_norms_over_streams(dtype, streams):
    """The layer norm alone; fused with the update of the streams that precedes it; with rows
    gathered (the streams stay); with the plain sum of the streams (the model's end)."""
    from fastgen_b200.parts import LayerNormParams, StreamUpdate, make_norm

    ops = _ops(dtype)
    g = torch.Generator().manual_seed(streams)
    t, dim = 9, 200
    norm = make_norm(PartSpec("layernorm", LayerNormParams(dim, 1e-5), {"weight": "w", "bias": "b"}))
    w, b = 1 + 0.3 * torch.randn(dim, generator=g), 0.2 * torch.randn(dim, generator=g)
    norm.bind({"weight": w.to(DEV), "bias": b.to(DEV)}, ops)
    x = 3 * torch.randn(t, streams, dim, generator=g) + 1.5
    y = torch.randn(t, dim, generator=g).to(dtype)
    mix, out, inc = (torch.rand(s, generator=g) for s in ((streams, streams), (streams,), (streams,)))
    tol = 2e-5 if dtype == torch.float32 else 1e-2

    h = x.clone().to(DEV)
    got = norm.streams_forward(h, update=StreamUpdate(y.to(DEV), mix.to(DEV), out.to(DEV)), in_coef=inc.to(DEV))
    new = torch.einsum("st,nsd->ntd", mix.double(), x.double()) + out.double()[None, :, None] * y.double()[:, None, :]
    want = pz.layer_norm(torch.einsum("s,nsd->nd", inc.double(), new), w.double(), b.double(), 1e-5)
    assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    assert float((h.double().cpu() - new).abs().max()) <= 1e-5 * float(new.abs().max())

    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    h2 = x.clone().to(DEV)
    got = norm.streams_forward(h2, update=StreamUpdate(y.to(DEV), mix.to(DEV), out.to(DEV)), rows=rows)
    want = pz.layer_norm(new.sum(1), w.double(), b.double(), 1e-5)[[7, 0, 7]]
    assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    assert torch.equal(h2.cpu(), x)

    if streams == 1:  # the ordinary "h += delta; norm(h)" and the norm alone
        h3 = x[:, 0].clone().to(DEV)
        got = norm.add_forward(h3, y.to(DEV))
        want = pz.layer_norm(x[:, 0].double() + y.double(), w.double(), b.double(), 1e-5)
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
        got = norm.forward(x[:, 0].to(DEV))
        want = pz.layer_norm(x[:, 0].double(), w.double(), b.double(), 1e-5)
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.gpu
def test_embedding_scale_and_copies():
    ops = _ops(torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 40, generator=g).bfloat16()
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty((4, 3, 40), dtype=torch.float32, device=DEV)
    ops.embedding(table.to(DEV), tokens, out, scale=0.3)
    want = (table.float()[tokens.cpu().long()] * torch.tensor(0.3, dtype=torch.float32))[:, None, :].expand(4, 3, 40)
    assert torch.equal(out.cpu(), want)
    ops.check_status()


def _run_mixer(mixer, cache, x, portions, dtype, rid="r", entry=0):
    """One request through a mixer in portions; returns the outputs and the request."""
    from fastgen_b200.engine.step import StepContext

    req = cache.admit(rid)
    outs, start = [], 0
    for n in portions:
        cache.reserve(req, start + n)
        cache.flush_tables()
        ctx = StepContext(DEV)
        ctx.host_seq_slot, ctx.host_seq_cached, ctx.host_seq_start = [req.slot], [start], [0, n]
        ctx.pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
        ctx.req = torch.full((n,), req.slot, dtype=torch.int32, device=DEV)
        ctx.seq_slot = torch.tensor([req.slot], dtype=torch.int32, device=DEV)
        ctx.seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        ctx.seq_cached = torch.tensor([start], dtype=torch.int32, device=DEV)
        ctx.n_tokens, ctx.n_seqs = n, 1
        outs.append(mixer.forward(x[start:start + n].to(DEV, dtype), ctx, cache.memory(entry)))
        cache.advance(req, start + n)
        start += n
    return torch.cat(outs).double().cpu(), req


def _mixer_and_cache(kind, m, dim, dtype, g, page=8, n_pages=16, std=0.3, tweak=None, eps=1e-5):
    """A mixer of the given sizes with random tensors, bound, with a cache of its own."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.config.zeladra import _MIXERS
    from fastgen_b200.parts import make_mixer
    from fastgen_b200.weights.random_init import draw

    ops = _ops(dtype)
    mixer = make_mixer(_MIXERS[kind](dim, eps, m, "mix.", "test"))
    w = {}
    for s in mixer.weight_specs():
        t = draw(s, g, 0.3)
        if s.init[0] == "normal":
            t = t * (std / s.init[1])
        w[s.name] = t.bfloat16()
    if tweak:
        tweak(w)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [mixer.state_spec()], [None], page, n_pages, 2, page * n_pages,
                         dtype=dtype, device=DEV, tensor_map_factory=ops.make_kv_tensor_maps)
    return mixer, cache, {k: v.double() for k, v in w.items()}, ops


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 24, 12, 2, 4, 2), (3, 16, 40, 3, 2, 1), (3, 40, 9, 1, 1, 3), (2, 64, 128, 1, 3, 2),
                                   (1, 8, 1, 1, 8, 1), (2, 24, 64, 2, 2, 1), (1, 17, 256, 1, 2, 1), (2, 16, 200, 1, 2, 2)])
def test_state_space_mixer_alone(dtype, sizes):
    """Convolution, recurrence, gate and norm in parts: a prompt portion, single tokens and short
    portions through the state of a slot; then the slot is used again and starts from zero."""
    g = torch.Generator().manual_seed(sum(sizes))
    m = _ssm(*sizes)
    mixer, cache, w, ops = _mixer_and_cache("mamba2", m, 72, dtype, g, std=0.2)
    x = torch.randn(60, 72, generator=g).to(dtype)
    ref = pz.mamba2_mixer(x.double(), w, "mix.", m, 1e-5)
    out, req = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 2, 3, 1, 14), dtype)
    ops.check_status()
    assert float((out - ref).abs().max()) <= _tol(dtype) * float(ref.abs().max())
    slot = req.slot
    cache.release("r")
    out2, req2 = _run_mixer(mixer, cache, x[:20], (1, 2, 17), dtype, rid="again")
    assert req2.slot == slot
    assert float((out2 - ref[:20]).abs().max()) <= _tol(dtype) * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_carries_what_was_long_ago(dtype):
    """A decay close to one: an input 150 tokens back still makes most of the output, through
    portions and single tokens (a state that was lost or zeroed on the way would show)."""
    g = torch.Generator().manual_seed(4)
    m = _ssm(2, 16, 8, 1, 2, 1)

    def tweak(w):
        w["mix.A_log"] = torch.full((2,), -9.0).bfloat16()   # exp(-exp(-9) dt): next to no decay
        w["mix.D"] = torch.zeros(2).bfloat16()
    mixer, cache, w, ops = _mixer_and_cache("mamba2", m, 32, dtype, g, n_pages=32, std=0.2, tweak=tweak)
    x = 0.02 * torch.randn(170, 32, generator=g)
    x[5] = 2.0 * torch.randn(32, generator=g)
    x = x.to(dtype)
    ref = pz.mamba2_mixer(x.double(), w, "mix.", m, 1e-5)
    x0 = x.clone()
    x0[5] = 0
    other = pz.mamba2_mixer(x0.double(), w, "mix.", m, 1e-5)
    assert float((ref[160] - other[160]).abs().max()) > 0.2 * float(ref[160].abs().max())
    out, _ = _run_mixer(mixer, cache, x, (4, 3, 90, 2) + (1,) * 50 + (21,), dtype)
    ops.check_status()
    assert float((out - ref).abs().max()) <= _tol(dtype) * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 16, 8, 24, 40, 48, None), (3, 24, 16, 40, 64, 80, (4.0, 64, 8.0, 1.0)),
                                   (1, 8, 2, 8, 8, 16, (2.0, 16, 4.0, 0.5)), (5, 32, 32, 16, 24, 136, None)])
def test_latent_mixer_alone(dtype, sizes):
    """Query latent, cached latent and shared turned key part, gate: a prompt portion and single
    tokens through the cache, against the form that makes every head's keys and values."""
    heads, d, r, dv, qr, kvr, scaling = sizes
    g = torch.Generator().manual_seed(9)
    m = _latent(heads, d, r, dv, qr, kvr, 0.3, 500.0, scaling)
    mixer, cache, w, ops = _mixer_and_cache("latent_attention", m, 72, dtype, g, std=0.2)
    assert mixer.cache_spec().n_pools == 1 and mixer.cache_spec().head_dim >= kvr + r
    x = torch.randn(50, 72, generator=g).to(dtype)
    ref = pz.latent_mixer(x.double(), w, "mix.", m, 1e-5, pz.latent_entries(x.double(), w, "mix.", m, 1e-5))
    out, _ = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 10), dtype)
    ops.check_status()
    assert float((out - ref).abs().max()) <= _tol(dtype) * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_far_key_shows(dtype):
    """One entry hundreds of positions back takes nearly all of a query's weight, through the
    turned key part (whose score the distance turns) across many pages; decoded alone and inside
    a portion."""
    heads, d, r, dv, n = 2, 16, 4, 16, 420
    g = torch.Generator().manual_seed(12)
    m = _latent(heads, d, r, dv, 24, 32, 0.1, 1e6)  # slow turns: the far score does not fade

    def tweak(w):
        w["mix.dkv"][32:, :] = 0
        w["mix.dkv"][32:, 0] = 1.0     # the first input coordinate drives the shared key part,
        w["mix.dq"][:, 1] = 3.0        # the second one the queries (a query's own key stays small)
        w["mix.uq"][:] = 0.02 * torch.randn(w["mix.uq"].shape, generator=g).bfloat16()
        for h in range(heads):
            w["mix.uq"][h * (d + r) + d:(h + 1) * (d + r), :] = 0.5
    mixer, cache, w, ops = _mixer_and_cache("latent_attention", m, 32, dtype, g, page=16, n_pages=32, std=0.05, tweak=tweak)
    x = 0.1 * torch.randn(n, 32, generator=g)
    x[:, :2] = 0.0
    far, q1, q2 = 3, n - 1, n - 40
    x[far, 0] = 4.0
    x[q1, 1] = x[q2, 1] = 4.0
    x = x.to(dtype)
    ref = pz.latent_mixer(x.double(), w, "mix.", m, 1e-5, pz.latent_entries(x.double(), w, "mix.", m, 1e-5))
    x0 = x.clone()
    x0[far] = 0
    other = pz.latent_mixer(x0.double(), w, "mix.", m, 1e-5, pz.latent_entries(x0.double(), w, "mix.", m, 1e-5))
    assert float((ref[q1] - other[q1]).abs().max()) > 0.15 * float(ref[q1].abs().max())
    out, _ = _run_mixer(mixer, cache, x, (300, 100) + (1,) * 20, dtype)
    ops.check_status()
    for i in (q1, q2):
        assert float((out[i] - ref[i]).abs().max()) <= _tol(dtype) * float(ref[i].abs().max()), i
    assert float((out - ref).abs().max()) <= _tol(dtype) * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
@pytest.mark.parametrize("d", [16, 64])
def test_window_edges_and_kept_first_positions_show(dtype, mode, d):
    """Four keys carry large scores: the last kept first position, the first one not kept, the key
    just inside the window and the key just outside.  The two that are visible make the output,
    the two that are not would change it by a large part: in a prompt portion and for a token
    decoded alone, with the kept positions on a page the window has long left."""
    heads, kv, window, keep, n = 2, 1, 70, 5, 200
    g = torch.Generator().manual_seed(11)
    m = _attn(heads, kv, d, d, 16.0 / d, mask=window, keep=keep)

    def tweak(w):
        w["mix.q"][:, 0] = 1.0
        w["mix.k"][:, 0] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 16, dtype, g, page=16, n_pages=16, std=0.05, tweak=tweak)
    x = 0.1 * torch.randn(n, 16, generator=g)
    x[:, 0] = 0.0
    query = n - 1
    marked = (query, query - window + 1, query - window, keep - 1, keep)
    for i in marked:
        x[i, 1:] = torch.randn(15, generator=g)  # values of their own
        x[i, 0] = 1.0
    x = x.to(dtype)
    ref = pz.gqa_mixer(x.double(), w, "mix.", m)
    scale = float(ref[query].abs().max())
    for other in (dict(size=window - 1, keep_first=keep), dict(size=window + 1, keep_first=keep),
                  dict(size=window, keep_first=keep - 1), dict(size=window, keep_first=keep + 1)):
        alt = pz.gqa_mixer(x.double(), w, "mix.", dict(m, mask=other))
        assert float((ref[query] - alt[query]).abs().max()) > 0.1 * scale, other
    portions = (150, 50) if mode == "prompt" else (150, 30) + (1,) * 20
    out, req = _run_mixer(mixer, cache, x, portions, dtype)
    ops.check_status()
    assert float((out[query] - ref[query]).abs().max()) <= _tol(dtype) * scale
    assert float((out - ref).abs().max()) <= _tol(dtype) * float(ref.abs().max())
    assert 0 in req.pages[0] and 1 not in req.pages[0] and len(req.pages[0]) <= -(-window // 16) + 2


# ---------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["za", "zb", "zc", "zd"])
@pytest.mark.parametrize("plan", ["whole", "decode", "portions", "mixed"])
def test_replay(tmp_path, name, dtype, plan):
    """Whole prompts, prompts with a decoded tail, portions of 2 to 17 tokens, and mixed batches
    of up to four requests whose pages and slots are used again, all against the plain
    implementation run on whole sequences."""
    d = make_dir(tmp_path, name)
    vocab = CONFIGS[name][0]["vocab"]
    page = 16
    if plan == "mixed":
        requests = _requests(vocab, [70, 33, 1, 90, 18, 64, 47, 2], 40)
        steps = H.plan_mixed(requests, seed=5)
    else:
        requests = _requests(vocab, [1, 2, 37, 150] if plan != "portions" else [2, 95], 20)
        steps = {"whole": H.plan_whole, "decode": lambda r: H.plan_decode_tail(r, 45), "portions": H.plan_portions}[plan](requests)
    outputs, engine = H.run_engine(d, dtype, steps, page, H.max_live_tokens(steps, page) + 2 * page)
    compare(d, requests, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0 and all(f == g.pool.n_pages for f, g in zip(engine.cache.free_pages(), engine.cache.groups))


def _random_config(seed):
    """A configuration drawn at random: layer kinds in any order, sizes that pad and sizes that do not,
    windows shorter and longer than the pages, kept positions beyond a window, latent layers that
    read an earlier one's cache, one to four streams or the ordinary one."""
    import random

    rng = random.Random(seed)
    layers, latents = [], []
    for i in range(rng.randint(3, 7)):
        kind = rng.choice(["latent_attention", "mamba2", "attention"])
        if kind == "attention":
            dim = rng.choice([16, 32, 48, 64])
            kv = rng.choice([1, 2, 4])
            mask = rng.choice([None, 1, 7, 40, 72, 130])
            m = _attn(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 16, 32]), dim ** -0.5, dims=rng.choice([dim, dim // 2, 8]),
                      base=rng.choice([1e4, 1e6]), mask=mask, keep=rng.choice([None, 0, 1, 4, 20, 70]) if mask else None)
        elif kind == "mamba2":
            heads = rng.choice([1, 2, 4, 6])
            vdim = rng.choice([8, 16, 24, 48])
            m = _ssm(heads, vdim, rng.choice([8, 16, 48, 64, 128]), rng.choice([g for g in (1, 2, 3) if heads % g == 0]),
                     rng.choice([1, 2, 4, 5]), rng.choice([q for q in (1, 2, 3, 4) if (heads * vdim) % q == 0]))
        else:
            src = rng.choice(latents) if latents and rng.random() < 0.4 else None
            heads, d, dv, qr = rng.choice([2, 4, 8]), rng.choice([16, 32]), rng.choice([16, 32, 64]), rng.choice([32, 64])
            if src is not None:
                b = layers[src]["mixer"]
                sc = tuple(b["rot"]["scaling"].values()) if "scaling" in b["rot"] else None
                m = _latent(heads, d, b["rot_dim"], dv, qr, b["kv_rank"], 0.12, b["rot"]["base"], sc, kv_from=src)
            else:
                sc = rng.choice([None, (2.0, 1024, 32.0, 1.0), (4.0, 64, 8.0, 1.0)])
                m = _latent(heads, d, rng.choice([4, 8, 16, 32]), dv, qr, rng.choice([32, 64, 128, 256]), 0.12,
                            rng.choice([1e4, 1e6]), sc)
                latents.append(i)
        layers.append(_layer(kind, m, rng.choice([None, 64, 136])))
    cfg = dict(architecture="Zeladra", vocab=rng.choice([97, 211, 256]), width=rng.choice([64, 96, 200]),
               norm=dict(eps=1e-5), embedding=dict(scale=rng.choice([0.5, 1.3])), layers=layers)
    streams = rng.choice([None, 1, 2, 3, 4])
    if streams is not None:
        cfg["streams"] = streams
    return cfg


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("seed", [11, 13, 25, 35, 37])
def test_configurations_drawn_at_random(tmp_path, dtype, seed):
    """Mixed batches of a model whose layers and sizes are drawn at random."""
    cfg = _random_config(seed)
    d = write_random_model(Path(tmp_path) / "m", cfg, seed, dtype=torch.bfloat16, norm_jitter=0.3, std=0.08)
    requests = _requests(cfg["vocab"], [150, 33, 1, 90, 18, 2], 40 + seed)
    steps = H.plan_mixed(requests, seed=seed)
    outputs, engine = H.run_engine(d, dtype, steps, 64, H.max_live_tokens(steps, 64) + 64)
    compare_most(d, requests, H.collect(steps, outputs), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["za", "zc"])
def test_batching_changes_nothing(tmp_path, dtype, name):
    """A request's logits in a batch of unequal requests equal those it gets alone (bitwise in
    float32, where every sum has a fixed order; within rounding in bfloat16)."""
    d = make_dir(tmp_path, name)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 60)
    alone = H.plan_portions(requests, sizes=(9, 1, 1, 30))
    out_a, _ = H.run_engine(d, dtype, alone, 8, H.max_live_tokens(alone, 8) + 32)
    got_a = H.collect(alone, out_a)
    mixed = H.plan_mixed(requests, seed=2)
    out_m, _ = H.run_engine(d, dtype, mixed, 8, H.max_live_tokens(mixed, 8) + 32)
    got_m = H.collect(mixed, out_m)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_a[rid][p], got_m[rid][p]), (rid, p)
            else:
                check_row(got_m[rid][p], got_a[rid][p], dtype, f"{rid} {p}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["za", "zc"])
def test_steps_replayed_from_graphs_change_nothing(tmp_path, dtype, name):
    """Steps captured as CUDA graphs (single tokens, and prompt portions padded to a few shapes)
    give what the same steps give launched kernel by kernel: states, convolution inputs and kept
    pages are advanced by the replays only, never by a capture."""
    d = make_dir(tmp_path, name)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 61)
    mixed = H.plan_mixed(requests, seed=3)
    room = H.max_live_tokens(mixed, 8) + 32
    out_g, eng = H.run_engine(d, dtype, mixed, 8, room, max_step_tokens=64)
    assert eng.graphs is not None and eng.step_graphs is not None and eng.step_graphs.replays > 0
    out_p, _ = H.run_engine(d, dtype, mixed, 8, room, num_cuda_graphs=0)
    got_g, got_p = H.collect(mixed, out_g), H.collect(mixed, out_p)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_g[rid][p], got_p[rid][p]), (rid, p)
            else:
                check_row(got_g[rid][p], got_p[rid][p], dtype, f"{rid} {p}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_past_windows_and_pages(tmp_path, dtype):
    """200 tokens decoded one by one after a two-token prompt: every window passes over decoded
    tokens, pages of the windowed layers come back (the kept ones stay) and are taken again."""
    d = make_dir(tmp_path, "za")
    requests = _requests(211, [202], 77)
    steps = H.plan_decode_tail(requests, 200)
    outputs, engine = H.run_engine(d, dtype, steps, 8, 232)
    compare(d, requests, H.collect(steps, outputs), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["za", "zc"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name):
    """``Fastgen.generate`` with its scheduler (portions of 16 tokens, batches of 3, graphs)
    against greedy decoding with the plain implementation."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    d = make_dir(tmp_path, name)
    cfg, w = pz.read_model(d)
    vocab = cfg["vocab"]
    prompts = [H.random_tokens(vocab, n, 90 + n) for n in (7, 1, 40, 23)]
    fg = Fastgen.build(HfLoader(d), GenArgs(use_sampling=False, max_gen=12, cache_block=16, max_seq=128, max_batch=3,
                                            max_prefill=16),
                       tp_mesh=None, device=torch.device(DEV), dtype=dtype)
    q = queue.Queue()
    for i, p in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=p))
    q.put(None)
    got = {pkt.thread_id: pkt.tokens for pkt in fg.generate(q)}
    fg.destroy()
    for i, p in enumerate(prompts):
        assert len(got[i]) == 12
        if dtype == torch.float32:
            assert got[i] == pz.greedy(cfg, w, p, 12), i
        else:
            seq = list(p)
            for tok in got[i]:
                logits = pz.forward(cfg, w, seq)[-1]
                assert float(logits[tok]) >= float(logits.max()) - 0.03 * float(logits.abs().max())
                seq.append(tok)
