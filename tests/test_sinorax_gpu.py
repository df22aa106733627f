"""Sinorax through the engine against the plain implementation of ``plain_sinorax.py``:
each mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, unequal batches, pages and slots used again, keys at the edges of windows and pages,
sizes that pad, and greedy generation through ``Fastgen.generate``."""

import json
import queue
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_sinorax as ps
from fastgen_b200.config import ConfigError, PartSpec, model_args_from_config
from fastgen_b200.weights import write_random_model

DEV = "cuda:0"


def _attn(heads, kv, dim, vdim, scale, dims=None, base=10000.0, factor=None, mask=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if dims:
        m["rot"] = dict(dims=dims, base=base)
        if factor:
            m["rot"]["scaling"] = dict(factor=factor)
    if mask:
        m["mask"] = dict(size=mask)
    return m


def _layer(kind, mixer, ff):
    return dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ff) if ff else None)


# value heads smaller and larger than query heads, a part of the head rotated, head sizes that
# pad (24, 40), a window shorter than a page and one longer, a layer without a feed-forward,
# groups of 1, 2 and 3 heads
SX_A = dict(
    architecture="Sinorax", vocab=211, width=96, norm=dict(eps=1e-5), logit_scale=1.5, logit_softcap=12.0,
    embedding=dict(bigram=dict(buckets=53, mul_prev=31, mul_cur=5)),
    layers=[
        _layer("attention", _attn(4, 2, 32, 16, 0.4, dims=16, base=1000.0, factor=4.0), 160),
        _layer("attention_2", _attn(3, 1, 24, 40, 0.3, mask=5), 72),
        _layer("attention", _attn(2, 2, 16, 16, 0.5, dims=16, base=300.0), None),
        _layer("attention_2", _attn(2, 2, 16, 32, 0.25, mask=37), 120),
    ],
)
# head size 64 (the tensor-core paths of the softmax attention), groups of 3, longer windows,
# no bigram table and no cap on the logits
SX_B = dict(
    architecture="Sinorax", vocab=300, width=128, norm=dict(eps=1e-6), logit_scale=0.7,
    layers=[
        _layer("attention_2", _attn(4, 4, 64, 32, 0.2, mask=70), 256),
        _layer("attention", _attn(6, 2, 64, 64, 0.3, dims=32, base=50000.0, factor=2.0), 256),
        _layer("attention", _attn(2, 1, 64, 128, 0.25, dims=64, base=10000.0), 200),
    ],
)
# a width and a vocabulary that are multiples of nothing, a window of one key (a token sees
# itself only), multipliers that overflow 32 bits when multiplied with a token id
SX_C = dict(
    architecture="Sinorax", vocab=331, width=200, norm=dict(eps=1e-5), logit_scale=2.0, logit_softcap=5.0,
    embedding=dict(bigram=dict(buckets=7, mul_prev=2000000011, mul_cur=1999999973)),
    layers=[
        _layer("attention_2", _attn(5, 5, 48, 80, 0.15, mask=1), 328),
        _layer("attention", _attn(5, 5, 48, 80, 0.2, dims=24, base=777.0, factor=1.5), 328),
        _layer("attention_2", _attn(4, 2, 16, 16, 0.3, mask=16), None),
    ],
)
CONFIGS = {"sx_a": (SX_A, 3), "sx_b": (SX_B, 5), "sx_c": (SX_C, 8)}


def make_dir(tmp_path, name, std=0.1):
    cfg, seed = CONFIGS[name]
    return write_random_model(Path(tmp_path) / name, cfg, seed, dtype=torch.bfloat16, norm_jitter=0.3, std=std)


_plain = {}


def plain_logits(model_dir, tokens):
    key = (str(model_dir), tuple(tokens))
    if key not in _plain:
        cfg, w = ps.read_model(model_dir, torch.float64)
        _plain[key] = ps.forward(cfg, w, list(tokens)).numpy()
    return _plain[key]


def compare(model_dir, requests, got, dtype):
    for rid, toks in requests.items():
        ref = plain_logits(model_dir, toks)
        assert set(got[rid]) == set(range(len(toks))), f"{rid}: positions missing"
        for p, row in got[rid].items():
            H.check_row(row, ref[p], dtype, f"{rid} pos {p}")


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------
# the description (no GPU)
# ---------------------------------------------------------------------------------
def test_description_reads_every_size_from_the_configuration():
    args = model_args_from_config(SX_A)
    assert args.architecture == "Sinorax" and args.dim == 96 and args.vocab_size == 211
    assert args.logit_scale == 1.5 and args.logit_softcap == 12.0
    assert args.embedder.kind == "bigram_hash" and args.embedder.params.buckets == 53
    kinds = [layer.mixer.kind for layer in args.layers]
    assert kinds == ["gqa_attention", "sigmoid_attention", "gqa_attention", "sigmoid_attention"]
    a = args.layers[0].mixer.params
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.v_head_dim, a.kernel_head_dim) == (4, 2, 32, 16, 32)
    assert a.bias and a.position.params.rot_dims == 16 and a.position.params.linear_factor == 4.0
    assert a.value_position.params.head_dim == 16 and a.value_position.params.linear_factor is None
    s = args.layers[1].mixer.params
    assert (s.head_dim, s.v_head_dim, s.kernel_head_dim, s.window) == (24, 40, 48, 5) and not s.bias
    assert args.layers[2].ffn is None and args.layers[2].ffn_norm is None
    assert "l2.norm2.alpha" in args.optional_tensors
    assert args.layers[0].mixer.names["bo"] == "l0.mix.o.b" and args.layers[1].mixer.names["gate"] == "l1.mix.pb"
    assert model_args_from_config(SX_B).embedder is None and model_args_from_config(SX_B).logit_softcap is None


def test_description_errors_name_the_place():
    with pytest.raises(ConfigError, match="width"):
        model_args_from_config({k: v for k, v in SX_A.items() if k != "width"})
    assert model_args_from_config({k: v for k, v in SX_A.items() if k != "logit_scale"}).logit_scale == 1.0
    bad = json.loads(json.dumps(SX_A))
    bad["layers"][1]["type"] = "attention_9"
    with pytest.raises(ConfigError, match=r"layers\[1\].*attention_9"):
        model_args_from_config(bad)
    bad = json.loads(json.dumps(SX_A))
    del bad["layers"][3]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match=r"layers\[3\].mixer.*vdim"):
        model_args_from_config(bad)
    bad = json.loads(json.dumps(SX_A))
    bad["layers"][0]["mixer"]["heads"] = 3
    with pytest.raises(ConfigError, match="grouped"):
        model_args_from_config(bad)


def test_random_folder_holds_exactly_the_tensors_of_the_description(tmp_path):
    from safetensors import safe_open

    d = make_dir(tmp_path, "sx_a")
    with safe_open(str(d / "model.safetensors"), "pt") as f:
        shapes = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
    assert shapes["bigram"] == (54, 96) and shapes["l0.mix.v"] == (32, 96) and shapes["l0.mix.o"] == (96, 64)
    assert shapes["l1.mix.pb"] == (3,) and shapes["l1.mix.v"] == (40, 96) and shapes["l0.norm1b.alpha"] == ()
    assert "l2.mlp.up" not in shapes and "l2.norm2" not in shapes and shapes["head"] == (211, 96)


def test_bigram_rows_of_the_plain_implementation():
    assert ps.bigram_rows([3, 4, 3], 10, 7, 2) == [10, (3 * 7 + 4 * 2) % 10, (4 * 7 + 3 * 2) % 10]


# ---------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------
def _ops(dtype):
    from fastgen_b200.csrc.ops import Ops
    return Ops(dtype, DEV)


def _dyt_part(dim, g, ops, name="n"):
    from fastgen_b200.parts import DynamicTanhParams, make_norm

    norm = make_norm(PartSpec("dynamic_tanh", DynamicTanhParams(dim), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"}))
    w = {name: (1 + 0.3 * torch.randn(dim, generator=g)).bfloat16(), name + ".b": (0.2 * torch.randn(dim, generator=g)).bfloat16(),
         name + ".alpha": torch.tensor(0.7 + 0.6 * float(torch.rand((), generator=g))).bfloat16()}
    norm.bind({"weight": w[name].to(DEV), "bias": w[name + ".b"].to(DEV), "alpha": w[name + ".alpha"].to(DEV)}, ops)
    return norm, {k: v.double() for k, v in w.items()}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_alone_and_fused_with_the_sum(dtype):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(0)
    tol = dict(rtol=1e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    norm, w = _dyt_part(200, g, ops, "a")
    post, wp = _dyt_part(200, g, ops, "b")
    assert [s.shape for s in norm.weight_specs()] == [(200,), (200,), ()]
    h = (2 * torch.randn(7, 200, generator=g)).to(DEV)
    d = torch.randn(7, 200, generator=g).to(DEV, dtype)
    assert torch.allclose(norm.forward(h).double().cpu(), ps.dyt(h.double().cpu(), w, "a"), **tol)
    # the sum, the summand's own norm and the norm of the sum in one launch
    h0 = h.clone()
    total = h0.double().cpu() + ps.dyt(d.double().cpu(), wp, "b")
    out = norm.add_forward(h, d, delta_norm=post)
    assert out.dtype == dtype and torch.allclose(out.double().cpu(), ps.dyt(total, w, "a"), **tol)
    assert torch.allclose(h.double().cpu(), total, rtol=1e-6, atol=1e-6)  # the stream holds the 32-bit sum
    # gathered rows leave the stream as it was
    h1 = h0.clone()
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = norm.add_forward(h1, d, rows=rows, delta_norm=post)
    assert torch.equal(h1, h0) and torch.allclose(out.double().cpu(), ps.dyt(total, w, "a")[[5, 0, 5]], **tol)
    # the sum without a norm of the summand
    h2 = h0.clone()
    out = norm.add_forward(h2, d)
    assert torch.allclose(out.double().cpu(), ps.dyt(h0.double().cpu() + d.double().cpu(), w, "a"), **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_summand_with_a_norm_of_another_kind(dtype):
    """The closing norm of a sub-layer need not be of the kind of the norm that follows: an
    RMSNorm after a Dynamic Tanh summand, and the other way round, compose the same sum."""
    import plain_llama as pl
    from fastgen_b200.parts import RMSNormParams, make_norm

    ops = _ops(dtype)
    g = torch.Generator().manual_seed(3)
    tol = dict(rtol=1e-5, atol=5e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    dyt, wd = _dyt_part(64, g, ops, "a")
    rms = make_norm(PartSpec("rmsnorm", RMSNormParams(64, 1e-5), {"weight": "w"}))
    w = (1 + 0.1 * torch.randn(64, generator=g)).bfloat16()
    rms.bind({"weight": w.to(DEV)}, ops)
    h = torch.randn(5, 64, generator=g).to(DEV)
    d = torch.randn(5, 64, generator=g).to(DEV, dtype)
    hd, dd = h.double().cpu(), d.double().cpu()
    out = rms.add_forward(h.clone(), d, delta_norm=dyt)
    assert torch.allclose(out.double().cpu(), pl.rmsnorm(hd + ps.dyt(dd, wd, "a"), w.double(), 1e-5), **tol)
    out = dyt.add_forward(h.clone(), d, delta_norm=rms)
    assert torch.allclose(out.double().cpu(), ps.dyt(hd + pl.rmsnorm(dd, w.double(), 1e-5), wd, "a"), **tol)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    out = rms.add_forward(h.clone(), d, rows=rows, delta_norm=dyt)
    assert torch.allclose(out.double().cpu(), pl.rmsnorm(hd + ps.dyt(dd, wd, "a"), w.double(), 1e-5)[[4, 1]], **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [3, 40])
def test_dense_feed_forward_alone(dtype, tokens):
    """A few tokens (the activation is the epilogue of the weight-streaming product) and many
    (the library's product and a kernel of its own)."""
    from fastgen_b200.parts import DenseMLPParams, make_feed_forward

    ops = _ops(dtype)
    g = torch.Generator().manual_seed(1)
    ffn = make_feed_forward(PartSpec("dense_mlp", DenseMLPParams(72, 200), {"up": "u", "down": "d"}))
    assert {(s.name, s.shape) for s in ffn.weight_specs()} == {("u", (200, 72)), ("d", (72, 200))}
    t = {k: (torch.randn(*s, generator=g) * 0.3).to(DEV, torch.bfloat16) for k, s in (("up", (200, 72)), ("down", (72, 200)))}
    ffn.bind(t, ops)
    x = torch.randn(tokens, 72, generator=g).to(DEV, dtype)
    ref = ps.gelu_erf(x.double().cpu() @ t["up"].double().cpu().T) @ t["down"].double().cpu().T
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=6e-2)
    assert torch.allclose(ffn.forward(x, None).double().cpu(), ref, **tol)


@pytest.mark.gpu
def test_activations_of_the_kernel():
    ops = _ops(torch.float32)
    z = torch.linspace(-6, 6, 1001, device=DEV).reshape(1, -1).contiguous()
    erf = ops.bias_act(z.clone(), "gelu_erf").cpu().double()
    assert torch.allclose(erf, ps.gelu_erf(z.cpu().double()), atol=1e-6)
    zt = z.cpu().double()
    ref = 0.5 * zt * (1 + torch.tanh(np.sqrt(2 / np.pi) * (zt + 0.044715 * zt ** 3)))
    assert torch.allclose(ops.bias_act(z.clone(), "gelu_tanh").cpu().double(), ref, atol=1e-6)
    logits = torch.linspace(-50, 50, 64, device=DEV).reshape(2, 32).contiguous()
    want = 9.0 * torch.tanh(logits.double().cpu() * 1.5 / 9.0)
    assert torch.allclose(ops.scale_softcap(logits.clone(), 1.5, 9.0).double().cpu(), want, atol=1e-5)
    assert torch.allclose(ops.scale_softcap(logits.clone(), 0.5, None), logits * 0.5)


@pytest.mark.gpu
def test_bigram_embedder_keeps_the_previous_token_per_slot():
    """Portions of two sequences in one step, a sequence that sits a step out, a slot that is
    given to a new request: the first token of a portion finds its predecessor in the slot's
    state, the first token of a sequence takes the table's last row."""
    from fastgen_b200.engine.step import StepContext
    from fastgen_b200.parts import BigramHashParams, make_embedder

    ops = _ops(torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    vocab, dim, buckets, mp, mc = 50, 24, 11, 2000000011, 13
    emb = make_embedder(PartSpec("bigram_hash", BigramHashParams(vocab, dim, buckets, mp, mc), {"table": "e", "bigram": "b"}))
    assert emb.state_spec().dtype == torch.int32
    table = torch.randn(vocab, dim, generator=g).bfloat16()
    bigram = torch.randn(buckets + 1, dim, generator=g).bfloat16()
    emb.bind({"table": table.to(DEV), "bigram": bigram.to(DEV)}, ops)
    state = torch.zeros(3, 1, dtype=torch.int32, device=DEV)
    w = {"embed": table.double(), "bigram": bigram.double()}
    cfg = dict(embedding=dict(bigram=dict(buckets=buckets, mul_prev=mp, mul_cur=mc)))
    seqs = {0: H.random_tokens(vocab, 9, 1), 2: H.random_tokens(vocab, 7, 2)}
    want = {s: ps.embed(t, cfg, w) for s, t in seqs.items()}
    at = {0: 0, 2: 0}

    def step(parts):
        toks, pos, req = [], [], []
        for slot, n in parts:
            toks += seqs[slot][at[slot]:at[slot] + n]
            pos += range(at[slot], at[slot] + n)
            req += [slot] * n
        req += [-1, -1]  # padding lanes of a captured step
        toks += [0, 0]
        pos += [0, 0]
        ctx = StepContext(DEV)
        ctx.tokens, ctx.pos, ctx.req = (torch.tensor(a, dtype=torch.int32, device=DEV) for a in (toks, pos, req))
        out = torch.empty(len(toks), dim, dtype=torch.float32, device=DEV)
        emb.forward(ctx, state, out)
        row = 0
        for slot, n in parts:
            assert torch.allclose(out[row:row + n].double().cpu(), want[slot][at[slot]:at[slot] + n], atol=1e-6), (slot, at)
            row += n
            at[slot] += n
        assert float(out[row:].abs().max()) == 0.0

    step([(0, 3), (2, 1)])
    step([(2, 2)])           # slot 0 sits out
    step([(0, 1), (2, 1)])   # single tokens
    step([(0, 5), (2, 3)])
    ops.check_status()
    # slot 2 goes to a new request: its state is not read at position 0
    seqs[2], at[2] = H.random_tokens(vocab, 4, 9), 0
    want[2] = ps.embed(seqs[2], cfg, w)
    step([(2, 2)])
    step([(2, 2)])


@pytest.mark.gpu
def test_rotation_tables():
    from fastgen_b200.parts import RopeParams, make_position

    t = make_position(PartSpec("rope", RopeParams(32, 1000.0, rot_dims=8, linear_factor=4.0))).table(DEV).cpu()
    assert t.shape == (16,) and float(t[4:].abs().max()) == 0.0
    want = torch.tensor([1000.0 ** (-2 * i / 8) / 4.0 for i in range(4)])
    assert torch.allclose(t[:4], want.float(), rtol=1e-6)


def _run_mixer(mixer, cache, x, portions, dtype):
    from fastgen_b200.engine.step import StepContext

    req = cache.admit("r")
    outs, start = [], 0
    for n in portions:
        cache.reserve(req, start + n)
        cache.flush_tables()
        ctx = StepContext(DEV)
        ctx.host_seq_slot, ctx.host_seq_cached, ctx.host_seq_start = [req.slot], [start], [0, n]
        ctx.pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
        ctx.req = torch.full((n,), req.slot, dtype=torch.int32, device=DEV)
        ctx.n_tokens = n
        outs.append(mixer.forward(x[start:start + n].to(DEV, dtype), ctx, cache.memory(0)))
        cache.advance(req, start + n)
        start += n
    return torch.cat(outs).double().cpu(), req


def _mixer_and_cache(kind, m, dim, dtype, g, page=8, n_pages=16, std=0.3, tweak=None):
    """A Sinorax mixer of the given sizes with random tensors, bound, with a cache of its own."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.config.sinorax import _MIXERS
    from fastgen_b200.parts import make_mixer

    ops = _ops(dtype)
    spec = _MIXERS[kind](dim, m, "mix.", "test")
    mixer = make_mixer(spec)
    w = {}
    for s in mixer.weight_specs():
        t = torch.randn(*s.shape, generator=g) * std
        if s.name in ("mix.r1", "mix.r2"):
            t = t.abs() + 0.2
        w[s.name] = t.bfloat16()
    if tweak:
        tweak(w)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [None], [None], page, n_pages, 2, page * n_pages, dtype=dtype, device=DEV,
                         tensor_map_factory=ops.make_kv_tensor_maps)
    return mixer, cache, {k: v.double() for k, v in w.items()}, ops


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 16, 16), (6, 2, 64, 64, 64), (3, 3, 24, 40, 8), (2, 1, 64, 128, 32)])
def test_softmax_mixer_alone(dtype, sizes):
    """Biases, a part of the head rotated with scaled frequencies, values turned by their own
    position and the output turned back: a prompt portion and single tokens through a cache."""
    heads, kv, d, dv, dims = sizes
    g = torch.Generator().manual_seed(7)
    m = _attn(heads, kv, d, dv, 0.35, dims=dims, base=500.0, factor=3.0)
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 72, dtype, g, std=0.2)
    assert mixer.cache_spec().head_dim == -(-max(d, dv) // 16) * 16
    x = torch.randn(50, 72, generator=g).to(dtype)
    ref = ps.softmax_attention(x.double(), m, w, "mix.")
    out, _ = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 10), dtype)
    ops.check_status()
    scale = float(ref.abs().max())
    assert float((out - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 2.5e-2) * scale


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 1, 24, 40, 5), (4, 4, 64, 32, 20), (2, 2, 16, 16, 1), (6, 2, 48, 48, 33)])
def test_sigmoid_mixer_alone(dtype, sizes):
    heads, kv, d, dv, window = sizes
    g = torch.Generator().manual_seed(8)
    m = _attn(heads, kv, d, dv, 0.3, mask=window)
    mixer, cache, w, ops = _mixer_and_cache("attention_2", m, 72, dtype, g)
    x = torch.randn(60, 72, generator=g).to(dtype)
    ref = ps.sigmoid_attention(x.double(), m, w, "mix.")
    out, req = _run_mixer(mixer, cache, x, (2, 31, 1, 1, 9, 1, 15), dtype)
    ops.check_status()
    scale = float(ref.abs().max())
    assert float((out - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 2.5e-2) * scale
    assert len(req.pages[0]) <= -(-window // 8) + 1  # the window gave pages back


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
@pytest.mark.parametrize("d", [16, 64, 128])
def test_sigmoid_window_edge_shows(dtype, mode, d):
    """The key just outside the window would carry the whole output if it were seen, and the key
    just inside does: queries and keys are made so that the scores of these two keys stand out
    against hundreds of others, in a prompt portion and for a token decoded alone."""
    # (head sizes 64 and 128 take the tcgen05 prompt kernel in bfloat16, 16 the mma.sync one)
    heads, kv, dv, window, n = 2, 1, d, 70, 200
    g = torch.Generator().manual_seed(11)
    m = _attn(heads, kv, d, dv, 16.0 / d, mask=window)

    def tweak(w):
        w["mix.pb"] = torch.full((heads,), -12.0).bfloat16()  # an ordinary key weighs e^-12
        # the first input coordinate drives every dimension of queries and keys
        w["mix.q"][:, 0] = 1.0
        w["mix.k"][:, 0] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention_2", m, 16, dtype, g, page=16, n_pages=16, std=0.05, tweak=tweak)
    x = 0.1 * torch.randn(n, 16, generator=g)
    x[:, 0] = 0.0
    query = n - 1
    inside, outside = query - window + 1, query - window
    for i in (query, inside, outside):
        x[i, 0] = 1.0  # score 16 against the gate's -12
    x = x.to(dtype)
    ref = ps.sigmoid_attention(x.double(), m, w, "mix.")
    without = ps.sigmoid_attention(x.double(), dict(m, mask=dict(size=window - 1)), w, "mix.")
    wider = ps.sigmoid_attention(x.double(), dict(m, mask=dict(size=window + 1)), w, "mix.")
    scale = float(ref[query].abs().max())
    # the construction works: one key more or less changes the row by a large part of itself
    assert float((ref[query] - without[query]).abs().max()) > 0.2 * scale
    assert float((ref[query] - wider[query]).abs().max()) > 0.2 * scale
    portions = (150, 50) if mode == "prompt" else (150, 30) + (1,) * 20
    out, _ = _run_mixer(mixer, cache, x, portions, dtype)
    ops.check_status()
    tol = (2e-5 if dtype == torch.float32 else 2.5e-2) * scale
    assert float((out[query] - ref[query]).abs().max()) <= tol
    assert float((out - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 2.5e-2) * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_far_key_shows(dtype):
    """One key hundreds of positions back takes nearly all of a query's weight (their vectors are
    scaled so that the score stands out), across many pages; its value arrives turned by the
    distance.  Decoded alone and inside a portion."""
    heads, kv, d, dv, n = 2, 1, 64, 64, 420
    g = torch.Generator().manual_seed(12)
    m = _attn(heads, kv, d, dv, 0.25, dims=2, base=10000.0)  # one pair turns: the far score does not fade

    def tweak(w):
        # the first input coordinate drives every dimension of queries and keys
        w["mix.q"][:, 0] = 1.0
        w["mix.k"][:, 0] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 32, dtype, g, page=16, n_pages=32, std=0.05, tweak=tweak)
    x = 0.1 * torch.randn(n, 32, generator=g)
    x[:, 0] = 0.0
    far, q1, q2 = 3, n - 1, n - 40
    for i in (far, q1, q2):
        x[i, 0] = 1.0  # score 16 among scores near 0
    x = x.to(dtype)
    ref = ps.softmax_attention(x.double(), m, w, "mix.")
    # without the far key the rows would be others
    x0 = x.clone()
    x0[far] = 0
    other = ps.softmax_attention(x0.double(), m, w, "mix.")
    assert float((ref[q1] - other[q1]).abs().max()) > 0.15 * float(ref[q1].abs().max())
    out, _ = _run_mixer(mixer, cache, x, (300, 100) + (1,) * 20, dtype)
    ops.check_status()
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    for i in (q1, q2):
        assert float((out[i] - ref[i]).abs().max()) <= tol * float(ref[i].abs().max()), i
    assert float((out - ref).abs().max()) <= tol * float(ref.abs().max())


# ---------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["sx_a", "sx_b", "sx_c"])
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
    outputs, engine = H.run_engine(d, dtype, steps, page, H.max_live_tokens(steps, page))
    compare(d, requests, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0 and all(f == g.pool.n_pages for f, g in zip(engine.cache.free_pages(), engine.cache.groups))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_batching_changes_nothing(tmp_path, dtype):
    """A request's logits in a batch of unequal requests equal those it gets alone (bitwise in
    float32, where every sum has a fixed order; within rounding in bfloat16, where the products
    of a few tokens and of many run in different kernels)."""
    d = make_dir(tmp_path, "sx_a")
    requests = _requests(211, [41, 5, 77, 20], 60)
    alone = H.plan_portions(requests, sizes=(9, 1, 1, 30))
    out_a, _ = H.run_engine(d, dtype, alone, 8, H.max_live_tokens(alone, 8))
    got_a = H.collect(alone, out_a)
    mixed = H.plan_mixed(requests, seed=2)
    out_m, _ = H.run_engine(d, dtype, mixed, 8, H.max_live_tokens(mixed, 8))
    got_m = H.collect(mixed, out_m)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_a[rid][p], got_m[rid][p]), (rid, p)
            else:
                H.check_row(got_m[rid][p], got_a[rid][p], dtype, f"{rid} {p}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_past_windows_and_pages(tmp_path, dtype):
    """200 tokens decoded one by one after a two-token prompt: every window passes over decoded
    tokens, pages of the windowed layers come back and are taken again."""
    d = make_dir(tmp_path, "sx_a")
    requests = _requests(211, [202], 77)
    steps = H.plan_decode_tail(requests, 200)
    outputs, engine = H.run_engine(d, dtype, steps, 8, 208)
    compare(d, requests, H.collect(steps, outputs), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    """``Fastgen.generate`` with its scheduler (portions of 16 tokens, batches of 3, graphs for
    the decode steps) against greedy decoding with the plain implementation."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    d = make_dir(tmp_path, "sx_a")
    cfg, w = ps.read_model(d, torch.float64)
    prompts = [H.random_tokens(211, n, 90 + n) for n in (7, 1, 40, 23)]
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
            assert got[i] == ps.greedy(cfg, w, p, 12), i
        else:
            seq = list(p)
            for tok in got[i]:
                logits = ps.forward(cfg, w, seq)[-1]
                assert float(logits[tok]) >= float(logits.max()) - 0.03 * float(logits.abs().max())
                seq.append(tok)
