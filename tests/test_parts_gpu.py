"""Each part alone against the plain implementation's function for it, and a toy mixer with state of its
own that is registered, built and stepped without touching the package."""
import dataclasses
import math
from typing import ClassVar

import numpy as np
import pytest
import torch

import helpers
import plain_opt
from swifttransformer_b200 import ops
from swifttransformer_b200.cache import CacheManager
from swifttransformer_b200.config.base import ModelConfig, register_config
from swifttransformer_b200.engine.step import ModelRunner, StepEntry
from swifttransformer_b200.models import LayerStep, ModelDef, load_model, register_model, write_random_model
from swifttransformer_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Delta, Embedding,
                                         Mixer, OutputHead, ResidualStream, StateSpec)
from swifttransformer_b200.parts.base import FeedForward
from swifttransformer_b200.parts.position import PositionEncoding
from swifttransformer_b200.weights import MATRIX, ParamSpec

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).normal(size=shape) * scale).astype(np.float32)


def dev(a, dtype=torch.float32):
    return torch.tensor(a).to(dtype).to(DEV)


def bf(a):
    """Round to bfloat16 and back: what a bfloat16 part sees."""
    return torch.tensor(a).to(torch.bfloat16).float().numpy()


def close(got, ref, dtype, rel32=3e-6, rel16=1.2e-2):
    got = got.float().cpu().numpy()
    tol = (rel32 if dtype == torch.float32 else rel16) * max(np.abs(ref).max(), 1e-6)
    assert np.abs(got - ref).max() <= tol, (np.abs(got - ref).max(), tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    W, n = 200, 9
    x, g, b = rnd((n, W), 1) + 5, 1 + rnd((W,), 2, 0.1), rnd((W,), 3, 0.1)
    norm = NORMS.build("layernorm", width=W, eps=2e-4, affine=True, prefix="n")
    assert [s.name for s in norm.param_specs()] == ["n.weight", "n.bias"]
    norm.bind({"n.weight": dev(g), "n.bias": dev(b)})
    xs = dev(x)
    out = norm.apply(xs, None, act_dtype=dtype)
    close(out, plain_opt.layer_norm(x.astype(np.float64), g, b, 2e-4), dtype)
    assert torch.equal(xs.cpu(), torch.tensor(x))
    plain = NORMS.build("layernorm", width=W, eps=2e-4, affine=False, prefix="n")
    assert plain.param_specs() == []
    close(plain.apply(dev(x), None, act_dtype=dtype), plain_opt.layer_norm(x.astype(np.float64), None, None, 2e-4), dtype)
    rms = NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix="r")
    rms.bind({"r.weight": dev(g)})
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6) * g
    close(rms.apply(dev(x), None, act_dtype=dtype), ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_feed_forward_part(dtype, act):
    H, F, n = 72, 200, 11
    w1, b1, w2, b2 = rnd((F, H), 4, 0.2), rnd((F,), 5, 0.2), rnd((H, F), 6, 0.2), rnd((H,), 7, 0.2)
    x = rnd((n, H), 8)
    if dtype == torch.bfloat16:
        w1, w2, x = bf(w1), bf(w2), bf(x)
    ffn = FEED_FORWARDS.build("dense", hidden=H, inner=F, activation=act, fc1_name="f1", fc2_name="f2", bias=True)
    ffn.bind({"f1.weight": dev(w1, dtype), "f1.bias": dev(b1), "f2.weight": dev(w2, dtype), "f2.bias": dev(b2)})
    d = ffn.forward(dev(x, dtype), None)
    got = d.value.float() + d.bias
    w = {"fc1.weight": w1.astype(np.float64), "fc1.bias": b1, "fc2.weight": w2.astype(np.float64), "fc2.bias": b2}
    ref = plain_opt.feed_forward(x.astype(np.float64), w, "", dict(enable_bias=True, activation_function=act))
    close(got, ref, dtype)
    with pytest.raises(ValueError, match="swish"):
        FEED_FORWARDS.build("dense", hidden=H, inner=F, activation="swish", fc1_name="a", fc2_name="b")


class OneStep:
    """A hand-made step context for one request that brings all its tokens at once."""

    def __init__(self, n, cache, slot, start=0):
        i32 = dict(dtype=torch.int32, device=DEV)
        self.n_tokens, self.n_seqs = n, 1
        self.token_ids = torch.zeros(n, **i32)
        self.positions = torch.arange(start, start + n, **i32)
        self.seq_of_token = torch.zeros(n, **i32)
        self.q_start = torch.tensor([0, n], **i32)
        self.start_pos = torch.tensor([start], **i32)
        self.kv_len = torch.tensor([start + n], **i32)
        self.slots = torch.tensor([slot], **i32)
        self.status = torch.zeros(1, **i32)
        from swifttransformer_b200.parts.attention import AttentionStepView
        tr = ops.attention_prefill_tile_rows()
        tiles = torch.tensor([v for off in range(0, n, tr) for v in (0, off)] or [0], **i32)
        self._plan = AttentionStepView(torch.arange(n, **i32), n if n < 16 else 0, tiles,
                                       0 if n < 16 else (n + tr - 1) // tr, start + n)
        self._buf = None

    def plan(self, name):
        assert name == "paged_attention"
        return self._plan

    def scratch_f32(self, k):
        self._buf = torch.empty(max(k, 1), device=DEV)
        return self._buf


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [7, 90, 128])
def test_attention_part(dtype, n):
    H, nh = 96, 3
    d = H // nh
    ws = {k: rnd((H, H), 10 + i, 0.15) for i, k in enumerate("qkvo")}
    bs = {k: rnd((H,), 20 + i, 0.1) for i, k in enumerate("qkvo")}
    x = rnd((n, H), 30)
    if dtype == torch.bfloat16:
        ws = {k: bf(v) for k, v in ws.items()}
        x = bf(x)
    mixer = MIXERS.build("attention", hidden=H, num_heads=nh, head_dim=d, bias=True,
                         names={k: f"a.{k}" for k in "qkvo"})
    assert len(mixer.param_specs()) == 8
    t = {}
    for k in "qkvo":
        t[f"a.{k}.weight"], t[f"a.{k}.bias"] = dev(ws[k], dtype), dev(bs[k])
    mixer.bind(t)
    cache = CacheManager([mixer.cache_spec()], dtype, DEV, page_size=8, num_pages=20, max_seqs=2, max_seq_len=160)
    slot = cache.alloc_slot()
    assert cache.reserve(slot, 0, n)
    for idx, val in cache.groups[0].take_updates():
        cache.groups[0].block_table.view(-1)[idx] = val
    ctx = OneStep(n, cache, slot)
    out = mixer.forward(dev(x, dtype), ctx, cache.entries()[0].view())
    got = out.value.float() + out.bias
    w = {}
    for k, name in zip("qkvo", ("q_proj", "k_proj", "v_proj", "out_proj")):
        w[f"{name}.weight"], w[f"{name}.bias"] = ws[k].astype(np.float64), bs[k].astype(np.float64)
    ref = plain_opt.attention_block(x.astype(np.float64), w, "", dict(num_attention_heads=nh, enable_bias=True))
    close(got, ref, dtype, rel16=2e-2)
    assert int(ctx.status.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    V, E, H, P, off = 300, 40, 56, 30, 2
    table, pin, pout, ptab = rnd((V, E), 40), rnd((H, E), 41, 0.2), rnd((E, H), 42, 0.2), rnd((P + off, H), 43)
    if dtype == torch.bfloat16:
        table, pin, pout, ptab = bf(table), bf(pin), bf(pout), bf(ptab)
    emb = Embedding(V, E, H, "tok", "pin")
    pos = POSITION_ENCODINGS.build("learned", max_positions=P, width=H, offset=off, name="pos")
    head = OutputHead(V, E, H, "head", tied_to="tok", project_out_name="pout")
    assert [s.shape for s in pos.param_specs()] == [(P + off, H)]
    tensors = {"tok": dev(table, dtype), "pin": dev(pin, dtype), "pos": dev(ptab, dtype), "pout": dev(pout, dtype)}
    tensors["head"] = tensors["tok"]
    for p in (emb, pos, head):
        p.bind(tensors)
    ids = np.array([5, 299, 0, 17, 5])
    positions = np.array([0, 1, 29, 3, 4])
    x = emb.forward(dev(ids, torch.int32), dev(positions, torch.int32), pos)
    ref = plain_opt.linear(plain_opt.embed_tokens(ids, table.astype(np.float64)), pin.astype(np.float64)) \
        + plain_opt.learned_positions(positions, ptab.astype(np.float64), off)
    close(x, ref, dtype, rel16=6e-3)
    h = rnd((4, H), 44)
    if dtype == torch.bfloat16:
        h = bf(h)
    logits = head.forward(dev(h, dtype))
    assert logits.dtype == torch.float32
    ref = plain_opt.linear(plain_opt.linear(h.astype(np.float64), pout.astype(np.float64)), table.astype(np.float64))
    close(logits, ref, dtype, rel16=8e-3)
    with pytest.raises(ValueError, match="input projection"):
        Embedding(V, E, H, "tok", None)


@pytest.mark.parametrize("order", ["pre_norm", "post_norm"])
def test_block_arrangement(order):
    """A block with stand-in sub-layers: only the wiring around the residual stream is under test."""
    W, n = 48, 6

    class Scale(Mixer):
        def __init__(self, k):
            self.k = k

        def forward(self, h, ctx, cache=None):
            return Delta((h.float() * self.k).to(h.dtype), torch.full((W,), 0.25, device=DEV))
    n1 = NORMS.build("layernorm", width=W, eps=1e-5, affine=False, prefix="a")
    n2 = NORMS.build("layernorm", width=W, eps=1e-5, affine=False, prefix="b")
    blk = BLOCKS.build(order, mixer=Scale(2.0), feed_forward=Scale(-0.5), norm1=n1, norm2=n2)
    x = rnd((n, W), 50)
    stream = ResidualStream(dev(x), torch.float32)
    blk.forward(stream, None, None)
    got = stream.materialise().cpu().numpy()
    ln = lambda t: plain_opt.layer_norm(t, None, None, 1e-5)
    x64 = x.astype(np.float64)
    if order == "pre_norm":
        r = x64 + 2.0 * ln(x64) + 0.25
        ref = r + (-0.5) * ln(r) + 0.25
    else:
        r = ln(x64 + 2.0 * x64 + 0.25)
        ref = ln(r + (-0.5) * r + 0.25)
    assert np.abs(got - ref).max() < 2e-5


# ---------------------------------------------------------------------------------------------
# A toy architecture defined here: layers alternate the package's attention with a mixer that keeps
# a running average per request in a state slot.  Nothing in the package knows about it.
# ---------------------------------------------------------------------------------------------
@register_config
@dataclasses.dataclass(frozen=True)
class ToyConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "ToyStateForCausalLM"
    vocab_size: int
    width: int
    layers: int
    heads: int
    inner: int
    decay: float
    max_positions: int
    on_device: bool = False      # the running average computed by device operations only (its steps can be recorded)


@MIXERS.register("toy_running_average")
class RunningAverage(Mixer):
    """s_t = decay * s_{t-1} + (1 - decay) * h_t per request;  out_t = s_t W^T.  State: s, [width] float32."""
    graph_safe = False

    def __init__(self, width, decay, name):
        self.width, self.decay, self.name = width, decay, name

    def param_specs(self):
        return [ParamSpec(self.name + ".weight", (self.width, self.width), MATRIX)]

    def bind(self, tensors):
        self.w = tensors[self.name + ".weight"]

    def cache_spec(self):
        return StateSpec((self.width,), torch.float32)

    def forward(self, h, ctx, cache):
        out = torch.empty_like(h)
        for i, slot in enumerate(ctx.h_slots):
            s = cache.state[slot]
            for t in range(ctx.h_q_start[i], ctx.h_q_start[i + 1]):
                s.mul_(self.decay).add_(h[t].float(), alpha=1 - self.decay)
                out[t] = (s @ self.w.float().t()).to(h.dtype)
        return Delta(out)


@MIXERS.register("toy_running_average_on_device")
class RunningAverageOnDevice(RunningAverage):
    """The same mixer without host work, so that its steps are recorded and replayed: the portion's tokens are
    folded with a prefix sum (s_t = decay^(j+1) s_before + (1 - decay) sum_{u <= t} decay^(t-u) h_u, j the token's
    place in its portion), padding tokens (position -1) contribute nothing, and a request's state moves by the
    difference its last token makes (a fixed-shape scatter-add; padding adds zero)."""
    graph_safe = True

    def forward(self, h, ctx, cache):
        n = h.shape[0]
        seq = ctx.seq_of_token.long()
        live = ctx.positions >= 0
        first = ctx.q_start.long()[seq]
        t = torch.arange(n, device=h.device)
        j = (t - first).clamp(min=0).double()
        hd = torch.where(live[:, None], h.double(), torch.zeros((), dtype=torch.float64, device=h.device))
        scaled = hd * (self.decay ** -j)[:, None]
        run = torch.cumsum(scaled, 0)
        within = (run - (run[first] - scaled[first])) * (self.decay ** j)[:, None]
        slot = ctx.slots.long()[seq]
        before = cache.state[slot].double()
        s = (self.decay ** (j + 1))[:, None] * before + (1 - self.decay) * within
        out = (s.float() @ self.w.float().t()).to(h.dtype)
        is_last = live & (t + 1 == ctx.q_start.long()[seq + 1])
        cache.state.index_add_(0, slot, ((s - before) * is_last[:, None]).float())
        return Delta(out)


@register_model(ToyConfig.ARCHITECTURE)
def build_toy(cfg):
    W = cfg.width
    emb = Embedding(cfg.vocab_size, W, W, "tok.weight")
    pos = POSITION_ENCODINGS.build("learned", max_positions=cfg.max_positions, width=W, offset=0, name="pos.weight")
    blocks = []
    for i in range(cfg.layers):
        if i % 2 == 0:
            mixer = MIXERS.build("toy_running_average_on_device" if cfg.on_device else "toy_running_average",
                                 width=W, decay=cfg.decay, name=f"l{i}.avg")
        else:
            mixer = MIXERS.build("attention", hidden=W, num_heads=cfg.heads, head_dim=W // cfg.heads, bias=False,
                                 names={k: f"l{i}.{k}" for k in "qkvo"})
        ffn = FEED_FORWARDS.build("dense", hidden=W, inner=cfg.inner, activation="relu", fc1_name=f"l{i}.up",
                                  fc2_name=f"l{i}.down", bias=False)
        blocks.append(BLOCKS.build("pre_norm", mixer=mixer, feed_forward=ffn,
                                   norm1=NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix=f"l{i}.n1"),
                                   norm2=NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix=f"l{i}.n2")))
    head = OutputHead(cfg.vocab_size, W, W, "head.weight", tied_to="tok.weight")
    # the order of layers is data: layer 1 (attention) runs a second time at the end with a cache of its own
    order = [LayerStep(i, i) for i in range(cfg.layers)] + [LayerStep(1, cfg.layers)]
    return ModelDef(cfg, emb, pos, blocks, order, NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix="fn"), head)


def toy_plain(model_dir, cfg, ids):
    _, w = plain_opt.load_model(model_dir)
    rms = lambda x, g: x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6) * g
    x = w["tok.weight"][ids] + w["pos.weight"][np.arange(len(ids))]
    for i in list(range(cfg.layers)) + [1]:
        h = rms(x, w[f"l{i}.n1.weight"])
        if i % 2 == 0:
            s, rows = np.zeros(cfg.width), []
            for t in range(len(ids)):
                s = cfg.decay * s + (1 - cfg.decay) * h[t]
                rows.append(s @ w[f"l{i}.avg.weight"].T)
            a = np.stack(rows)
        else:
            q, k, v = (h @ w[f"l{i}.{n}.weight"].T for n in "qkv")
            a = plain_opt.causal_attention(q, k, v, cfg.heads) @ w[f"l{i}.o.weight"].T
        x = x + a
        h = rms(x, w[f"l{i}.n2.weight"])
        x = x + np.maximum(h @ w[f"l{i}.up.weight"].T, 0) @ w[f"l{i}.down.weight"].T
    return rms(x, w["fn.weight"]) @ w["tok.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_runs_through_the_engine(tmp_path, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    cfg = ToyConfig(vocab_size=211, width=48, layers=3, heads=3, inner=100, decay=0.8, max_positions=96)
    d = write_random_model(str(tmp_path / "toy"), cfg, seed=3, std=0.15)
    model = load_model(d, dtype, DEV)
    specs = model.definition.cache_specs()
    assert isinstance(specs[0], StateSpec) and isinstance(specs[2], StateSpec) and len(specs) == 4
    assert not model.graph_safe()
    reqs = {"p": helpers.random_tokens(211, 70, 1), "q": helpers.random_tokens(211, 41, 2),
            "r": helpers.random_tokens(211, 23, 3)}
    refs = {k: toy_plain(d, cfg, np.array(v)) for k, v in reqs.items()}
    for build in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, max_live=2, chunk=9)):
        steps = build(reqs)
        s = TraceSession(d, dtype, helpers.live_token_need(steps), page_size=8, max_requests=2)
        got = helpers.replay(s, steps)
        for k in reqs:
            scale = np.abs(refs[k]).max()
            bad = helpers.first_bad(got[k], refs[k], helpers.TOL[dtype] * scale)
            assert bad is None, (k, bad)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_steps_move_per_request_state_once(tmp_path, dtype):
    """A mixer with state of its own and no host work: its steps are recorded as graphs.  The first use of a
    shape (the pass that sizes scratch memory, then the recording, then the replay) must move a request's
    state exactly once: the logits of recorded steps equal the plain implementation's and those of the same
    steps launched one by one."""
    from swifttransformer_b200.engine.replay import TraceSession
    cfg = ToyConfig(vocab_size=211, width=48, layers=3, heads=3, inner=100, decay=0.8, max_positions=96, on_device=True)
    d = write_random_model(str(tmp_path / "toyd"), cfg, seed=3, std=0.15)
    model = load_model(d, dtype, DEV)
    assert model.graph_safe() and isinstance(model.definition.cache_specs()[0], StateSpec)
    reqs = {"p": helpers.random_tokens(211, 70, 1), "q": helpers.random_tokens(211, 41, 2),
            "r": helpers.random_tokens(211, 23, 3)}
    refs = {k: toy_plain(d, cfg, np.array(v)) for k, v in reqs.items()}
    for build in (helpers.trace_whole, lambda r: helpers.trace_decode_tail(r, tail=20), helpers.trace_portions,
                  lambda r: helpers.trace_mixed(r, max_live=2, chunk=9)):
        steps = build(reqs)
        outs = []
        for graphs in (True, False):
            s = TraceSession(d, dtype, helpers.live_token_need(steps), page_size=8, max_requests=2)
            s.runner.use_cuda_graphs = graphs
            outs.append(helpers.replay(s, steps))
            assert (s.runner.graph_steps + s.runner.padded_graph_steps > 0) == graphs
        for k in reqs:
            scale = np.abs(refs[k]).max()
            bad = helpers.first_bad(outs[0][k], refs[k], helpers.TOL[dtype] * scale)
            assert bad is None, ("recorded against plain", k, bad)
            tol = (1e-5 if dtype == "float32" else 3e-2) * scale
            assert helpers.first_bad(outs[0][k], outs[1][k], tol) is None, ("recorded against launched one by one", k)


# ---------------------------------------------------------------------------------------------
# A second toy architecture: attention only, but the layers differ.  Even layers see every key, odd layers
# a window of them with grouped queries, so the model has two cache groups with pages of their own (the
# window group's pages are given back while a request runs); the last step of the layer order runs layer 0
# again and reads layer 0's cache instead of writing one.
# ---------------------------------------------------------------------------------------------
@register_config
@dataclasses.dataclass(frozen=True)
class ToyWindowConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "ToyWindowForCausalLM"
    vocab_size: int
    width: int
    layers: int
    heads: int
    kv_heads: int
    window: int
    inner: int
    max_positions: int


@register_model(ToyWindowConfig.ARCHITECTURE)
def build_toy_window(cfg):
    W, d = cfg.width, cfg.width // cfg.heads
    emb = Embedding(cfg.vocab_size, W, W, "tok.weight")
    pos = POSITION_ENCODINGS.build("learned", max_positions=cfg.max_positions, width=W, offset=0, name="pos.weight")
    blocks = []
    for i in range(cfg.layers):
        odd = i % 2 == 1
        mixer = MIXERS.build("attention", hidden=W, num_heads=cfg.heads, head_dim=d, bias=True,
                             num_kv_heads=cfg.kv_heads if odd else cfg.heads, window=cfg.window if odd else None,
                             names={k: f"l{i}.{k}" for k in "qkvo"})
        ffn = FEED_FORWARDS.build("dense", hidden=W, inner=cfg.inner, activation="gelu", fc1_name=f"l{i}.up",
                                  fc2_name=f"l{i}.down", bias=True)
        blocks.append(BLOCKS.build("pre_norm", mixer=mixer, feed_forward=ffn,
                                   norm1=NORMS.build("layernorm", width=W, eps=1e-5, affine=True, prefix=f"l{i}.n1"),
                                   norm2=NORMS.build("layernorm", width=W, eps=1e-5, affine=True, prefix=f"l{i}.n2")))
    head = OutputHead(cfg.vocab_size, W, W, "head.weight", tied_to="tok.weight")
    order = [LayerStep(i, i) for i in range(cfg.layers)] + [LayerStep(0, 0, writes_cache=False)]
    return ModelDef(cfg, emb, pos, blocks, order, NORMS.build("layernorm", width=W, eps=1e-5, affine=True, prefix="fn"), head)


def toy_window_plain(model_dir, cfg, ids):
    """Whole sequence, no cache.  The repeated layer 0 reads the keys and values its first run wrote."""
    _, w = plain_opt.load_model(model_dir)
    ln = lambda x, p: plain_opt.layer_norm(x, w[p + ".weight"], w[p + ".bias"], 1e-5)
    lin = lambda x, p: x @ w[p + ".weight"].T + w[p + ".bias"]
    x = w["tok.weight"][ids] + w["pos.weight"][np.arange(len(ids))]
    kv0 = None
    for step, i in enumerate(list(range(cfg.layers)) + [0]):
        odd = i % 2 == 1
        h = ln(x, f"l{i}.n1")
        q, k, v = (lin(h, f"l{i}.{n}") for n in "qkv")
        if step == 0:
            kv0 = (k, v)
        if step == cfg.layers:
            k, v = kv0
        if odd:      # grouped queries: every kv head serves heads / kv_heads query heads
            d = cfg.width // cfg.heads
            rep = cfg.heads // cfg.kv_heads
            k = np.repeat(k.reshape(len(ids), cfg.kv_heads, d), rep, axis=1).reshape(len(ids), -1)
            v = np.repeat(v.reshape(len(ids), cfg.kv_heads, d), rep, axis=1).reshape(len(ids), -1)
        a = plain_opt.causal_attention(q, k, v, cfg.heads, window=cfg.window if odd else None)
        x = x + lin(a, f"l{i}.o")
        h = ln(x, f"l{i}.n2")
        x = x + lin(plain_opt.activation(lin(h, f"l{i}.up"), "gelu"), f"l{i}.down")
    return ln(x, "fn") @ w["tok.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_and_a_shared_cache_run_through_the_engine(tmp_path, dtype):
    """Two cache groups (all keys; a window of 40 with two kv heads for four query heads), a layer that runs
    twice and reads its own first cache: whole, in portions, decoded one by one and mixed with page reuse, the
    logits match a plain implementation; the window group needs far fewer pages than the tokens it saw."""
    from swifttransformer_b200.engine.replay import TraceSession
    cfg = ToyWindowConfig(vocab_size=301, width=128, layers=4, heads=4, kv_heads=2, window=40, inner=200,
                          max_positions=400)
    d = write_random_model(str(tmp_path / "toyw"), cfg, seed=5, std=0.1)
    model = load_model(d, dtype, DEV)
    specs = model.definition.cache_specs()
    assert [s.window for s in specs] == [None, 40, None, 40]
    reqs = {"p": helpers.random_tokens(301, 330, 11), "q": helpers.random_tokens(301, 150, 12),
            "r": helpers.random_tokens(301, 77, 13), "s": helpers.random_tokens(301, 200, 14)}
    refs = {k: toy_window_plain(d, cfg, np.array(v)) for k, v in reqs.items()}
    for build in (helpers.trace_whole, helpers.trace_decode_tail, helpers.trace_portions,
                  lambda r: helpers.trace_mixed(r, max_live=3, chunk=50)):
        steps = build(reqs)
        s = TraceSession(d, dtype, helpers.live_token_need(steps), page_size=16, max_requests=3)
        got = helpers.replay(s, steps)
        for k in reqs:
            scale = np.abs(refs[k]).max()
            bad = helpers.first_bad(got[k], refs[k], helpers.TOL[dtype] * scale)
            assert bad is None, (build, k, bad)
        s.runner.check_status()
    # the window group gives pages back while a request runs: 330 tokens pass through 6 pages of 16
    from swifttransformer_b200.cache import CacheManager
    cm = CacheManager(specs, model.dtype, DEV, 16, 24, 2, 400)
    g_win = next(g for g in cm.groups if g.spec.window == 40)
    slot = cm.alloc_slot()
    peak = 0
    for start in range(0, 330, 10):
        assert cm.reserve(slot, start, min(330, start + 10))
        cm.commit(slot, min(330, start + 10))
        peak = max(peak, g_win.pool.num_pages - g_win.pool.num_free)
    assert peak <= 5 and cm.groups[0].pool.num_pages - cm.groups[0].pool.num_free == 21


# ---------------------------------------------------------------------------------------------
# A third toy architecture, for the two remaining kinds of part: a position encoding that acts on queries and
# keys (pairs of dimensions turned by an angle that grows with the position; the hidden state gets no
# position at all), and a feed-forward that routes every token to two of its experts.  Both are defined here
# with device operations only, registered, and run through the engine; nothing in the package knows them.
# ---------------------------------------------------------------------------------------------
@register_config
@dataclasses.dataclass(frozen=True)
class ToyRoutedConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "ToyRoutedForCausalLM"
    vocab_size: int
    width: int
    layers: int
    heads: int
    experts: int
    inner: int
    turn: float


@POSITION_ENCODINGS.register("toy_turn")
class ToyTurn(PositionEncoding):
    """Dimension pair (2i, 2i+1) of every query and key head is turned by position * turn / (i + 1)."""

    def __init__(self, turn, head_dim):
        self.turn, self.head_dim = turn, head_dim

    def apply_qk(self, q, k, ctx):
        i = torch.arange(self.head_dim // 2, device=q.device, dtype=torch.float32)
        ang = ctx.positions.to(torch.float32)[:, None] * (self.turn / (i + 1))[None, :]      # [N, d/2], float32
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for x in (q, k):
            a, b = x[..., 0::2].float(), x[..., 1::2].float()
            even, odd = a * c - b * s, a * s + b * c            # both before either is stored: float() may be a view
            x[..., 0::2] = even.to(x.dtype)
            x[..., 1::2] = odd.to(x.dtype)


@FEED_FORWARDS.register("toy_routed")
class ToyRouted(FeedForward):
    """y = sum over the two experts e with the largest router logits of softmax-weight_e * W2_e relu(W1_e h);
    router logits and weights in float32."""

    def __init__(self, hidden, inner, experts, prefix):
        self.hidden, self.inner, self.experts, self.prefix = hidden, inner, experts, prefix

    def param_specs(self):
        p = self.prefix
        return [ParamSpec(p + ".router.weight", (self.experts, self.hidden), MATRIX),
                ParamSpec(p + ".w1", (self.experts * self.inner, self.hidden), MATRIX),
                ParamSpec(p + ".w2", (self.experts * self.hidden, self.inner), MATRIX)]

    def bind(self, tensors):
        p = self.prefix
        self.router = tensors[p + ".router.weight"]
        self.w1 = tensors[p + ".w1"].view(self.experts, self.inner, self.hidden)
        self.w2 = tensors[p + ".w2"].view(self.experts, self.hidden, self.inner)

    def forward(self, h, ctx):
        logits = h.float() @ self.router.float().t()                       # [N, E]
        top, idx = torch.topk(logits, 2, dim=-1)
        gate = torch.softmax(top, dim=-1)                                   # over the two chosen
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in range(self.experts):                                       # every expert on all rows, masked: no host sync
            wgt = (gate * (idx == e)).sum(-1, keepdim=True)
            u = ops.linear(h, self.w1[e].contiguous(), None, "relu")
            out += wgt * ops.linear(u, self.w2[e].contiguous(), None, "none", torch.float32)
        return Delta(out.to(h.dtype))

    def param_bytes(self):
        return (self.router.numel() + self.w1.numel() + self.w2.numel()) * self.w1.element_size()


@register_model(ToyRoutedConfig.ARCHITECTURE)
def build_toy_routed(cfg):
    W, d = cfg.width, cfg.width // cfg.heads
    emb = Embedding(cfg.vocab_size, W, W, "tok.weight")
    turn = POSITION_ENCODINGS.build("toy_turn", turn=cfg.turn, head_dim=d)
    blocks = []
    for i in range(cfg.layers):
        mixer = MIXERS.build("attention", hidden=W, num_heads=cfg.heads, head_dim=d, bias=True, qk_position=turn,
                             names={k: f"l{i}.{k}" for k in "qkvo"})
        ffn = FEED_FORWARDS.build("toy_routed", hidden=W, inner=cfg.inner, experts=cfg.experts, prefix=f"l{i}.moe")
        blocks.append(BLOCKS.build("pre_norm", mixer=mixer, feed_forward=ffn,
                                   norm1=NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix=f"l{i}.n1"),
                                   norm2=NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix=f"l{i}.n2")))
    head = OutputHead(cfg.vocab_size, W, W, "head.weight", tied_to="tok.weight")
    return ModelDef(cfg, emb, POSITION_ENCODINGS.build("none"), blocks, [LayerStep(i, i) for i in range(cfg.layers)],
                    NORMS.build("rmsnorm", width=W, eps=1e-6, affine=True, prefix="fn"), head)


def toy_routed_plain(model_dir, cfg, ids):
    _, w = plain_opt.load_model(model_dir)
    rms = lambda x, g: x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6) * g
    T, d = len(ids), cfg.width // cfg.heads
    ang = np.arange(T)[:, None] * (cfg.turn / (np.arange(d // 2) + 1))[None, :]
    c, s = np.cos(ang), np.sin(ang)

    def turn(x):
        x = x.reshape(T, cfg.heads, d).copy()
        a, b = x[..., 0::2].copy(), x[..., 1::2].copy()
        x[..., 0::2] = a * c[:, None, :] - b * s[:, None, :]
        x[..., 1::2] = a * s[:, None, :] + b * c[:, None, :]
        return x.reshape(T, -1)

    x = w["tok.weight"][ids]
    sure = T          # positions before this one are routed with a clear margin in every layer
    for i in range(cfg.layers):
        h = rms(x, w[f"l{i}.n1.weight"])
        q, k, v = (h @ w[f"l{i}.{n}.weight"].T + w[f"l{i}.{n}.bias"] for n in "qkv")
        a = plain_opt.causal_attention(turn(q), turn(k), v, cfg.heads)
        x = x + a @ w[f"l{i}.o.weight"].T + w[f"l{i}.o.bias"]
        h = rms(x, w[f"l{i}.n2.weight"])
        logits = h @ w[f"l{i}.moe.router.weight"].T
        w1 = w[f"l{i}.moe.w1"].reshape(cfg.experts, cfg.inner, cfg.width)
        w2 = w[f"l{i}.moe.w2"].reshape(cfg.experts, cfg.width, cfg.inner)
        y = np.zeros_like(x)
        for t in range(T):
            ranked = np.sort(logits[t])[::-1]
            if ranked[1] - ranked[2] < 0.02 * np.abs(logits[t]).max():
                sure = min(sure, t)
            best = np.argsort(-logits[t], kind="stable")[:2]
            g = np.exp(logits[t][best] - logits[t][best].max())
            g = g / g.sum()
            for e, ge in zip(best, g):
                y[t] += ge * (w2[e] @ np.maximum(w1[e] @ h[t], 0))
        x = x + y
    return rms(x, w["fn.weight"]) @ w["tok.weight"].T, sure


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_query_key_positions_run_through_the_engine(tmp_path, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    cfg = ToyRoutedConfig(vocab_size=257, width=64, layers=2, heads=2, experts=4, inner=96, turn=0.37)
    d = write_random_model(str(tmp_path / "toyr"), cfg, seed=25, std=0.2)     # a seed with late near-ties
    model = load_model(d, dtype, DEV)
    assert model.graph_safe()
    reqs = {"p": helpers.random_tokens(257, 90, 21), "q": helpers.random_tokens(257, 41, 22),
            "r": helpers.random_tokens(257, 64, 23)}
    refs = {k: toy_routed_plain(d, cfg, np.array(v)) for k, v in reqs.items()}
    compared = 0
    for build in (helpers.trace_whole, helpers.trace_decode_tail, helpers.trace_portions,
                  lambda r: helpers.trace_mixed(r, max_live=3, chunk=20)):
        steps = build(reqs)
        s = TraceSession(d, dtype, helpers.live_token_need(steps), page_size=16, max_requests=3)
        got = helpers.replay(s, steps)
        for k in reqs:
            ref, sure = refs[k]
            scale = np.abs(ref).max()
            # bfloat16 may route a token whose second and third router logits are nearly tied to another
            # expert, and every later position reads that token's keys: a request is compared up to its
            # first such token.  float32 is compared everywhere.
            n = len(ref) if dtype == "float32" else sure
            compared += n
            bad = helpers.first_bad(got[k][:n], ref[:n], helpers.TOL[dtype] * scale)
            assert bad is None, (k, bad)
        s.runner.check_status()
        if build is helpers.trace_decode_tail:
            assert s.runner.graph_steps > 0, "decode steps of the toy model are recorded and replayed too"
    assert compared >= 4 * 100


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_without_a_position_table_generates_through_the_engine(tmp_path, dtype):
    """The third toy architecture has no position table, so nothing in the model bounds a request's length: the
    limit comes from the engine's configuration, block tables are sized by it, and requests generate through
    LLMEngine - continuous batching, recorded decode steps, a pool so small that requests are preempted and
    computed again - to the tokens the plain implementation gives."""
    from swifttransformer_b200.engine.engine import DEFAULT_MAX_SEQ_LEN, LLMEngine
    from swifttransformer_b200.sampling import SamplingParams
    cfg = ToyRoutedConfig(vocab_size=257, width=64, layers=2, heads=2, experts=4, inner=96, turn=0.37)
    d = write_random_model(str(tmp_path / "toyg"), cfg, seed=25, std=0.2)
    model = load_model(d, dtype, DEV)
    assert model.max_positions is None
    assert LLMEngine(model, page_size=16, num_pages=8, max_num_seqs=2).max_seq_len == DEFAULT_MAX_SEQ_LEN
    eng = LLMEngine(model, page_size=16, num_pages=7, max_batch_tokens=64, chunk_size=32, max_num_seqs=4,
                    max_seq_len=96)
    assert eng.cache.groups[0].block_table.shape == (4, 6)
    prompts = [helpers.random_tokens(257, n, 30 + i) for i, n in enumerate([15, 31, 14, 30, 9])]
    new = 12
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    eng.runner.check_status()
    assert eng.stats["preemptions"] > 0, "the pool was made too small for the requests to finish side by side"
    assert eng.runner.graph_steps > 0 and eng.cache.free_pages == eng.cache.total_pages
    for p, o in zip(prompts, outs):
        assert len(o) == new
        ids = list(p)
        for tok in o:
            logits, sure = toy_routed_plain(d, cfg, np.array(ids))
            if dtype == "bfloat16" and sure < len(ids):
                break                      # a nearly tied routing decision: bfloat16 may take the other expert
            best = int(np.argmax(logits[-1]))
            if dtype == "float32":
                assert tok == best
            elif tok != best:
                assert logits[-1][best] - logits[-1][tok] < 4e-2 * np.abs(logits[-1]).max()
            ids.append(tok)
    # a request may not outgrow the engine's limit
    with pytest.raises(ValueError, match="exceeds"):
        eng.add_request([5] * 97)
    out = eng.generate([[5] * 90], SamplingParams(max_new_tokens=50, ignore_eos=True))[0]
    assert len(out) == 6
