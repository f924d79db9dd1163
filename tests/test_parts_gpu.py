"""Each part alone against the plain implementation's function for it, and a toy model made
of parts the framework has never seen: a mixer with a state of its own, different mixers in
different layers, a layer that runs twice and a layer that reads another layer's cache; a
position encoding that turns queries and keys; a feed-forward with routing and another norm."""
import dataclasses
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _np(t):
    return t.detach().float().cpu().numpy()


def _spec(kind, params, names):
    from sandyrt_b200.models.spec import PartSpec

    return PartSpec(kind, params, {n: n for n in names})


def _harness(family, spec, dtype, **kw):
    """The host library's part of this description, alone: bound to seeded random tensors, with a
    poisoned cache of its own."""
    from sandyrt_b200.parts.harness import PartHarness

    return PartHarness(family, spec, dtype, **kw)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_layernorm_part(dtype, tol):
    part = _harness("norm", _spec("layernorm", {"width": 96, "eps": 1e-6}, ["weight", "bias"]), dtype, seed=1)
    w = part.tensors()
    x = torch.randn(11, 96, device=DEV) * 2 + 0.5
    out = torch.empty(11, 96, dtype=dtype, device=DEV)
    part.run_norm(x, out)
    rnd = plain.round_bf16 if dtype == torch.bfloat16 else (lambda a: a)
    want = plain.layer_norm(_np(x), rnd(w["weight"]), rnd(w["bias"]), 1e-6)
    assert np.abs(_np(out) - want).max() < tol
    # selected rows only (what the final norm does with the wanted rows)
    some = torch.empty(3, 96, dtype=dtype, device=DEV)
    part.run_norm(x, some, rows=[7, 0, 10])
    assert np.abs(_np(some) - want[[7, 0, 10]]).max() < tol


def test_embedding_with_learned_positions():
    emb = _harness("embedding", _spec("token_embedding", {"vocab_size": 77, "width": 48}, ["weight"]), torch.float32,
                   position=_spec("learned_absolute", {"width": 48, "max_positions": 20}, ["weight"]), seed=1)
    we, wp = emb.tensors(), emb.position_tensors()
    ids = [5, 76, 0, 13, 9, 9]
    emb.set_step([(3, 4), (0, 2)], ids)
    x = torch.empty(6, 48, device=DEV)
    emb.run_embedding(x)
    want = plain.embedding(ids, we["weight"]) + plain.embedding([3, 4, 5, 6, 0, 1], wp["weight"])
    np.testing.assert_allclose(_np(x), want, atol=1e-7)
    assert emb.info()["max_positions"] == 20
    nopos = _harness("embedding", _spec("token_embedding", {"vocab_size": 77, "width": 48}, ["weight"]), torch.float32,
                     position=_spec("none", {}, []), seed=1)
    assert nopos.info()["max_positions"] is None
    nopos.set_step([(3, 4), (0, 2)], ids)
    nopos.run_embedding(x)
    np.testing.assert_allclose(_np(x), plain.embedding(ids, nopos.tensors()["weight"]), atol=1e-7)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("activation,layout", [("gelu_new", "in_out"), ("gelu", "out_in")])
def test_dense_mlp_part(dtype, tol, activation, layout):
    part = _harness("feed_forward", _spec(
        "dense_mlp", {"width": 64, "inner": 200, "activation": activation, "weight_layout": layout},
        ["up.weight", "up.bias", "down.weight", "down.bias"]), dtype, seed=3)
    w = part.tensors()
    part.set_step([(0, 9)])
    h = torch.randn(9, 64, device=DEV).to(dtype)
    x = torch.randn(9, 64, device=DEV)
    x0 = _np(x).copy()
    part.run_feed_forward(h, x)
    store = "bf16" if dtype == torch.bfloat16 else "f32"
    rnd = plain.round_bf16 if store == "bf16" else (lambda a: a)
    wt = (lambda a: a) if layout == "in_out" else (lambda a: a.T)
    u = plain.linear_in_out(_np(h), rnd(wt(w["up.weight"])), rnd(w["up.bias"]))
    g = rnd(plain.gelu_new(u) if activation == "gelu_new" else plain.gelu_erf(u))
    want = x0 + plain.linear_in_out(g, rnd(wt(w["down.weight"])), rnd(w["down.bias"]))
    assert np.abs(_np(x) - want).max() < tol
    assert part.info()["weight_bytes"] == (2 * 64 * 200 + 200 + 64) * (2 if dtype == torch.bfloat16 else 4)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim,window", [(4, 4, 16, None), (6, 2, 32, None), (3, 3, 32, 9)])
def test_attention_part_whole_then_in_portions(dtype, tol, n_heads, n_kv_heads, head_dim, window):
    """The attention part over its own cache: a sequence in one step equals the same
    sequence in two portions plus single tokens (grouped heads and a window included)."""
    width = 80
    spec = _spec("causal_attention", {"width": width, "n_heads": n_heads, "n_kv_heads": n_kv_heads, "head_dim": head_dim,
                                      "scale": 0.3, "window": window, "weight_layout": "out_in"},
                 ["qkv.weight", "qkv.bias", "out.weight", "out.bias"])
    T = 37
    h_all = (torch.randn(T, width, device=DEV) * 1.5).to(dtype)
    w = None

    def run(cuts):
        nonlocal w
        part = _harness("mixer", spec, dtype, seed=4)      # a fresh cache; the same seed gives the same tensors
        w = part.tensors()
        outs, before = [], 0
        for n in cuts:
            part.set_step([(before, n)])
            x = torch.zeros(n, width, device=DEV)
            part.run_mixer(h_all[before:before + n].contiguous(), x)
            outs.append(_np(x))
            before += n
        return np.concatenate(outs)

    whole = run([T])
    parts = run([20, 2, 1, 1, 13])
    assert np.abs(whole - parts).max() < tol
    # against the plain functions
    rnd = plain.round_bf16 if dtype == torch.bfloat16 else (lambda a: a)
    qkv = rnd(plain.linear_in_out(_np(h_all), rnd(w["qkv.weight"].T), rnd(w["qkv.bias"])))
    qc, kc = n_heads * head_dim, n_kv_heads * head_dim
    split = lambda t, nh: t.reshape(T, nh, head_dim).transpose(1, 0, 2)
    o = plain.causal_attention(split(qkv[:, :qc], n_heads), split(qkv[:, qc:qc + kc], n_kv_heads),
                               split(qkv[:, qc + kc:], n_kv_heads), 0.3, window or 0)
    o = rnd(o.transpose(1, 0, 2).reshape(T, qc))
    want = plain.linear_in_out(o, rnd(w["out.weight"].T), rnd(w["out.bias"]))
    assert np.abs(whole - want).max() < tol


# ---- a toy architecture assembled from registered parts ---------------------------------------
def _register_toy():
    """Registers, from outside the framework: a mixer with per-request state of fixed size
    (an exponential moving average of its input), and an architecture that mixes it with
    attention layers, runs one layer twice and lets one layer read another layer's cache."""
    from sandyrt_b200.config.base import ModelConfig
    from sandyrt_b200.models.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
    from sandyrt_b200.parts.base import Mixer, StateSpec
    from sandyrt_b200.registry import register_architecture, register_part
    from sandyrt_b200.weights.loader import TensorRequest

    class EmaMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t (per channel);  x_t += s_t * gain.  State: s, float32 [width]."""
        graph_safe = False        # it plans its work from the step's host-side lists

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.decay = int(self.params["width"]), float(self.params["decay"])

        def requests(self):
            return {"gain": TensorRequest((self.width,), init="gamma")}

        def bind(self, tensors, device, dtype):
            self.gain = tensors["gain"].to(device=device, dtype=torch.float32)

        def cache_spec(self):
            return StateSpec((self.width,))

        def forward(self, ctx, h, x, call):
            state = ctx.caches.state(call.cache)
            t0 = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slots):
                s = state[slot].clone()
                for i in range(n):
                    s = self.decay * s + h[t0 + i].float()
                    x[t0 + i] += s * self.gain
                state[slot] = s
                t0 += n

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "ToyMixedModel"
        width: int = 0
        vocab_size: int = 0
        decay: float = 0.9

        @classmethod
        def from_dict(cls, raw):
            return cls(width=raw["width"], vocab_size=raw["vocab_size"], decay=raw["decay"])

        def to_dict(self):
            return {"architectures": [self.architecture], "width": self.width, "vocab_size": self.vocab_size,
                    "decay": self.decay}

        def validate(self):
            assert self.width % 16 == 0

    def describe(cfg):
        E = cfg.width
        norm = lambda n: PartSpec("layernorm", {"width": E, "eps": 1e-5}, {"weight": n + ".g", "bias": n + ".b"})
        mlp = lambda p: PartSpec("dense_mlp", {"width": E, "inner": 2 * E, "activation": "gelu_new",
                                               "weight_layout": "out_in"},
                                 {"up.weight": p + "up.w", "up.bias": p + "up.b", "down.weight": p + "dn.w",
                                  "down.bias": p + "dn.b"})
        attn = lambda p: PartSpec("causal_attention", {"width": E, "n_heads": 2, "n_kv_heads": 1, "head_dim": E // 2,
                                                       "scale": 1 / math.sqrt(E // 2), "weight_layout": "out_in"},
                                  {"qkv.weight": p + "qkv.w", "qkv.bias": p + "qkv.b", "out.weight": p + "o.w",
                                   "out.bias": p + "o.b"})
        layers = [
            LayerSpec("pre_norm", PartSpec("toy_ema", {"width": E, "decay": cfg.decay}, {"gain": "l0.gain"}),
                      mlp("l0."), {"mixer": norm("l0.n1"), "feed_forward": norm("l0.n2")}),
            LayerSpec("pre_norm", attn("l1."), mlp("l1."), {"mixer": norm("l1.n1"), "feed_forward": norm("l1.n2")}),
            LayerSpec("pre_norm", attn("l2."), mlp("l2."), {"mixer": norm("l2.n1"), "feed_forward": norm("l2.n2")}),
        ]
        schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(1, 2),          # layer 1 runs twice, two caches
                    LayerCall(2, 1, write_cache=False)]                          # layer 2 reads layer 1's first cache
        return ModelSpec(architecture=cfg.architecture, width=E, vocab_size=cfg.vocab_size, max_positions=None,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": E}, {"weight": "emb"}),
                         position=PartSpec("none", {}, {}), layers=layers, schedule=schedule,
                         final_norm=norm("nf"), head=PartSpec("output_head", {"vocab_size": cfg.vocab_size, "width": E,
                                                                              "tied": True}, {}))

    register_part("mixer", "toy_ema", EmaMixer)
    register_architecture("ToyMixedModel", ToyConfig, describe)
    return ToyConfig


def _toy_plain_logits(w, ids, decay, E):
    """The toy model, whole sequence, written with the plain implementation's functions."""
    T = len(ids)
    x = plain.embedding(ids, w["emb"])
    ln = lambda x, n: plain.layer_norm(x, w[n + ".g"], w[n + ".b"], 1e-5)
    lin = lambda h, p: plain.linear_in_out(h, w[p + "w"].T, w[p + "b"])
    mlp = lambda x, p: x + lin(plain.gelu_new(lin(ln(x, p + "n2"), p + "up.")), p + "dn.")
    D = E // 2
    split = lambda t, nh: t.reshape(T, nh, D).transpose(1, 0, 2)

    def attn(x, p, kv=None):
        qkv = lin(ln(x, p + "n1"), p + "qkv.")
        q = split(qkv[:, :E], 2)
        k, v = (split(qkv[:, E:E + D], 1), split(qkv[:, E + D:], 1)) if kv is None else kv
        o = plain.causal_attention(q, k, v, 1 / math.sqrt(D)).transpose(1, 0, 2).reshape(T, E)
        return x + lin(o, p + "o."), (k, v)

    h = ln(x, "l0.n1")
    s = np.zeros(E, np.float32)
    y = np.zeros_like(x)
    for t in range(T):
        s = decay * s + h[t]
        y[t] = s * w["l0.gain"]
    x = mlp(x + y, "l0.")
    x, kv1 = attn(x, "l1."); x = mlp(x, "l1.")
    x, _ = attn(x, "l1."); x = mlp(x, "l1.")
    x, _ = attn(x, "l2.", kv=kv1); x = mlp(x, "l2.")
    return plain.layer_norm(x, w["nf.g"], w["nf.b"], 1e-5) @ w["emb"].T


def test_toy_model_with_stateful_mixer_registers_builds_and_steps(tmp_path):
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model
    from sandyrt_b200.weights.random_init import write_random_model

    ToyConfig = _register_toy()
    cfg = ToyConfig(width=32, vocab_size=90, decay=0.8)
    d = write_random_model(cfg, str(tmp_path / "toy"), seed=3, dtype=torch.float32)
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["ToyMixedModel"]
    model = load_model(d, device=DEV, dtype=torch.float32)          # chosen by config.json through the registry
    assert not model.graph_safe
    eng = Engine(model, max_tokens=256, page_size=8, max_requests=3)
    layout = eng.cache.layout
    assert list(layout.state_of_cache) == [0] and len(layout.groups) == 1 and layout.groups[0].caches == [1, 2]
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    rng = np.random.default_rng(0)
    seqs = {name: rng.integers(0, 90, size=n).tolist() for name, n in (("a", 23), ("b", 9), ("c", 31), ("d", 14))}
    want = {k: _toy_plain_logits(w, v, 0.8, 32) for k, v in seqs.items()}
    got = {k: [] for k in seqs}
    # a and b start together; c joins when b has ended and takes over b's slot and pages
    plan = [
        [("a", 10), ("b", 9)], [("a", 1)], [("a", 2), ("c", 16)], [("c", 1), ("a", 10)], [("c", 14)],
        [("d", 14)],
    ]
    fed = {k: 0 for k in seqs}
    for step in plan:
        entries = [StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in step]
        out = eng.step(entries).cpu().numpy()
        r = 0
        for k, n in step:
            got[k].append(out[r:r + n].copy()); r += n; fed[k] += n
            if fed[k] == len(seqs[k]):
                eng.release(k)
        eng.cache.alloc.check()
    for k in seqs:
        np.testing.assert_allclose(np.concatenate(got[k]), want[k], atol=3e-5, rtol=1e-4, err_msg=f"sequence {k}")
    assert eng.cache.alloc.free_slots() == 3


def test_a_reused_state_slot_starts_from_zero_through_the_entry_point(tmp_path):
    """Generation admits requests through the scheduler.  With one slot, the second request gets
    the slot the first one left; its fixed-size state must start as zeros, so its tokens equal
    those of the same request on a fresh engine."""
    from sandyrt_b200.engine.llm import LLM
    from sandyrt_b200.weights.random_init import write_random_model

    ToyConfig = _register_toy()
    cfg = ToyConfig(width=32, vocab_size=90, decay=0.95)
    d = write_random_model(cfg, str(tmp_path / "toy"), seed=4, dtype=torch.float32)
    rng = np.random.default_rng(1)
    first, second = rng.integers(0, 90, size=19).tolist(), rng.integers(0, 90, size=7).tolist()
    llm = LLM(d, dtype="float32", cache_tokens=256, page_size=8, max_live=1)
    both = llm.generate([first, second], max_tokens=10)
    alone = LLM(d, dtype="float32", cache_tokens=256, page_size=8, max_live=1).generate(second, max_tokens=10)
    assert both[1].output_ids == alone[0].output_ids
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    ids = list(second)
    for tok in both[1].output_ids:
        assert tok == int(np.argmax(_toy_plain_logits(w, ids, 0.95, 32)[-1]))
        ids.append(tok)


# ---- a position encoding that acts on queries and keys ----------------------------------------
def _register_rotary():
    """Registers, from outside the framework, a position encoding that turns pairs of query and
    key channels by an angle that grows with the position, and a two-layer architecture using
    it.  The attention part then cannot let its projection write keys into the pages (they are
    turned first): it rotates, appends with the separate key/value write, and attends."""
    from sandyrt_b200.config.base import ModelConfig
    from sandyrt_b200.models.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
    from sandyrt_b200.parts.base import PositionEncoding
    from sandyrt_b200.registry import register_architecture, register_part

    class ToyRotary(PositionEncoding):
        rotates = True
        graph_safe = False
        max_positions = None

        def __init__(self, spec):
            super().__init__(spec)
            self.head_dim, self.base = int(self.params["head_dim"]), float(self.params["base"])

        def _turn(self, ctx, t):
            T, D = t.shape[0], self.head_dim
            x = t.float().reshape(T, -1, D // 2, 2)
            freq = self.base ** (-torch.arange(D // 2, device=t.device, dtype=torch.float32) / (D // 2))
            ang = ctx.positions.to(torch.float32)[:, None, None] * freq[None, None, :]
            c, s = torch.cos(ang), torch.sin(ang)
            y = torch.stack((x[..., 0] * c - x[..., 1] * s, x[..., 0] * s + x[..., 1] * c), dim=-1)
            t.copy_(y.reshape(T, -1).to(t.dtype))

        def rotate(self, ctx, q, k):
            self._turn(ctx, q)
            if k is not None:
                self._turn(ctx, k)

    @dataclasses.dataclass(frozen=True)
    class RotaryConfig(ModelConfig):
        architecture = "ToyRotaryModel"
        width: int = 0
        vocab_size: int = 0
        n_heads: int = 0
        base: float = 100.0

        @classmethod
        def from_dict(cls, raw):
            return cls(width=raw["width"], vocab_size=raw["vocab_size"], n_heads=raw["n_heads"], base=raw["base"])

        def to_dict(self):
            return {"architectures": [self.architecture], "width": self.width, "vocab_size": self.vocab_size,
                    "n_heads": self.n_heads, "base": self.base}

        def validate(self):
            assert (self.width // self.n_heads) % 16 == 0

    def describe(cfg):
        E, H = cfg.width, cfg.n_heads
        D = E // H
        norm = lambda n: PartSpec("layernorm", {"width": E, "eps": 1e-5}, {"weight": n + ".g", "bias": n + ".b"})
        layers = []
        for i in range(2):
            p = f"l{i}."
            layers.append(LayerSpec(
                "pre_norm",
                PartSpec("causal_attention", {"width": E, "n_heads": H, "n_kv_heads": H, "head_dim": D,
                                              "scale": 1 / math.sqrt(D), "weight_layout": "out_in"},
                         {"qkv.weight": p + "qkv.w", "qkv.bias": p + "qkv.b", "out.weight": p + "o.w",
                          "out.bias": p + "o.b"}),
                PartSpec("dense_mlp", {"width": E, "inner": 2 * E, "activation": "gelu", "weight_layout": "out_in"},
                         {"up.weight": p + "up.w", "up.bias": p + "up.b", "down.weight": p + "dn.w",
                          "down.bias": p + "dn.b"}),
                {"mixer": norm(p + "n1"), "feed_forward": norm(p + "n2")}))
        return ModelSpec(architecture=cfg.architecture, width=E, vocab_size=cfg.vocab_size, max_positions=None,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": E}, {"weight": "emb"}),
                         position=PartSpec("toy_rotary", {"head_dim": D, "base": cfg.base}, {}),
                         layers=layers, schedule=[LayerCall(0, 0), LayerCall(1, 1)], final_norm=norm("nf"),
                         head=PartSpec("output_head", {"vocab_size": cfg.vocab_size, "width": E, "tied": True}, {}))

    register_part("position", "toy_rotary", ToyRotary)
    register_architecture("ToyRotaryModel", RotaryConfig, describe)
    return RotaryConfig


def _rotary_plain_logits(w, ids, E, H, base, rnd):
    T, D = len(ids), E // H
    x = plain.embedding(ids, w["emb"])
    ln = lambda x, n: plain.layer_norm(x, w[n + ".g"], w[n + ".b"], 1e-5)
    lin = lambda h, p: plain.linear_in_out(h, rnd(w[p + "w"]).T, rnd(w[p + "b"]))
    freq = base ** (-np.arange(D // 2, dtype=np.float32) / (D // 2))
    ang = np.arange(T, dtype=np.float32)[:, None, None] * freq[None, None, :]
    c, s = np.cos(ang), np.sin(ang)

    def turn(t):
        v = t.reshape(T, H, D // 2, 2)
        return np.stack((v[..., 0] * c - v[..., 1] * s, v[..., 0] * s + v[..., 1] * c), axis=-1).reshape(T, E)

    split = lambda t: t.reshape(T, H, D).transpose(1, 0, 2)
    for i in range(2):
        p = f"l{i}."
        qkv = rnd(lin(rnd(ln(x, p + "n1")), p + "qkv."))
        q, k, v = rnd(turn(qkv[:, :E])), rnd(turn(qkv[:, E:2 * E])), qkv[:, 2 * E:]
        o = plain.causal_attention(split(q), split(k), split(v), 1 / math.sqrt(D)).transpose(1, 0, 2).reshape(T, E)
        x = x + lin(rnd(o), p + "o.")
        x = x + lin(rnd(plain.gelu_erf(lin(rnd(ln(x, p + "n2")), p + "up."))), p + "dn.")
    return rnd(ln(x, "nf")) @ rnd(w["emb"]).T


@pytest.mark.parametrize("dtype,atol,rtol", [("float32", 3e-5, 1e-4), ("bfloat16", 6e-3, 2e-2)])
def test_position_encoding_that_rotates_queries_and_keys(tmp_path, dtype, atol, rtol):
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model
    from sandyrt_b200.weights.random_init import write_random_model

    RotaryConfig = _register_rotary()
    cfg = RotaryConfig(width=96, vocab_size=130, n_heads=3, base=50.0)
    d = write_random_model(cfg, str(tmp_path / "rot"), seed=6, dtype=torch.float32)
    model = load_model(d, device=DEV, dtype=getattr(torch, dtype))
    assert model.max_positions is None and not model.graph_safe
    eng = Engine(model, max_tokens=256, page_size=8, max_requests=2)
    eng.cache.device_caches.poison()
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    ids = np.random.default_rng(2).integers(0, 130, size=45).tolist()
    rnd = plain.round_bf16 if dtype == "bfloat16" else (lambda a: a)
    want = _rotary_plain_logits(w, ids, 96, 3, 50.0, rnd)
    for cuts in ([45], [20, 2, 1, 1, 21], [1] * 6 + [39]):
        rows, pos = [], 0
        for n in cuts:
            rows.append(eng.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
            pos += n
        eng.release("r")
        np.testing.assert_allclose(np.concatenate(rows), want, atol=atol, rtol=rtol, err_msg=f"cuts {cuts}")
    eng.check_status()


# ---- a feed-forward with routing, and a norm of another kind -----------------------------------
def _register_routed():
    """Registers, from outside the framework: a feed-forward that sends every token to the best
    `top` of its experts (router logits and their softmax in float32; an expert is two small
    matrices with a squared ReLU between), a norm without a mean (root mean square, one gain), and
    an architecture whose layers differ: the first has the routed feed-forward, the second the
    library's dense one, and both use the toy norm in front of the feed-forward only."""
    from sandyrt_b200.config.base import ModelConfig
    from sandyrt_b200.models.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
    from sandyrt_b200.parts.base import FeedForward, Norm
    from sandyrt_b200.registry import register_architecture, register_part
    from sandyrt_b200.weights.loader import TensorRequest

    class RoutedFF(FeedForward):
        graph_safe = False        # the number of tokens an expert gets is read on the host

        def __init__(self, spec):
            super().__init__(spec)
            p = self.params
            self.width, self.inner, self.n, self.top = int(p["width"]), int(p["inner"]), int(p["experts"]), int(p["top"])

        def requests(self):
            E, I, n = self.width, self.inner, self.n
            return {"router": TensorRequest((n, E)), "up": TensorRequest((n, I, E)), "down": TensorRequest((n, E, I))}

        def bind(self, tensors, device, dtype):
            self.router = tensors["router"].to(device=device, dtype=torch.float32)       # routing stays in float32
            self.up = tensors["up"].to(device=device, dtype=dtype)
            self.down = tensors["down"].to(device=device, dtype=dtype)

        def forward(self, ctx, h, x):
            logits = h.float() @ self.router.T
            best, which = torch.topk(logits, self.top, dim=-1)
            gate = torch.softmax(best, dim=-1)                                            # over the chosen experts only
            for e in range(self.n):
                tok, k = torch.nonzero(which == e, as_tuple=True)
                if tok.numel() == 0:
                    continue
                a = torch.relu(h[tok] @ self.up[e].T) ** 2
                x.index_add_(0, tok, (a.to(h.dtype) @ self.down[e].T).float() * gate[tok, k][:, None])

    class RmsNorm(Norm):
        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.eps = int(self.params["width"]), float(self.params["eps"])

        def requests(self):
            return {"gain": TensorRequest((self.width,), init="gamma")}

        def bind(self, tensors, device, dtype):
            self.gain = tensors["gain"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, x, out, rows=None):
            src = x if rows is None else x[rows.long()]
            y = src * torch.rsqrt((src * src).mean(dim=-1, keepdim=True) + self.eps) * self.gain
            out.copy_(y.to(out.dtype))

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architecture = "ToyRoutedModel"
        width: int = 0
        vocab_size: int = 0
        experts: int = 0
        top: int = 1
        eps: float = 1e-6

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: raw[k] for k in ("width", "vocab_size", "experts", "top", "eps")})

        def to_dict(self):
            return {"architectures": [self.architecture], "width": self.width, "vocab_size": self.vocab_size,
                    "experts": self.experts, "top": self.top, "eps": self.eps}

        def validate(self):
            assert self.width % 16 == 0 and 1 <= self.top <= self.experts

    def describe(cfg):
        E = cfg.width
        ln = lambda n: PartSpec("layernorm", {"width": E, "eps": 1e-5}, {"weight": n + ".g", "bias": n + ".b"})
        rms = lambda n: PartSpec("toy_rms", {"width": E, "eps": cfg.eps}, {"gain": n + ".gain"})
        attn = lambda p: PartSpec("causal_attention", {"width": E, "n_heads": 3, "n_kv_heads": 3, "head_dim": E // 3,
                                                       "scale": 1 / math.sqrt(E // 3), "weight_layout": "out_in"},
                                  {"qkv.weight": p + "qkv.w", "qkv.bias": p + "qkv.b", "out.weight": p + "o.w",
                                   "out.bias": p + "o.b"})
        layers = [
            LayerSpec("pre_norm", attn("l0."),
                      PartSpec("toy_routed", {"width": E, "inner": E + 16, "experts": cfg.experts, "top": cfg.top},
                               {"router": "l0.router", "up": "l0.up", "down": "l0.down"}),
                      {"mixer": ln("l0.n1"), "feed_forward": rms("l0.n2")}),
            LayerSpec("pre_norm", attn("l1."),
                      PartSpec("dense_mlp", {"width": E, "inner": 2 * E, "activation": "gelu_new", "weight_layout": "out_in"},
                               {"up.weight": "l1.up.w", "up.bias": "l1.up.b", "down.weight": "l1.dn.w", "down.bias": "l1.dn.b"}),
                      {"mixer": ln("l1.n1"), "feed_forward": rms("l1.n2")}),
        ]
        return ModelSpec(architecture=cfg.architecture, width=E, vocab_size=cfg.vocab_size, max_positions=None,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": E}, {"weight": "emb"}),
                         position=PartSpec("none", {}, {}), layers=layers, schedule=[LayerCall(0, 0), LayerCall(1, 1)],
                         final_norm=rms("nf"), head=PartSpec("output_head", {"vocab_size": cfg.vocab_size, "width": E,
                                                                             "tied": True}, {}))

    register_part("feed_forward", "toy_routed", RoutedFF)
    register_part("norm", "toy_rms", RmsNorm)
    register_architecture("ToyRoutedModel", RoutedConfig, describe)
    return RoutedConfig


def _routed_plain_logits(w, ids, E, top, eps):
    """The routed toy model, whole sequence, token by token where the routing is."""
    T, D = len(ids), E // 3
    x = plain.embedding(ids, w["emb"])
    ln = lambda x, n: plain.layer_norm(x, w[n + ".g"], w[n + ".b"], 1e-5)
    rms = lambda x, n: x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w[n + ".gain"]
    lin = lambda h, p: plain.linear_in_out(h, w[p + "w"].T, w[p + "b"])
    split = lambda t: t.reshape(T, 3, D).transpose(1, 0, 2)

    def attn(x, p):
        qkv = lin(ln(x, p + "n1"), p + "qkv.")
        o = plain.causal_attention(split(qkv[:, :E]), split(qkv[:, E:2 * E]), split(qkv[:, 2 * E:]), 1 / math.sqrt(D))
        return x + lin(o.transpose(1, 0, 2).reshape(T, E), p + "o.")

    x = attn(x, "l0.")
    h = rms(x, "l0.n2")
    chosen = []
    for t in range(T):
        logits = w["l0.router"] @ h[t]
        order = np.argsort(-logits)[:top]
        g = np.exp(logits[order] - logits[order].max()); g /= g.sum()
        chosen.append(tuple(int(e) for e in order))
        for e, ge in zip(order, g):
            x[t] += ge * (w["l0.down"][e] @ (np.maximum(w["l0.up"][e] @ h[t], 0) ** 2))
    x = attn(x, "l1.")
    x = x + lin(plain.gelu_new(lin(rms(x, "l1.n2"), "l1.up.")), "l1.dn.")
    return rms(x, "nf") @ w["emb"].T, chosen


@pytest.mark.parametrize("top", [1, 2])
def test_feed_forward_with_routing_and_a_norm_of_another_kind(tmp_path, top):
    """A feed-forward that routes and a norm the library does not have, defined here, are
    registered, built from config.json and stepped in mixed batches; the layers of the model
    differ in their feed-forward.  Every expert is used, or the test would not see a wrong one."""
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model
    from sandyrt_b200.weights.random_init import write_random_model

    RoutedConfig = _register_routed()
    cfg = RoutedConfig(width=48, vocab_size=75, experts=3, top=top, eps=1e-4)
    d = write_random_model(cfg, str(tmp_path / "routed"), seed=8, dtype=torch.float32)
    model = load_model(d, device=DEV, dtype=torch.float32)
    assert not model.graph_safe
    eng = Engine(model, max_tokens=128, page_size=8, max_requests=2)
    eng.cache.device_caches.poison()
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    rng = np.random.default_rng(5)
    seqs = {name: rng.integers(0, 75, size=n).tolist() for name, n in (("a", 29), ("b", 12), ("c", 21))}
    want, used = {}, set()
    for k, ids in seqs.items():
        want[k], chosen = _routed_plain_logits(w, ids, 48, top, 1e-4)
        used.update(e for c in chosen for e in c)
    assert used == {0, 1, 2}
    plan = [[("a", 11), ("b", 2)], [("a", 1), ("b", 10)], [("a", 1), ("c", 5)], [("c", 16), ("a", 16)]]
    got, fed = {k: [] for k in seqs}, {k: 0 for k in seqs}
    for step in plan:
        out = eng.step([StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in step]).cpu().numpy()
        r = 0
        for k, n in step:
            got[k].append(out[r:r + n].copy()); r += n; fed[k] += n
            if fed[k] == len(seqs[k]):
                eng.release(k)
        eng.cache.alloc.check()
    for k in seqs:
        np.testing.assert_allclose(np.concatenate(got[k]), want[k], atol=5e-5, rtol=1e-4, err_msg=f"sequence {k}")
    eng.check_status()
