"""Generality of the layer assembly, shown with toy parts that live in this file:

* a mixer with a state of its own (a decaying sum per sequence) is registered,
  put into a model next to attention layers, built, loaded and stepped — prompt,
  decode, captured decode, batches, slot reuse — without touching the package;
* a run order that names a layer twice and lets a layer read another layer's
  cache;
* a feed-forward with routing (one expert of several per token, chosen by
  float32 router logits) and a position encoding that the fused kernel does not
  know (rotation of neighbouring pairs with positions divided by a factor), in
  different layers of one model.

The toys use torch operations; they are test fixtures, not models."""
import dataclasses
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from wick_b200.parts.base import CacheNeed, FeedForward, Mixer, Position, TensorSpec, register_part  # noqa: E402
from helpers import CONFIG_A, CONFIG_B, assert_logits_close, random_tokens, tmp_root  # noqa: E402
from plain import qwen3_plain as P  # noqa: E402


class DecayMixer(Mixer):
    """state <- decay * state + x_t ;  out_t = state W^T.  One float32 record of
    ``width`` numbers per sequence, kept in the cache's fixed-size state store."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.decay = int(params["width"]), float(params["decay"])
        self.w = None

    def tensor_specs(self):
        return [TensorSpec("mix.weight", (self.width, self.width))]

    def load(self, fetch):
        self.w = self.ctx.hold(fetch("mix.weight"), "matrix")

    def cache_need(self):
        return CacheNeed("state", shape=(self.width,), dtype=torch.float32)

    def forward(self, x, batch, cache, write_cache):
        slots = batch.slots.long()
        xf = x.float()
        if batch.is_decode:                                   # device tensors only: safe inside a captured step
            s = cache.state[slots] * self.decay + xf
            cache.state.index_copy_(0, slots, s)
            states = s
        else:
            rows, t0 = [], 0
            for b, n in enumerate(batch.q_lens):
                s = cache.state[slots[b]].clone()
                for t in range(n):
                    s = s * self.decay + xf[t0 + t]
                    rows.append(s)
                cache.state[slots[b]] = s
                t0 += n
            states = torch.stack(rows)
        return (states.to(self.ctx.dtype).float() @ self.w.float().T).unsqueeze(0)


register_part("mixer", "toy_decay", DecayMixer)


@dataclasses.dataclass(frozen=True)
class ToyConfig(wick.Qwen3Config):
    decay: float = 0.5

    @classmethod
    def from_json(cls, j, architecture="ToyMixForCausalLM"):
        base = wick.Qwen3Config.from_json(j, architecture)
        return cls(**{**base.__dict__, "decay": float(j.get("toy_decay", 0.5))})

    def to_json(self):
        return {**super().to_json(), "architectures": [self.architecture], "toy_decay": self.decay}


def build_toy_spec(cfg: ToyConfig):
    spec = wick.get_architecture("qwen3").build_spec(cfg)
    layers = list(spec.layers)
    for i in range(1, len(layers), 2):                         # odd layers get the toy mixer
        layers[i] = dataclasses.replace(
            layers[i], mixer=wick.PartSpec("toy_decay", {"width": cfg.hidden_size, "decay": cfg.decay}),
            names={**layers[i].names, "mixer": "toy."})
    return dataclasses.replace(spec, layers=tuple(layers))


def build_looped_spec(cfg):
    spec = wick.get_architecture("qwen3").build_spec(cfg)
    E = wick.ScheduleEntry
    return dataclasses.replace(spec, schedule=(E(0), E(1), E(1), E(0, read_cache_of=0)))


wick.register_architecture(wick.Architecture(("ToyMixForCausalLM",), ToyConfig, build_toy_spec))
wick.register_architecture(wick.Architecture(("LoopedForCausalLM",), wick.Qwen3Config, build_looped_spec))


def plain_toy_forward(cfg, w, tokens, decay):
    toks = torch.as_tensor(tokens)
    T = len(tokens)
    x = w["model.embed_tokens.weight"][toks]
    for layer in range(cfg["layers"]):
        p = f"model.layers.{layer}."
        xn = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if layer % 2 == 1:
            s, rows = torch.zeros(cfg["hidden"]), []
            for t in range(T):
                s = s * decay + xn[t]
                rows.append(s)
            d = torch.stack(rows) @ w[p + "toy.mix.weight"].T
        else:
            d, _ = P.attention_block(xn, w, p, cfg, torch.arange(T))
        x = x + d
        xn = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + P.swiglu(xn, w, p)
    xn = P.rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return xn @ head.T


@pytest.mark.parametrize("graphs", [False, True])
def test_a_mixer_with_its_own_state_is_registered_built_and_stepped(graphs):
    cfgj = dict(CONFIG_B, architectures=["ToyMixForCausalLM"], toy_decay=0.75, num_hidden_layers=4)
    cfg = wick.config_from_json(cfgj)
    assert isinstance(cfg, ToyConfig) and cfg.decay == 0.75
    d = os.path.join(tmp_root(), "toy-mix")
    wick.write_random_model(cfg, 5, d, dtype=torch.float32)
    assert wick.load_config(d) == cfg
    eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=512, use_graphs=graphs)
    kinds = [g.need.kind for g in eng.cache.groups]
    assert sorted(kinds) == ["paged_kv", "state"] and all(len(g.entries) == 2 for g in eng.cache.groups)
    assert not eng.prompt_graphs            # (the toy mixer walks the host's lists of lengths: its prompt steps are never captured)
    table = eng.model.tensor_table()
    assert "model.layers.1.toy.mix.weight" in table and "model.layers.1.self_attn.q_proj.weight" not in table
    pc, pw = P.read_model_dir(d)
    seqs = [random_tokens(1000, n, 400 + n) for n in (9, 30, 4)]
    refs = [plain_toy_forward(pc, pw, s, 0.75) for s in seqs]
    for rnd in range(2):                                       # the second round reuses the slots: state must restart
        slots = [eng.open_seq() for _ in seqs]
        got = eng.step(slots, [s[:-3] for s in seqs], [list(range(len(s) - 3)) for s in seqs]).clone()
        off = 0
        for s, r in zip(seqs, refs):
            assert_logits_close(got[off:off + len(s) - 3], r[:len(s) - 3], "float32", f"toy prompt round {rnd}")
            off += len(s) - 3
        for k in range(3, 0, -1):
            got = eng.step(slots, [[s[-k]] for s in seqs]).clone()
            for i, (s, r) in enumerate(zip(seqs, refs)):
                assert_logits_close(got[i], r[len(s) - k], "float32", f"toy decode round {rnd}")
        for sl in slots:
            eng.close_seq(sl)
    out = wick.generate(eng, [seqs[0]], wick.GenOptions(max_tokens=3, sampler=wick.SamplerConfig.greedy()))
    assert len(out[0].tokens) == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_named_twice_and_a_layer_reading_anothers_cache(dtype):
    cfg = wick.config_from_json(dict(CONFIG_A, architectures=["LoopedForCausalLM"]))
    d = os.path.join(tmp_root(), "toy-loop")
    wick.write_random_model(cfg, 6, d)
    eng = wick.Engine.from_dir(d, dtype=dtype, max_tokens=512)
    assert len(eng.model.blocks) == 2 and len(eng.spec.schedule) == 4
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [0, 1, 2], \
        "three entries own a cache, the fourth reads the first one's"
    pc, pw = P.read_model_dir(d)
    toks = random_tokens(512, 80, 77)
    ref = P.forward(pc, pw, toks, schedule=[(0, None), (1, None), (1, None), (0, 0)])
    s = eng.open_seq()
    got = [eng.step([s], [toks[:70]], [list(range(70))]).clone()]
    got += [eng.step([s], [[t]]).clone() for t in toks[70:]]
    assert_logits_close(torch.cat(got), ref, dtype, "looped schedule")
    assert eng.model.weight_bytes_per_step() > 0


# ---------------------------------------------------------------------------
class RoutedExperts(FeedForward):
    """Each token goes to the one expert with the largest router logit (the first
    of equals); out = logit-softmax weight of that expert * W2 relu(W1 x)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.inner, self.experts = int(params["width"]), int(params["inner"]), int(params["experts"])

    def tensor_specs(self):
        specs = [TensorSpec("router.weight", (self.experts, self.width))]
        for e in range(self.experts):
            specs += [TensorSpec(f"experts.{e}.w1.weight", (self.inner, self.width)),
                      TensorSpec(f"experts.{e}.w2.weight", (self.width, self.inner))]
        return specs

    def load(self, fetch):
        self.router = self.ctx.hold(fetch("router.weight"), "matrix")
        self.w1 = torch.stack([self.ctx.hold(fetch(f"experts.{e}.w1.weight"), "matrix") for e in range(self.experts)])
        self.w2 = torch.stack([self.ctx.hold(fetch(f"experts.{e}.w2.weight"), "matrix") for e in range(self.experts)])

    def forward(self, x, batch):
        xf = x.float()
        logits = xf @ self.router.float().T                                  # router logits in float32
        probs = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        gate = probs.gather(1, choice[:, None])
        h = torch.relu(torch.bmm(self.w1.float()[choice], xf[:, :, None]))    # [n, inner, 1]
        y = torch.bmm(self.w2.float()[choice], h)[:, :, 0] * gate
        return y.unsqueeze(0)


class NeighbourPairRotary(Position):
    """Pairs (2i, 2i+1) of every head rotated by (position / factor) * theta^(-2i/d)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        d = int(params["head_dim"])
        self.factor = float(params["factor"])
        self.inv_freq = torch.tensor([float(params["theta"]) ** (-2.0 * i / d) for i in range(d // 2)],
                                     dtype=torch.float32, device=ctx.device)

    def apply(self, q, k, positions):
        angle = (positions.float() / self.factor)[:, None] * self.inv_freq[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        for t in (q, k):
            a, b = t[..., 0::2].clone(), t[..., 1::2].clone()
            t[..., 0::2] = a * cos - b * sin
            t[..., 1::2] = b * cos + a * sin


register_part("ffn", "toy_routed", RoutedExperts)
register_part("position", "toy_neighbour_pairs", NeighbourPairRotary)

TOY_EXPERTS, TOY_INNER, TOY_FACTOR = 3, 40, 4.0


def build_routed_spec(cfg):
    spec = wick.get_architecture("qwen3").build_spec(cfg)
    layers = list(spec.layers)
    pos = wick.PartSpec("toy_neighbour_pairs", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "factor": TOY_FACTOR})
    for i in range(len(layers)):
        L = layers[i]
        if i % 2 == 0:                                         # even layers: the other position encoding
            L = dataclasses.replace(L, mixer=wick.PartSpec(L.mixer.kind, {**L.mixer.params, "position": pos}))
        else:                                                  # odd layers: the routed feed-forward
            L = dataclasses.replace(
                L, ffn=wick.PartSpec("toy_routed", {"width": cfg.hidden_size, "inner": TOY_INNER, "experts": TOY_EXPERTS}),
                names={**L.names, "ffn": "moe."})
        layers[i] = L
    return dataclasses.replace(spec, layers=tuple(layers))


wick.register_architecture(wick.Architecture(("ToyRoutedForCausalLM",), wick.Qwen3Config, build_routed_spec))


def plain_routed_forward(cfg, w, tokens):
    toks = torch.as_tensor(tokens)
    T = len(tokens)
    H, KV, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    x = w["model.embed_tokens.weight"][toks]
    pos = torch.arange(T)
    for layer in range(cfg["layers"]):
        p = f"model.layers.{layer}."
        xn = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if layer % 2 == 0:
            q = P.rms_norm((xn @ w[p + "self_attn.q_proj.weight"].T).view(T, H, D), w[p + "self_attn.q_norm.weight"], cfg["eps"])
            k = P.rms_norm((xn @ w[p + "self_attn.k_proj.weight"].T).view(T, KV, D), w[p + "self_attn.k_norm.weight"], cfg["eps"])
            v = (xn @ w[p + "self_attn.v_proj.weight"].T).view(T, KV, D)
            inv = torch.tensor([cfg["theta"] ** (-2.0 * i / D) for i in range(D // 2)], dtype=torch.float32)
            ang = (pos.float() / TOY_FACTOR)[:, None] * inv[None, :]
            c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

            def rot(t):
                a, b = t[..., 0::2], t[..., 1::2]
                return torch.stack([a * c - b * s_, b * c + a * s_], dim=-1).reshape(t.shape)
            d = P.causal_attention(rot(q), rot(k), v).reshape(T, H * D) @ w[p + "self_attn.o_proj.weight"].T
        else:
            d, _ = P.attention_block(xn, w, p, cfg, pos)
        x = x + d
        xn = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        if layer % 2 == 1:
            logits = xn @ w[p + "moe.router.weight"].T
            rows = []
            for t in range(T):
                e = int(P.argmax_first(logits[t]))
                g = P.softmax_rows(logits[t:t + 1])[0, e]
                h = torch.relu(w[p + f"moe.experts.{e}.w1.weight"] @ xn[t])
                rows.append((w[p + f"moe.experts.{e}.w2.weight"] @ h) * g)
            x = x + torch.stack(rows)
        else:
            x = x + P.swiglu(xn, w, p)
    xn = P.rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return xn @ head.T


@pytest.mark.parametrize("graphs", [False, True])
def test_a_routed_feed_forward_and_another_position_encoding(graphs):
    cfg = wick.config_from_json(dict(CONFIG_B, architectures=["ToyRoutedForCausalLM"], num_hidden_layers=4))
    d = os.path.join(tmp_root(), "toy-routed")
    wick.write_random_model(cfg, 11, d, dtype=torch.float32, std=0.08)
    eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=512, use_graphs=graphs)
    table = eng.model.tensor_table()
    assert "model.layers.1.moe.experts.2.w2.weight" in table and "model.layers.1.mlp.gate_proj.weight" not in table
    assert "model.layers.0.mlp.gate_proj.weight" in table
    pc, pw = P.read_model_dir(d)
    seqs = [random_tokens(1000, n, 900 + n) for n in (70, 13, 5)]
    refs = [plain_routed_forward(pc, pw, s) for s in seqs]
    used = set()
    for s in seqs:                                             # the router does choose: more than one expert is in use
        x = pw["model.embed_tokens.weight"][torch.as_tensor(s)]
        used |= set((x @ pw["model.layers.1.moe.router.weight"].T).argmax(-1).tolist())
    assert len(used) > 1
    slots = [eng.open_seq() for _ in seqs]
    got = eng.step(slots, [s[:-4] for s in seqs], [list(range(len(s) - 4)) for s in seqs]).clone()
    off = 0
    for s, r in zip(seqs, refs):
        assert_logits_close(got[off:off + len(s) - 4], r[:len(s) - 4], "float32", "routed prompt")
        off += len(s) - 4
    for k in range(4, 0, -1):
        got = eng.step(slots, [[s[-k]] for s in seqs]).clone()
        for i, (s, r) in enumerate(zip(seqs, refs)):
            assert_logits_close(got[i], r[len(s) - k], "float32", "routed decode")
    for sl in slots:
        eng.close_seq(sl)


# ---------------------------------------------------------------------------
# A mixer that reads only the last few positions, with a kind of cache storage of its own:
# both are registered here; the package's files know nothing of either.
from wick_b200.cache import CacheView, Storage, register_storage  # noqa: E402


class LastRows(Storage):
    """[entries, slots, window, width] float32: row ``position % window`` of a sequence's
    slot holds what the mixer stored for that position."""
    kind = "toy_last_rows"

    def shape(self):
        return (self.n_entries, self.n_slots, self.need.window) + tuple(self.need.shape)

    def view(self, idx, batch):
        return CacheView(rows=self.tensor[idx], slots=batch.slots, window=self.need.window)

    def open_seq(self, slot):
        self.tensor[:, slot] = float("nan")                   # nothing stored yet: a read of it must show

    def read_bytes(self, cached_tokens, n_seqs):
        n = self.element_size() * self.need.window
        for d in self.need.shape:
            n *= d
        return n_seqs * self.n_entries * n


register_storage("toy_last_rows", LastRows)


class WindowMean(Mixer):
    """out_t = W mean(x_s for s in the last ``window`` positions up to t)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.window = int(params["width"]), int(params["window"])

    def tensor_specs(self):
        return [TensorSpec("mix.weight", (self.width, self.width))]

    def load(self, fetch):
        self.w = self.ctx.hold(fetch("mix.weight"), "matrix")

    def cache_need(self):
        return CacheNeed("toy_last_rows", window=self.window, shape=(self.width,), dtype=torch.float32)

    def forward(self, x, batch, cache, write_cache):
        W = self.window
        xf = x.float()
        slots = cache.slots.long()
        if batch.is_decode:                                   # device tensors only: safe inside a captured step
            pos = batch.positions.long()
            cache.rows[slots, pos % W] = xf
            have = torch.clamp(pos + 1, max=W)                # positions stored so far, at most the window
            keep = (torch.arange(W, device=x.device)[None, :] < have[:, None])
            # rows of the ring that hold one of the last `have` positions: all of them once the
            # ring is full, rows 0..pos before
            rows = torch.where(keep[:, :, None], cache.rows[slots], torch.zeros((), device=x.device))
            means = rows.sum(1) / have[:, None].float()
        else:
            out, t0 = [], 0
            for b, n in enumerate(batch.q_lens):
                start = batch.starts[b]
                for t in range(n):
                    p = start + t
                    cache.rows[slots[b], p % W] = xf[t0 + t]
                    have = min(p + 1, W)
                    idx = torch.tensor([(p - i) % W for i in range(have)], device=x.device)
                    out.append(cache.rows[slots[b]][idx].sum(0) / have)
                t0 += n
            means = torch.stack(out)
        return (means.to(self.ctx.dtype).float() @ self.w.float().T).unsqueeze(0)


register_part("mixer", "toy_window_mean", WindowMean)


def build_window_spec(cfg):
    spec = wick.get_architecture("qwen3").build_spec(cfg)
    layers = list(spec.layers)
    layers[1] = dataclasses.replace(layers[1], mixer=wick.PartSpec("toy_window_mean", {"width": cfg.hidden_size, "window": 5}),
                                    names={**layers[1].names, "mixer": "win."})
    return dataclasses.replace(spec, layers=tuple(layers))


wick.register_architecture(wick.Architecture(("ToyWindowForCausalLM",), wick.Qwen3Config, build_window_spec))


def plain_window_forward(cfg, w, tokens, window):
    toks = torch.as_tensor(tokens)
    T = len(tokens)
    x = w["model.embed_tokens.weight"][toks]
    for layer in range(cfg["layers"]):
        p = f"model.layers.{layer}."
        xn = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if layer == 1:
            d = torch.stack([xn[max(0, t - window + 1):t + 1].mean(0) for t in range(T)]) @ w[p + "win.mix.weight"].T
        else:
            d, _ = P.attention_block(xn, w, p, cfg, torch.arange(T))
        x = x + d
        xn = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + P.swiglu(xn, w, p)
    xn = P.rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return xn @ head.T


@pytest.mark.parametrize("graphs", [False, True])
def test_a_windowed_mixer_with_a_storage_kind_of_its_own(graphs):
    """One layer keeps the last five positions in a ring per sequence (a storage class registered
    in this file), the others all keys in pages: groups of layers with different needs, each with
    storage of its own.  Prompts shorter and longer than the window, decoding across the ring's
    wrap, slots used again (a new sequence must not see the last one's rows)."""
    cfg = wick.config_from_json(dict(CONFIG_B, architectures=["ToyWindowForCausalLM"]))
    d = os.path.join(tmp_root(), "toy-window")
    wick.write_random_model(cfg, 8, d, dtype=torch.float32)
    eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=512, use_graphs=graphs)
    assert [g.need.kind for g in eng.cache.groups] == ["paged_kv", "toy_last_rows"]
    assert [len(g.entries) for g in eng.cache.groups] == [2, 1]
    assert eng.cache.groups[1].storage.shape[2:] == (5, 96)
    # what a decode step reads: pages by position, the ring by sequence
    assert eng.cache.read_bytes(100, 2) == 100 * eng.cache.bytes_per_token() + 2 * 5 * 96 * 4
    pc, pw = P.read_model_dir(d)
    seqs = [random_tokens(1000, n, 600 + n) for n in (3, 12, 7)]
    refs = [plain_window_forward(pc, pw, s + random_tokens(1000, 9, 700 + len(s)), 5) for s in seqs]
    full = [s + random_tokens(1000, 9, 700 + len(s)) for s in seqs]
    for rnd in range(2):
        slots = [eng.open_seq() for _ in seqs]
        got = eng.step(slots, seqs, [list(range(len(s))) for s in seqs]).clone()
        off = 0
        for s, r in zip(seqs, refs):
            assert_logits_close(got[off:off + len(s)], r[:len(s)], "float32", f"window prompt round {rnd}")
            off += len(s)
        for k in range(9):
            got = eng.step(slots, [[f[len(s) + k]] for s, f in zip(seqs, full)]).clone()
            for i, (s, r) in enumerate(zip(seqs, refs)):
                assert_logits_close(got[i], r[len(s) + k], "float32", f"window decode {k} round {rnd}")
        for sl in slots:
            eng.close_seq(sl)
