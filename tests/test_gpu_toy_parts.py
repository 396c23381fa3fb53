"""Generality of the layer assembly, shown with toy parts that live in this file:

* a mixer with a state of its own (a decaying sum per sequence) is registered,
  put into a model next to attention layers, built, loaded and stepped — prompt,
  decode, captured decode, batches, slot reuse — without touching the package;
* a run order that names a layer twice and lets a layer read another layer's
  cache.

The toys use torch operations; they are test fixtures, not models."""
import dataclasses
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from wick_b200.parts.base import CacheNeed, Mixer, TensorSpec, register_part  # noqa: E402
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
