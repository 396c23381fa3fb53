"""A plain, slow implementation of the Qwen3 dense decoder, the tests' oracle.

It rests on the formulas of pMag11-alt/wick's Rust sources (each function cites
the file and lines it restates).  wick cannot be compiled here (no Rust
toolchain) and has no importable module, so this file is not checked against
wick's own binary; it IS checked, in ``tests/test_plain_anchor.py``, against the
logits that wick's repository records for its tiny Qwen3 fixture
(``tests/fixtures/tiny/qwen3-qknorm-f32/expected.json``, made with transformers
by wick's ``scripts/make_tiny.py``), wherever that fixture can be read.

Whole sequences, no cache, one function per part, torch on the CPU.  It shares
no code with ``wick_b200``: it has its own safetensors reader, its own config
reading and its own sampler.  ``dtype`` may be float32 (the comparison that
counts) or float64 (to tell which of two float32 results is the closer one).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


# ---------------------------------------------------------------------------
# files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """safetensors.rs:81-119: u64 header length, JSON header, raw little-endian data."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = raw[base + b:base + e]
        dt = info["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif dt == "F16":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f2").copy()).float()
        elif dt == "BF16":
            # quant.rs:38-40: a bf16 is the upper half of an f32
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        else:
            raise ValueError(f"{name}: unsupported dtype {dt}")
        out[name] = t.reshape(info["shape"])
    return out


def read_model_dir(model_dir: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return plain_config(cfg), read_safetensors(os.path.join(model_dir, "model.safetensors"))


def plain_config(j: dict) -> dict:
    """config.rs:55-133, the keys the Qwen3 decoder uses."""
    heads = j["num_attention_heads"]
    rp = j.get("rope_parameters") or {}
    theta = j.get("rope_theta", rp.get("rope_theta", 10000.0))
    return dict(
        hidden=j["hidden_size"], heads=heads, kv_heads=j.get("num_key_value_heads", heads),
        head_dim=j.get("head_dim", j["hidden_size"] // heads), intermediate=j["intermediate_size"],
        layers=j["num_hidden_layers"], vocab=j["vocab_size"], eps=j.get("rms_norm_eps", 1e-6),
        theta=float(theta), tied=bool(j.get("tie_word_embeddings", False)))


# ---------------------------------------------------------------------------
# parts
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """kernels.rs:343-349: ss = mean(x^2); scale = 1/sqrt(ss+eps); (x*scale)*w, over the last axis."""
    ss = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(ss + torch.tensor(eps, dtype=x.dtype))
    return (x * scale) * w.to(x.dtype)


def rope_inv_freq(theta: float, head_dim: int) -> torch.Tensor:
    """config.rs:162-167: 1 / theta^(2i/d) in f64, then cast to f32."""
    return torch.tensor([1.0 / (float(theta) ** (2.0 * i / head_dim)) for i in range(head_dim // 2)],
                        dtype=torch.float64).to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """model.rs:404-414: pairs (i, i+half) of every head rotated by pos*inv_freq[i];
    the angle is a float32 product.  x: [T, heads, head_dim]."""
    half = x.shape[-1] // 2
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]           # f32, as `pos as f32 * inv_freq[i]`
    sin, cos = torch.sin(angle).to(x.dtype)[:, None, :], torch.cos(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """kernels.rs:360-371: subtract the max, exp, multiply by 1/sum."""
    m = s.max(-1, keepdim=True).values
    e = torch.exp(s - m)
    return e * (1.0 / e.sum(-1, keepdim=True))


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """model.rs:520-553: token i, head h reads kv head h / (heads/kv_heads) at
    positions 0..=i; score = (q.k)*scale with scale = 1/sqrt(head_dim); softmax;
    weighted sum of v.  q: [T, heads, d]; k, v: [T, kv_heads, d] -> [T, heads, d]."""
    T, H, D = q.shape
    group = H // k.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.empty_like(q)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    for h in range(H):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h, :] = softmax_rows(s) @ v[:, kh, :]
    return out


def attention_block(x, w, p, cfg, positions, kv_override=None):
    """model.rs:452-486: projections without bias, per-head norm of q and k
    (475-478), rotation (479-480), attention, output projection.  Returns the
    delta and the (k, v) it produced."""
    T = x.shape[0]
    H, KV, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    dt = x.dtype
    q = (x @ w[p + "self_attn.q_proj.weight"].to(dt).T).view(T, H, D)
    q = rms_norm(q, w[p + "self_attn.q_norm.weight"], cfg["eps"])
    inv = rope_inv_freq(cfg["theta"], D)
    q = rope(q, positions, inv)
    if kv_override is None:
        k = (x @ w[p + "self_attn.k_proj.weight"].to(dt).T).view(T, KV, D)
        v = (x @ w[p + "self_attn.v_proj.weight"].to(dt).T).view(T, KV, D)
        k = rms_norm(k, w[p + "self_attn.k_norm.weight"], cfg["eps"])
        k = rope(k, positions, inv)
    else:
        k, v = kv_override
    att = causal_attention(q, k, v).reshape(T, H * D)
    return att @ w[p + "self_attn.o_proj.weight"].to(dt).T, (k, v)


def swiglu(x, w, p):
    """model.rs:493-502 with kernels.rs:374-378: down( g/(1+exp(-g)) * u )."""
    dt = x.dtype
    g = x @ w[p + "mlp.gate_proj.weight"].to(dt).T
    u = x @ w[p + "mlp.up_proj.weight"].to(dt).T
    return (g / (1.0 + torch.exp(-g)) * u) @ w[p + "mlp.down_proj.weight"].to(dt).T


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float32,
            schedule: Optional[Sequence[Tuple[int, Optional[int]]]] = None) -> torch.Tensor:
    """model.rs:420-516 for one whole sequence from position 0: logits [T, vocab].

    schedule: the order in which layers run, as (layer, index of the earlier
    entry whose keys/values this entry reads instead of making its own, or
    None); default: every layer once."""
    toks = torch.as_tensor(list(tokens), dtype=torch.long)
    T = toks.numel()
    positions = torch.arange(T)
    x = w["model.embed_tokens.weight"].to(dtype)[toks]                       # model.rs:443-445
    schedule = schedule or [(i, None) for i in range(cfg["layers"])]
    kvs: List[Optional[tuple]] = []
    for layer, read_of in schedule:
        p = f"model.layers.{layer}."
        xn = rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])        # 449-451
        d, kv = attention_block(xn, w, p, cfg, positions, None if read_of is None else kvs[read_of])
        kvs.append(kv if read_of is None else None)
        x = x + d                                                            # 487
        xn = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])  # 490-492
        x = x + swiglu(xn, w, p)                                             # 503
    xn = rms_norm(x, w["model.norm.weight"], cfg["eps"])                     # 510-512
    head = w["model.embed_tokens.weight"] if (cfg["tied"] or "lm_head.weight" not in w) else w["lm_head.weight"]
    return (xn @ head.to(dtype).T).to(torch.float32)                         # 513-515, tie rule 190


# ---------------------------------------------------------------------------
# sampling
def argmax_first(x) -> int:
    """sampler.rs:129-137: first index of the maximum (strict >)."""
    best = 0
    xs = [float(v) for v in x]
    for i, v in enumerate(xs):
        if v > xs[best]:
            best = i
    return best


def greedy(cfg, w, prompt: Sequence[int], n: int, dtype=torch.float32, stop=()) -> List[int]:
    """engine.rs:178-206 with a greedy sampler, recomputing the whole sequence each time."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = argmax_first(forward(cfg, w, seq, dtype)[-1])
        if tok in stop:
            break
        out.append(tok)
        seq.append(tok)
    return out


class PlainRng:
    """sampler.rs:29-61."""
    M = (1 << 64) - 1

    def __init__(self, seed):
        z = seed & self.M
        self.s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & self.M
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & self.M
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & self.M
            self.s.append(x ^ (x >> 31))

    def next_u64(self):
        s, M = self.s, self.M
        rot = lambda v, k: ((v << k) | (v >> (64 - k))) & M
        out = (rot((s[1] * 5) & M, 7) * 9) & M
        t = (s[1] << 17) & M
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]
        s[2] ^= t
        s[3] = rot(s[3], 45)
        return out

    def next_f32(self):
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def sample_plain(logits, history, *, temperature, top_k, top_p, min_p, repetition_penalty, rng: PlainRng) -> int:
    """sampler.rs:74-126, step by step in float32."""
    f = np.float32
    l = np.array(logits, dtype=f).copy()
    if repetition_penalty != 1.0:
        for t in dict.fromkeys(history):
            if t < len(l):
                l[t] = l[t] / f(repetition_penalty) if l[t] > 0 else l[t] * f(repetition_penalty)
    if temperature <= 0:
        return argmax_first(l)
    k = len(l) if top_k == 0 else min(top_k, len(l))
    order = sorted(range(len(l)), key=lambda i: (-float(l[i]), i))[:k]
    mx = l[order[0]]
    probs = [f(np.exp(f((l[i] - mx) / f(temperature)))) for i in order]
    s = f(0)
    for p in probs:
        s = f(s + p)
    probs = [f(p / s) for p in probs]
    keep = len(probs)
    if min_p > 0:
        floor = f(probs[0] * f(min_p))
        for i, p in enumerate(probs):
            if p < floor:
                keep = max(i, 1)
                break
    if top_p < 1.0:
        acc = f(0)
        for i in range(keep):
            acc = f(acc + probs[i])
            if acc >= f(top_p):
                keep = i + 1
                break
    tot = f(0)
    for p in probs[:keep]:
        tot = f(tot + p)
    r = f(rng.next_f32() * tot)
    for i in range(keep):
        r = f(r - probs[i])
        if r <= 0:
            return order[i]
    return order[keep - 1]
