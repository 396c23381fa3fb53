"""Each part alone, built from a spec with sizes of its own, against the plain
function of the same part."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from wick_b200.cache import Cache  # noqa: E402
from wick_b200.engine.engine import Workspace  # noqa: E402
from wick_b200.parts.base import BuildContext, Hidden, build_part  # noqa: E402
from wick_b200.parts import standard  # noqa: E402,F401
from plain import qwen3_plain as P  # noqa: E402
from test_gpu_kernels import FakeBatch  # noqa: E402

DTYPES = [torch.float32, torch.bfloat16]


def ctx(dtype):
    return BuildContext(dtype=dtype, device=torch.device("cuda"))


def tol(dtype, scale):
    return (3e-5 if dtype == torch.float32 else 2e-2) * scale


def feed(part, tensors):
    part.load(lambda n: tensors.get(n))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    n = build_part("norm", wick.PartSpec("rms", {"width": 100, "eps": 1e-5}), ctx(dtype))
    assert [(s.name, s.shape, s.role) for s in n.tensor_specs()] == [("weight", (100,), "vector")]
    w = 1 + 0.1 * torch.randn(100)
    feed(n, {"weight": w.to(torch.bfloat16)})
    assert n.weight.dtype == torch.float32
    x = torch.randn(7, 100)
    ref = P.rms_norm(x, w.to(torch.bfloat16).float(), 1e-5)
    assert (n.forward(x.cuda(), dtype).float().cpu() - ref).abs().max() < tol(dtype, 4)
    d = torch.randn(1, 7, 100)
    xc = x.cuda()
    out = n.add_forward(xc, d.cuda(), dtype)
    ref = P.rms_norm(x + d[0], w.to(torch.bfloat16).float(), 1e-5)
    assert (out.float().cpu() - ref).abs().max() < tol(dtype, 4) and torch.allclose(xc.cpu(), x + d[0])


def test_rotary_part_tables_and_inv_freq():
    r = build_part("position", wick.PartSpec("rotary_half_split", {"head_dim": 48, "theta": 50000.0}), ctx(torch.float32))
    assert torch.equal(r.rotary_inv_freq().cpu(), P.rope_inv_freq(50000.0, 48))
    b = FakeBatch([3, 2], [10, 0], [[1], [2]]).sb
    cos, sin = r.tables(b)
    assert r.tables(b)[0] is cos, "computed once per step"
    pos = torch.tensor([10, 11, 12, 0, 1]).float()
    assert (cos.cpu() - torch.cos(pos[:, None] * P.rope_inv_freq(50000.0, 48))).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("qk_norm", [True, False])
def test_attention_part(dtype, qk_norm):
    width, heads, kvh, hd = 72, 6, 2, 32
    spec = wick.PartSpec("gqa_attention", {
        "width": width, "heads": heads, "kv_heads": kvh, "head_dim": hd,
        "qk_norm": wick.PartSpec("rms", {"width": hd, "eps": 1e-6}) if qk_norm else None,
        "position": wick.PartSpec("rotary_half_split", {"head_dim": hd, "theta": 1e4}), "scale": None})
    att = build_part("mixer", spec, ctx(dtype))
    names = [s.name for s in att.tensor_specs()]
    assert names[:4] == ["q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight"]
    assert ("q_norm.weight" in names) == qk_norm
    torch.manual_seed(1)
    t = {"q_proj.weight": torch.randn(heads * hd, width) / 8, "k_proj.weight": torch.randn(kvh * hd, width) / 8,
         "v_proj.weight": torch.randn(kvh * hd, width) / 8, "o_proj.weight": torch.randn(width, heads * hd) / 12,
         "q_norm.weight": 1 + 0.1 * torch.randn(hd), "k_norm.weight": 1 + 0.1 * torch.randn(hd)}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    feed(att, t)
    need = att.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim) == ("paged_kv", kvh, hd)
    cache = Cache([need], max_tokens=256, dtype=dtype, device="cuda")
    cache.groups[0].storage.fill_(float("nan"))
    T = 90
    x = torch.randn(T, width).to(dtype)
    b = FakeBatch([T], [0], [[2, 1]]).sb
    b.workspace = Workspace(torch.device("cuda"))
    out = att.forward(x.cuda(), b, cache.view(0), True)
    # plain: the same weights under the names the plain block expects
    w = {"L.self_attn." + k: v.float() for k, v in t.items()}
    if not qk_norm:
        w["L.self_attn.q_norm.weight"] = torch.ones(hd) * math.sqrt(1.0)
        w["L.self_attn.k_norm.weight"] = torch.ones(hd)
    cfg = dict(heads=heads, kv_heads=kvh, head_dim=hd, eps=1e-6, theta=1e4)
    if qk_norm:
        ref, _ = P.attention_block(x.float(), w, "L.", cfg, torch.arange(T))
    else:
        xf = x.float()
        q = (xf @ w["L.self_attn.q_proj.weight"].T).view(T, heads, hd)
        k = (xf @ w["L.self_attn.k_proj.weight"].T).view(T, kvh, hd)
        v = (xf @ w["L.self_attn.v_proj.weight"].T).view(T, kvh, hd)
        inv = P.rope_inv_freq(1e4, hd)
        q, k = P.rope(q, torch.arange(T), inv), P.rope(k, torch.arange(T), inv)
        ref = P.causal_attention(q, k, v).reshape(T, -1) @ w["L.self_attn.o_proj.weight"].T
    assert out.dtype == torch.float32 and out.dim() == 3
    assert (out.sum(0).cpu() - ref).abs().max() < tol(dtype, ref.abs().max())
    # one more token through the decode form
    x1 = torch.randn(1, width).to(dtype)
    b1 = FakeBatch([1], [T], [[2, 1]]).sb
    b1.workspace = b.workspace
    out1 = att.forward(x1.cuda(), b1, cache.view(0), True)
    if qk_norm:
        ref1, _ = P.attention_block(torch.cat([x, x1]).float(), w, "L.", cfg, torch.arange(T + 1))
        assert (out1.sum(0).cpu() - ref1[-1:]).abs().max() < tol(dtype, ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    mlp = build_part("ffn", wick.PartSpec("gated_mlp", {"width": 72, "intermediate": 100, "activation": "silu"}), ctx(dtype))
    t = {"gate_proj.weight": torch.randn(100, 72) / 8, "up_proj.weight": torch.randn(100, 72) / 8,
         "down_proj.weight": torch.randn(72, 100) / 10}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    feed(mlp, t)
    x = torch.randn(5, 72).to(dtype)
    out = mlp.forward(x.cuda(), None)
    ref = P.swiglu(x.float(), {"L.mlp." + k: v.float() for k, v in t.items()}, "L.")
    assert (out.sum(0).cpu() - ref).abs().max() < tol(dtype, ref.abs().max())
    with pytest.raises(ValueError, match="unsupported activation"):
        build_part("ffn", wick.PartSpec("gated_mlp", {"width": 8, "intermediate": 8, "activation": "gelu"}), ctx(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    emb = build_part("embedding", wick.PartSpec("table", {"vocab": 333, "width": 72}), ctx(dtype))
    table = (torch.randn(333, 72) / 4).to(torch.bfloat16)
    feed(emb, {"weight": table})
    tok = torch.tensor([5, 332, 0], dtype=torch.int32)
    assert torch.equal(emb.forward(tok.cuda()).cpu(), table.float()[tok.long()])
    x = torch.randn(4, 72).to(dtype)
    for tied in (True, False):
        head = build_part("head", wick.PartSpec("linear", {"vocab": 333, "width": 72, "tied": tied}), ctx(dtype))
        own = (torch.randn(333, 72) / 4).to(torch.bfloat16)
        assert head.PEERS == ("embedding",)
        head.attach({"embedding": emb})
        head.load(lambda n: own)
        logits = head.forward(x.cuda())
        assert logits.dtype == torch.float32 and head.is_tied == tied
        ref = x.float() @ (table if tied else own).float().T
        assert (logits.cpu() - ref).abs().max() < tol(dtype, ref.abs().max())


def test_unknown_kinds_and_sizes_are_refused():
    with pytest.raises(KeyError, match="no mixer part of kind 'mamba'"):
        build_part("mixer", wick.PartSpec("mamba", {}), ctx(torch.float32))
    for hd in (24, 8, 272):
        with pytest.raises(ValueError, match="multiple of 16"):
            build_part("mixer", wick.PartSpec("gqa_attention", {"width": 8, "heads": 1, "kv_heads": 1, "head_dim": hd}),
                       ctx(torch.float32))
    with pytest.raises(ValueError, match="windowed attention is not built"):
        build_part("mixer", wick.PartSpec("gqa_attention", {"width": 8, "heads": 1, "kv_heads": 1, "head_dim": 16,
                                                            "window": 64}), ctx(torch.float32))
