"""Shared pieces of the tests: two tiny configurations that differ in every size
and option, model folders written to temporary places, and comparison helpers."""
from __future__ import annotations

import functools
import os
import shutil
import tempfile
from typing import Dict, List, Sequence, Tuple

import torch

import wick_b200 as wick
from plain import qwen3_plain as P

# Every size and option differs between A and B: layers 2/3, hidden 64/96, heads
# 4/6, kv heads 2/3 (groups of 2), head_dim 16/32 (coupled 4*16=64 vs decoupled
# 6*32=192 != 96), intermediate 192/160, vocabulary 512/1000 (no power of two),
# rope_theta 1e4/1e6 (top level vs inside rope_parameters), eps 1e-6/1e-5, tied
# vs untied head, max positions 256/512.  C has one kv head (a group of 5), a
# head_dim of 48 and odd widths.
CONFIG_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, intermediate_size=192, num_hidden_layers=2, vocab_size=512,
                max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                hidden_act="silu")
CONFIG_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, num_attention_heads=6,
                num_key_value_heads=3, head_dim=32, intermediate_size=160, num_hidden_layers=3, vocab_size=1000,
                max_position_embeddings=512, rope_parameters={"rope_theta": 1000000.0, "rope_type": "default"},
                rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu", eos_token_id=[7, 9])
CONFIG_C = dict(architectures=["Qwen3ForCausalLM"], hidden_size=72, num_attention_heads=5, num_key_value_heads=1,
                head_dim=48, intermediate_size=100, num_hidden_layers=1, vocab_size=333, max_position_embeddings=1024,
                rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
# D: head_dim 64 with a group of 4, the sizes at which the bfloat16 path takes its
# tensor-core attention kernels for decode as well as for prompts.
CONFIG_D = dict(architectures=["Qwen3ForCausalLM"], hidden_size=128, num_attention_heads=8, num_key_value_heads=2,
                head_dim=64, intermediate_size=256, num_hidden_layers=2, vocab_size=640, max_position_embeddings=2048,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
# E: head_dim 128 with ONE kv head and narrow matrices: every kernel of a decode
# step is short, so a captured step overlaps each kernel with the end of the one
# before it as far as programmatic dependent launch allows.
CONFIG_E = dict(architectures=["Qwen3ForCausalLM"], hidden_size=256, num_attention_heads=4, num_key_value_heads=1,
                head_dim=128, intermediate_size=384, num_hidden_layers=2, vocab_size=1003, max_position_embeddings=8192,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
# F: a group of 5 query heads per kv head at head_dim 128 (the grouping of Qwen3-14B), two kv heads.
CONFIG_F = dict(architectures=["Qwen3ForCausalLM"], hidden_size=320, num_attention_heads=10, num_key_value_heads=2,
                head_dim=128, intermediate_size=448, num_hidden_layers=2, vocab_size=777, max_position_embeddings=2048,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
# R: one layer with the real widths of Qwen3-8B (hidden 4096, 32 heads over 8 kv
# heads of 128, intermediate 12288) and a vocabulary that is no multiple of the
# kernels' tile sizes.
CONFIG_R = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, num_hidden_layers=1, vocab_size=20011,
                max_position_embeddings=4096, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E, "F": CONFIG_F, "R": CONFIG_R}

_tmp_root = None


def tmp_root() -> str:
    global _tmp_root
    if _tmp_root is None:
        _tmp_root = tempfile.mkdtemp(prefix="wick_b200_tests_")
        import atexit
        atexit.register(shutil.rmtree, _tmp_root, ignore_errors=True)
    return _tmp_root


@functools.lru_cache(maxsize=None)
def model_dir(name: str, seed: int = 7, std: float = 0.02, dtype: str = "bf16") -> str:
    """A folder with config.json and model.safetensors of random weights."""
    cfg = wick.config_from_json(CONFIGS[name])
    d = os.path.join(tmp_root(), f"{name}-{seed}-{std}-{dtype}")
    wick.write_random_model(cfg, seed, d, std=std, dtype=torch.bfloat16 if dtype == "bf16" else torch.float32)
    return d


@functools.lru_cache(maxsize=None)
def plain_model(name: str, seed: int = 7, std: float = 0.02, dtype: str = "bf16"):
    return P.read_model_dir(model_dir(name, seed, std, dtype))


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_plain_cache: Dict[tuple, torch.Tensor] = {}


def plain_logits(name: str, tokens: Sequence[int], seed: int = 7, std: float = 0.02) -> torch.Tensor:
    key = (name, seed, std, tuple(tokens))
    if key not in _plain_cache:
        cfg, w = plain_model(name, seed, std)
        _plain_cache[key] = P.forward(cfg, w, tokens)
    return _plain_cache[key]


# Tolerances.  float32: the engine and the plain implementation differ only in
# the order of float32 sums (1e-4 is wick's own bound for two cuttings of one
# sequence, tests/tiny_models.rs:91).  bfloat16: activations are rounded to 8
# bits of mantissa (2^-8 = 0.4 % each) a few times per layer, which gives errors
# of the order of 1 % of the logits' scale on these models; the bound is 2.5 %
# of the largest logit, and the mean cosine similarity of rows must stay above
# 0.9995 (the pattern of wick's tests/tiny_models.rs:115-132).
F32_TOL = 1e-4
BF16_REL = 2.5e-2
BF16_COS = 0.9995


def assert_logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    worst = diff.max().item()
    if dtype in ("float32", "f32"):
        if worst > F32_TOL:
            row = int(diff.max(-1).values.argmax()) if diff.dim() > 1 else 0
            raise AssertionError(f"{what}: float32 logits differ by {worst:.3e} (first bad row near {row})")
    else:
        scale = ref.abs().max().item()
        cos = torch.nn.functional.cosine_similarity(got.reshape(-1, got.shape[-1]),
                                                    ref.reshape(-1, ref.shape[-1]), dim=-1).mean().item()
        assert worst <= BF16_REL * scale, f"{what}: bfloat16 logits differ by {worst:.3e}, scale {scale:.3e}"
        assert cos >= BF16_COS, f"{what}: mean cosine similarity {cos:.5f}"


def make_engine(name: str, dtype: str, max_tokens: int = 2048, seed: int = 7, std: float = 0.02, **kw):
    return wick.Engine.from_dir(model_dir(name, seed, std), dtype=dtype, max_tokens=max_tokens, **kw)


def poison_free_pages(engine) -> None:
    """Fill every cache page that no sequence holds with NaN, so that a read of
    a position that was never written (or of a page given back) shows."""
    held = engine.cache.pages.held()
    for g in engine.cache.groups:
        if g.need.kind != "paged_kv":
            continue
        free = [p for p in range(engine.cache.n_pages) if p not in held and p != 0]
        if free:
            g.storage[:, torch.tensor(free, device=g.storage.device)] = float("nan")


def poison_all(engine) -> None:
    """NaN in every cache position (call while no sequence is live)."""
    for g in engine.cache.groups:
        if g.need.kind == "paged_kv":
            g.storage.fill_(float("nan"))
