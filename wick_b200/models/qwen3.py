"""The Qwen3 dense decoder as a model spec.

Every layer: pre-norm residual block of grouped-query attention (no projection
biases, an RMS norm per head on q and k before a half-split rotation over the
whole head) and a SwiGLU feed-forward; RMS norms share one eps; a final norm and
an output head that is tied to the embedding on request (wick ``src/model.rs``
``from_tensors`` 178-229 for the tensor names, ``forward`` 420-516 for the order,
``src/config.rs:122`` for the q/k norm being part of the architecture).
"""
from __future__ import annotations

from ..config.base import Architecture, register_architecture
from ..config.qwen3 import Qwen3Config
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    head_norm = PartSpec("rms", {"width": cfg.head_dim, "eps": cfg.rms_norm_eps})
    rope = PartSpec("rotary_half_split", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    mixer = PartSpec("gqa_attention", {
        "width": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim, "qk_norm": head_norm, "position": rope, "scale": None, "window": None})
    ffn = PartSpec("gated_mlp", {"width": cfg.hidden_size, "intermediate": cfg.intermediate_size,
                                 "activation": "silu"})
    names = {"mixer": "self_attn.", "mixer_norm": "input_layernorm.", "ffn": "mlp.",
             "ffn_norm": "post_attention_layernorm."}
    layers = tuple(
        LayerSpec(block=PartSpec("prenorm_residual"), mixer=mixer, mixer_norm=norm, ffn=ffn, ffn_norm=norm,
                  prefix=f"model.layers.{i}.", names=names)
        for i in range(cfg.num_hidden_layers))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab=cfg.vocab_size, width=cfg.hidden_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "width": cfg.hidden_size}),
        embedding_prefix="model.embed_tokens.",
        layers=layers,
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm, final_norm_prefix="model.norm.",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": cfg.hidden_size,
                                 "tied": cfg.tie_word_embeddings}),
        head_prefix="lm_head.",
        ignore_tensors=("*.rotary_emb.inv_freq",),
        stop_token_ids=cfg.eos_token_ids)
    spec.validate()
    return spec


QWEN3 = register_architecture(Architecture(
    names=("Qwen3ForCausalLM", "qwen3"), config_cls=Qwen3Config, build_spec=build_spec))
