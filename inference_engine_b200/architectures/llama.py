"""Llama: how its configuration becomes a model description.

Tensor names are Hugging Face's (engine/model/llama.py:3-8).  Every layer is a pre-norm
residual block of grouped-query attention with rotary position encoding and a gated
feed-forward; layers run once each, in order; the head is tied to the embedding table when
``tie_word_embeddings`` is set (the reference ties in its loader,
engine/model/loader.py:91-92,100-101).
"""

from __future__ import annotations

from dataclasses import asdict

from ..config.model_config import LlamaConfig, estimate_param_count, kv_bytes_per_token
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    scaling = None
    if cfg.rope_scaling is not None:
        scaling = asdict(cfg.rope_scaling)
    positions = {
        "rotary": PartSpec("rotary", {
            "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling,
        })
    }
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            prefix=p,
            block=PartSpec("prenorm_residual"),
            mixer=PartSpec("paged_attention", {
                "q_proj": f"{p}.self_attn.q_proj.weight",
                "k_proj": f"{p}.self_attn.k_proj.weight",
                "v_proj": f"{p}.self_attn.v_proj.weight",
                "o_proj": f"{p}.self_attn.o_proj.weight",
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "position": "rotary",
                "window": None,
            }),
            feed_forward=PartSpec("swiglu", {
                "gate_proj": f"{p}.mlp.gate_proj.weight",
                "up_proj": f"{p}.mlp.up_proj.weight",
                "down_proj": f"{p}.mlp.down_proj.weight",
                "intermediate_size": cfg.intermediate_size,
            }),
            norms={
                "pre_mixer": PartSpec("rms", {
                    "weight": f"{p}.input_layernorm.weight", "eps": cfg.rms_norm_eps}),
                "pre_feed_forward": PartSpec("rms", {
                    "weight": f"{p}.post_attention_layernorm.weight", "eps": cfg.rms_norm_eps}),
            },
        ))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {
            "weight": "model.embed_tokens.weight", "vocab_size": cfg.vocab_size}),
        positions=positions,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms", {"weight": "model.norm.weight", "eps": cfg.rms_norm_eps}),
        head=PartSpec("linear", {
            "weight": None if cfg.tie_word_embeddings else "lm_head.weight",
            "vocab_size": cfg.vocab_size}),
        eos_token_ids=cfg.eos_token_ids,
        bos_token_id=cfg.bos_token_id,
    )


def describe_llama(cfg: LlamaConfig) -> list[str]:
    """The lines ``engine info`` prints about the shape (engine/cli.py:24-33)."""
    return [
        f"architecture        {cfg.architecture}",
        f"layers / hidden     {cfg.num_hidden_layers} / {cfg.hidden_size}",
        f"heads (q / kv)      {cfg.num_attention_heads} / {cfg.num_key_value_heads}"
        f"  (GQA groups: {cfg.num_kv_groups}, head dim {cfg.head_dim})",
        f"parameters          {estimate_param_count(cfg) / 1e9:.2f} B",
        f"KV cache per token  {kv_bytes_per_token(cfg) / 1024:.0f} KiB (bf16)",
    ]


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec, describe_llama)
