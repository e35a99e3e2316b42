"""From a `LlamaConfig` to the list of layers the engine runs.

Formulas and their order are the reference's plain "llama" path: RMSNorm,
q/k/v projections without bias, rotary positions on q and k, causal
grouped-query attention, output projection added to the residual, RMSNorm,
SwiGLU feed-forward added to the residual; final RMSNorm and output head,
which is the embedding table when the model ties them
(src/model.rs:996-1188, src/model.rs:637-638).
"""
from __future__ import annotations

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .llama import LlamaConfig


def llama_rope_spec(cfg: LlamaConfig) -> PartSpec:
    params = {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.head_dim,      # the reference's rope_dim defaults to the head size (src/model.rs:205)
        "theta": cfg.rope_theta,
        # safetensors checkpoints keep q/k rows in the trained order, whose pairs are (i, i + half);
        # GGUF converters permute them for adjacent pairs (src/model.rs:27-28, scripts/csm-convert.py:33-35)
        "pairing": "half",
        "scaling": None,
    }
    if cfg.rope_scaling is not None:
        rs = cfg.rope_scaling
        params["scaling"] = {
            "rope_type": rs.rope_type,
            "factor": rs.factor,
            "low_freq_factor": rs.low_freq_factor,
            "high_freq_factor": rs.high_freq_factor,
            "original_max_position_embeddings": rs.original_max_position_embeddings,
        }
    return PartSpec("rotary", params)


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "scale": cfg.attention_scale,
        "window": None,
        "position": llama_rope_spec(cfg),
    })
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = tuple(
        LayerSpec(prefix=f"model.layers.{i}.", block="prenorm_residual", mixer_norm=norm, mixer=mixer,
                  ffn_norm=norm, ffn=ffn)
        for i in range(cfg.num_hidden_layers))
    spec = ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
        layers=layers,
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "tied": cfg.tie_word_embeddings}),
        stop_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec
