"""The Llama dense decoder as a ModelSpec: pre-norm blocks of grouped-query
attention with rotary encoding and a SiLU-gated feed-forward, RMSNorm, optional
tied head.  Tensor names are the checkpoint's own (the reference binds the same
names: kernels/gollmgo_model.cu:462-473, 565-586, 708-710, 731-750, 771-773).
"""
from __future__ import annotations

from ..config import LlamaConfig, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "scaling": cfg.rope_scaling, "interleaved": cfg.rope_interleaved})
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    ffn = PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size,
                                 "intermediate_size": cfg.intermediate_size,
                                 "activation": cfg.hidden_act})
    layers = []
    for i in range(cfg.num_hidden_layers):
        window = cfg.sliding_window if cfg.layer_types[i] == "sliding_attention" else None
        mixer = PartSpec("attention", {"hidden_size": cfg.hidden_size,
                                       "num_heads": cfg.num_attention_heads,
                                       "num_kv_heads": cfg.num_key_value_heads,
                                       "head_dim": cfg.head_dim, "window": window,
                                       "position": position})
        p = f"model.layers.{i}."
        layers.append(LayerSpec(PartSpec("pre_norm"), mixer, ffn, norm, norm,
                                mixer_prefix=p + "self_attn.", ffn_prefix=p + "mlp.",
                                mixer_norm_name=p + "input_layernorm.weight",
                                ffn_norm_name=p + "post_attention_layernorm.weight"))
    return ModelSpec(architecture="LlamaForCausalLM", vocab_size=cfg.vocab_size,
                     hidden_size=cfg.hidden_size, layers=tuple(layers),
                     run_order=tuple(RunEntry(i, i) for i in range(cfg.num_hidden_layers)),
                     final_norm=norm, tie_embeddings=cfg.tie_word_embeddings,
                     embed_name="model.embed_tokens.weight", final_norm_name="model.norm.weight",
                     head_name="lm_head.weight", max_positions=cfg.max_position_embeddings,
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id)


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)
