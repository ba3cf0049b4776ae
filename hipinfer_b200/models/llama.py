"""The dense Llama decoder as a ModelSpec: every layer a pre-norm block of grouped-query
attention with rotary positions and a SwiGLU feed-forward, RMSNorm everywhere, tied or untied
head; tensor names as in scripts/export.py:221-287 of the reference. This is the graph that
src/api.cu:1666-1718 runs (docs/porting-a-model.md:9-21).
"""
from __future__ import annotations

from ..config import LlamaConfig, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def llama_spec(c: LlamaConfig) -> ModelSpec:
    position = PartSpec("rope", dict(head_dim=c.head_dim, rotary_dim=c.head_dim, theta=c.rope_theta,
                                     scaling=c.rope_scaling.to_dict() if c.rope_scaling else None, pairing="half"))
    layers = []
    for l in range(c.num_hidden_layers):
        layers.append(LayerSpec(prefix=f"model.layers.{l}.", block="pre_norm", parts=dict(
            mixer=PartSpec("attention", dict(hidden_size=c.hidden_size, n_heads=c.num_attention_heads,
                                             n_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, window=0,
                                             position=position)),
            mixer_norm=PartSpec("rmsnorm", dict(name="input_layernorm.weight", size=c.hidden_size, eps=c.rms_norm_eps)),
            feed_forward=PartSpec("swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size)),
            feed_forward_norm=PartSpec("rmsnorm", dict(name="post_attention_layernorm.weight", size=c.hidden_size,
                                                       eps=c.rms_norm_eps)),
        )))
    embed_name = "model.embed_tokens.weight"
    head = dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)
    head.update(dict(tied_to=embed_name) if c.tie_word_embeddings else dict(name="lm_head.weight"))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.hidden_size, vocab_size=c.vocab_size,
        max_position=c.max_position_embeddings,
        embedding=PartSpec("token", dict(name=embed_name, vocab_size=c.vocab_size, hidden_size=c.hidden_size)),
        layers=tuple(layers), order=tuple(RunStep(l) for l in range(c.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(name="model.norm.weight", size=c.hidden_size, eps=c.rms_norm_eps)),
        head=PartSpec("linear", head), eos_token_ids=c.eos_token_ids)


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec)
