"""The GPT-2 style decoder of the reference (src/minigpt_infer/model.py:118-187) as data.

Learned absolute positions, ``n_layer`` identical pre-norm blocks of causal multi-head
attention (kv heads = heads) and a tanh-GELU MLP, a final LayerNorm, and an output head
tied to the token embedding.  Weight names are the reference's own.
"""

from __future__ import annotations

from ..config.model_config import GPTConfig
from ..config.registry import register_model
from ..parts.spec import LayerCall, ModelSpec, PartSpec, pre_norm_layer


@register_model("MiniGPTLMHeadModel", "minigpt", "MiniGPT", "GPT", config_class=GPTConfig)
def describe_minigpt(cfg: GPTConfig) -> ModelSpec:
    norm = {"width": cfg.n_embd, "eps": cfg.layer_norm_epsilon, "bias": cfg.bias}
    layers = []
    for i in range(cfg.n_layer):
        layers.append(pre_norm_layer(
            prefix=f"blocks.{i}.",
            norm1=PartSpec("layernorm", norm, "ln1"),
            mixer=PartSpec("causal_attention", {
                "width": cfg.n_embd, "n_head": cfg.n_head, "n_kv_head": cfg.n_head,
                "head_dim": cfg.head_dim, "bias": cfg.bias}, "attn"),
            norm2=PartSpec("layernorm", norm, "ln2"),
            feed_forward=PartSpec("dense_mlp", {
                "width": cfg.n_embd, "inner": cfg.n_inner, "bias": cfg.bias,
                "activation": cfg.activation_function}, "mlp")))
    return ModelSpec(
        architecture=cfg.architecture,
        width=cfg.n_embd,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding",
                           {"vocab_size": cfg.vocab_size, "width": cfg.n_embd}, "tok_emb"),
        position=PartSpec("learned_absolute",
                          {"n_positions": cfg.n_positions, "width": cfg.n_embd}, "pos_emb"),
        layers=tuple(layers),
        layer_order=tuple(LayerCall(i, i) for i in range(cfg.n_layer)),
        final_norm=PartSpec("layernorm", norm, "ln_f"),
        head=PartSpec("tied_head", {"vocab_size": cfg.vocab_size, "width": cfg.n_embd,
                                    "tied_to": "tok_emb.weight"}, "lm_head"))
