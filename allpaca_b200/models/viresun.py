"""The Viresun decoder as a :class:`ModelSpec`.

Embedding row plus a sinusoidal position vector (base 10000), RMS-normed; pre-norm layers whose
norms have one number as their weight; per layer a mixer (attention without rotation: weightless
RMS norm of queries and keys, a query temperature that grows with the logarithm of the position,
a logarithmic distance bias per head, a sliding window; or a Mamba-2 state-space mixer) and a
feed-forward (ReLU-gated dense, routed experts with a clamped sigmoid gate, or none); final norm
and head.  A layer that owns no tensors and computes with another layer's is a second entry of the
order naming that layer; the engine gives every entry of the order separate pages and state.

Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.viresun_config import ViresunConfig
from ..parts import LayerRun, ModelSpec, PartSpec
from .registry import register_architecture

SINUSOID_BASE = 10000.0
EXPERT_GATE_ALPHA = 1.702        # g * sigmoid(1.702 g)
EXPERT_UP_SHIFT = 1.0            # ... * (u + 1)


def viresun_spec(cfg: ViresunConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "scalar_weight": True, "weight_name": ""})
    blocks, prefixes, index_of, order = [], [], {}, []
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            order.append(LayerRun(index_of[L.weights_of]))
            continue
        m = L.mixer
        if L.type == "attention":
            mixer = PartSpec("distance_biased_attention", {
                "hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "scale": m.scale, "window": m.window, "qk_norm_eps": cfg.norm_eps,
                "q_temp": {"coef": m.q_temp[0], "every": m.q_temp[1]} if m.q_temp else None,
                "distance_bias": True})
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": H, "heads": m.heads, "value_dim": m.vdim, "state_size": m.state, "groups": m.groups,
                "conv_taps": m.conv, "norm_groups": m.norm_groups, "norm_eps": cfg.norm_eps})
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": L.mlp.ff, "activation": "relu",
                                      "names": ("gate", "up", "down")})
        elif L.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": H, "expert_size": L.mlp.ff, "experts": L.mlp.experts, "top": L.mlp.top,
                "activation": "clamped_sigmoid", "limit": L.mlp.limit, "alpha": EXPERT_GATE_ALPHA,
                "shift": EXPERT_UP_SHIFT, "router_bias": True})
        index_of[i] = len(blocks)
        order.append(LayerRun(len(blocks)))
        blocks.append(PartSpec("prenorm", {
            "hidden_size": H, "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm,
            "feed_forward_norm": norm if ffn is not None else None,
            "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.", "mixer_norm_prefix": "norm1",
            "feed_forward_norm_prefix": "norm2"}))
        prefixes.append(f"l{i}.")
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(blocks), layer_prefixes=tuple(prefixes),
        order=tuple(order), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        head_name="head", tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding_sinusoid_base=SINUSOID_BASE, embedding_norm=norm, embedding_norm_prefix="embed.norm")


register_architecture(("Viresun", "viresun"), ViresunConfig, viresun_spec)
