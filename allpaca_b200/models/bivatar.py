"""The Bivatar decoder as a :class:`ModelSpec`.

Embedding row times a constant; layers whose norms sit on the sublayers' outputs
(``x += m * norm(sublayer(x))``, one ``m`` for the model); per layer a mixer (attention through a
latent that all heads share, with a rotated key part under stretched rotary frequencies and an
output gate, possibly reading the latent an earlier layer keeps; or grouped-query attention with
weighted RMS norms of queries and keys, a linear distance penalty with fixed slopes per head, a
sliding window that keeps the sequence's first tokens, and an output gate) and a feed-forward
gated by the tanh form of GELU (or none); final norm and head.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.bivatar_config import BivatarConfig
from ..parts import LayerRun, ModelSpec, PartSpec
from .registry import register_architecture

SLOPE_EXPONENT = 8.0             # head h of H has the distance slope 2^(-8 (h + 1) / H)


def bivatar_spec(cfg: BivatarConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "weight_name": ""})
    blocks, prefixes, order = [], [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        cache_from = None
        if L.type == "latent_attention":
            scaling = None
            if m.rot.scaling is not None:
                factor, original, fast, slow = m.rot.scaling
                scaling = {"rope_type": "yarn", "factor": factor, "original": original, "fast": fast, "slow": slow}
            mixer = PartSpec("latent_attention", {
                "hidden_size": H, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": cfg.norm_eps,
                "rope": {"dims": m.rot.dims, "theta": m.rot.base, "scaling": scaling},
                "output_gate": True, "shares_latent": m.kv_from is not None})
            cache_from = m.kv_from             # every layer is one entry of the order, at its own index
        else:
            mixer = PartSpec("distance_biased_attention", {
                "hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "scale": m.scale, "window": m.window, "keep_first": m.keep_first,
                "qk_norm_eps": cfg.norm_eps, "qk_norm_weights": True, "q_temp": None,
                "distance_bias": "linear", "slope_exponent": SLOPE_EXPONENT, "output_gate": True})
        ffn = None
        if L.mlp is not None:
            ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": L.mlp.ff, "activation": "gelu_tanh",
                                      "names": ("gate", "up", "down")})
        order.append(LayerRun(len(blocks), cache_from))
        blocks.append(PartSpec("output_norm", {
            "hidden_size": H, "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm,
            "feed_forward_norm": norm if ffn is not None else None, "residual_mult": cfg.residual_mult,
            "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.", "mixer_norm_prefix": "norm1",
            "feed_forward_norm_prefix": "norm2"}))
        prefixes.append(f"l{i}.")
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(blocks), layer_prefixes=tuple(prefixes),
        order=tuple(order), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        head_name="head", tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings, embedding_scale=cfg.embedding_scale)


register_architecture(("Bivatar", "bivatar"), BivatarConfig, bivatar_spec)
