"""Tekenex as a ModelSpec: post-norm blocks with layer scale (the norm, a LayerNorm with bias,
sits on each sublayer's output; the sublayers read the residual stream itself), latent attention
without position encoding and with a sigmoid gate per head, and per layer a squared-ReLU
feed-forward, a mixture of SiLU-gated experts with a biased router and a shared expert, or no
feed-forward at all.  The head is the embedding table; the final norm is a LayerNorm.
Tensor names: layer i's start with "l<i>.", the mixer's with "l<i>.mix.", the feed-forward's with
"l<i>.mlp.".
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.tekenex_config import TekenexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _feed_forward(width: int, f) -> PartSpec:
    gated_names = ("gate", "up", "down")
    if f.kind == "dense":
        return PartSpec("mlp", {"hidden_size": width, "intermediate_size": f.ff, "activation": "relu2",
                                "names": ("up", "down")})
    shared = None
    if f.shared is not None:
        shared = PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": f.shared.ff,
                                        "activation": "silu", "names": gated_names})
    return PartSpec("moe", {"hidden_size": width, "intermediate_size": f.expert.ff, "experts": f.experts,
                            "top": f.top, "router_bias": True, "shared": shared})


def tekenex_spec(cfg: TekenexConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"size": cfg.width, "eps": cfg.eps})
    block = PartSpec("post_norm", {"layer_scale": True, "scale_names": ("ls1", "ls2")})
    layers, ignorable = [], []
    for i, lc in enumerate(cfg.layers):
        m = lc.mixer
        mixer = PartSpec("latent_attention", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim,
                                              "v_head_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                                              "eps": cfg.eps, "gate": True})
        p = f"l{i}."
        ff = _feed_forward(cfg.width, lc.mlp) if lc.mlp is not None else None
        if ff is None:
            ignorable += [p + "norm2", p + "norm2.b", p + "ls2"]
        layers.append(LayerSpec(block, mixer, ff, norm, norm if ff is not None else None,
                                mixer_prefix=p + "mix.", ffn_prefix=p + "mlp.", mixer_norm_name=p + "norm1",
                                ffn_norm_name=p + "norm2", block_prefix=p))
    n = len(layers)
    return ModelSpec(architecture="Tekenex", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
                     run_order=tuple(RunEntry(i, i) for i in range(n)), final_norm=norm, tie_embeddings=True,
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
                     bos_token_id=cfg.bos_token_id, ignorable_tensors=tuple(ignorable))


register_architecture("Tekenex", TekenexConfig.from_dict, tekenex_spec)
