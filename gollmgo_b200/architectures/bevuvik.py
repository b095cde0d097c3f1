"""Bevuvik as a ModelSpec: parallel blocks (one RMS norm; mixer and feed-forward read its output;
their sum, times a constant, is added to the stream), two kinds of mixer (differential attention
with a sliding window, biases and interleaved rotary positions stretched for long contexts; or a
softmax attention with capped scores beside a gated delta rule, each branch RMS-normed and the two
averaged), a clamped gated feed-forward, a run of layers that is repeated with the embedding output
mixed in again at the start of every pass, an RMS norm and an untied head.
Tensor names: layer i's start with "l<i>.", the mixer's with "l<i>.mix.", the feed-forward's with
"l<i>.mlp."; "loop.in" mixes the embedding output in.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.bevuvik_config import BevuvikConfig, DiffAttentionConfig
from ..parts.position import YarnScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position(rot, dim: int, interleaved: bool) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    scaling = YarnScaling(*rot.scaling) if rot.scaling else None
    return PartSpec("rope", {"head_dim": dim, "rotary_dim": rot.dims, "theta": rot.base, "scaling": scaling,
                             "interleaved": interleaved})


def _mixer(cfg: BevuvikConfig, m) -> PartSpec:
    names = ("q", "k", "v", "o")
    if isinstance(m, DiffAttentionConfig):
        return PartSpec("diff_attention", {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
                                           "head_dim": m.dim, "v_head_dim": m.vdim, "window": m.window,
                                           "position": _position(m.rot, m.dim, True), "scale": m.scale, "diff": m.diff,
                                           "eps": cfg.eps, "biases": True, "names": names,
                                           "defer_output_bias": True})      # the parallel block adds it with the stream
    left, right = m.left, m.right
    attn = PartSpec("attention", {"hidden_size": cfg.width, "num_heads": left.heads, "num_kv_heads": left.kv_heads,
                                  "head_dim": left.dim, "v_head_dim": left.vdim, "window": left.window,
                                  "position": _position(left.rot, left.dim, False), "scale": left.scale,
                                  "softcap": left.softcap, "names": names})
    delta = PartSpec("gated_delta", {"hidden_size": cfg.width, "num_heads": right.heads, "num_kv_heads": right.kv_heads,
                                     "head_dim": right.dim, "v_head_dim": right.vdim, "conv": right.conv, "eps": cfg.eps})
    return PartSpec("parallel", {"hidden_size": cfg.width, "eps": cfg.eps,
                                 "branches": ((attn, "left.", "left.out"), (delta, "right.", "right.out"))})


def run_order(num_layers: int, loop) -> tuple:
    """The layers in the order they run: those of the loop ``times`` times in a row, every pass
    with cache entries of its own and the embedding output mixed in before its first layer."""
    if loop is None:
        return tuple(RunEntry(i, i) for i in range(num_layers))
    order, cache = [], 0
    for i in range(loop.start):
        order.append(RunEntry(i, cache))
        cache += 1
    for _ in range(loop.times):
        for i in range(loop.start, loop.stop):
            order.append(RunEntry(i, cache, mix_input=(i == loop.start)))
            cache += 1
    for i in range(loop.stop, num_layers):
        order.append(RunEntry(i, cache))
        cache += 1
    return tuple(order)


def bevuvik_spec(cfg: BevuvikConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps})
    block = PartSpec("parallel", {"residual_mult": cfg.residual_mult})
    layers = []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        ff = None
        if lc.mlp is not None:
            ff = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": lc.mlp.ff,
                                        "activation": "clamped_swish", "limit": lc.mlp.limit,
                                        "names": ("gate", "up", "down")})
        layers.append(LayerSpec(block, _mixer(cfg, lc.mixer), ff, norm, None, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp.", mixer_norm_name=p + "norm1", block_prefix=p))
    return ModelSpec(architecture="Bevuvik", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
                     run_order=run_order(len(layers), cfg.loop), final_norm=norm, tie_embeddings=False,
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
                     bos_token_id=cfg.bos_token_id, input_mix_name="loop.in" if cfg.loop is not None else "")


register_architecture("Bevuvik", BevuvikConfig.from_dict, bevuvik_spec)
