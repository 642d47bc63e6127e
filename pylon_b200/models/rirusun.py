"""Rirusun as a :class:`ModelSpec`.

The configuration lists the layers; each is a ``parallel_sublayers`` block - one ``dynamic_tanh`` norm whose output both the
mixer and the feed-forward read, their outputs added to the residual sum together - around one of three mixers and an
``expert_mixture`` or none.  The mixers: ``weighted_mixers`` of a ``gqa_attention`` (no rotation; q and k normed over their
whole rows; a bias by distance from a table of logarithmic buckets; a sliding window that keeps the first tokens; a sink)
beside a ``gated_linear_recurrence``, each output times a factor; ``matrix_memory``; and ``latent_attention`` whose queries
come straight from the input and whose shared key part is rotated in halves with YaRN-scaled frequencies.  The experts are
ungated (erf gelu), routed by sigmoid scores with a correction inside the best groups, with a gated shared expert.  The run
order repeats the loop's span, each pass with caches of its own.  Tensor names: ``embed``, ``l<i>.norm1`` (``.alpha``, ``.b``),
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from pylon_b200.config.model_config import ConfigError, RirusunConfig, RirusunLayer
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

MAX_POSITIONS = 1 << 20    # no learnt table limits a request's length; the rotation tables are cut to the engine's longest context
DECAY_FACTOR = 8.0         # log a = -DECAY_FACTOR * r * softplus(lam) in the gated linear recurrence
MEMORY_EPS = 1e-6          # added below the matrix memory's read-out
SHARE_EPS = 1e-20          # added to the sum the chosen experts' scores are divided by


def _mixer(config: RirusunConfig, layer: RirusunLayer, index: int, positions: int) -> PartSpec:
    if layer.kind == "parallel":
        left, right = layer.left, layer.right
        if left.bias_rows is None:
            raise ConfigError(f"layer {index}: the rows of the bias table are not known: the checkpoint's tensor shapes give them, or the key 'bias_rows'")
        attention = PartSpec("gqa_attention", {
            "width": config.width, "n_heads": left.heads, "n_kv_heads": left.kv_heads, "head_dim": left.dim, "value_dim": left.vdim,
            "scale": left.scale, "window": left.window, "keep_first": left.keep_first, "qk_norm": "whole", "qk_norm_eps": config.norm_eps,
            "distance_bias": {"rows": left.bias_rows, "far": left.bias_max}, "sink": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "distance_bias": "rel", "sink": "sink"},
        })
        recurrent = PartSpec("gated_linear_recurrence", {
            "width": config.width, "channels": right.width, "blocks": right.blocks, "conv_taps": right.conv, "decay_factor": DECAY_FACTOR,
        })
        return PartSpec("weighted_mixers", {"mixers": (attention, recurrent), "prefixes": ("left.", "right."), "scales": (layer.left_scale, layer.right_scale)})
    if layer.kind == "mlstm":
        heads, dim, vdim, cap = layer.memory
        return PartSpec("matrix_memory", {"width": config.width, "n_heads": heads, "head_dim": dim, "value_dim": vdim, "gate_cap": cap,
                                          "norm_eps": config.norm_eps, "read_eps": MEMORY_EPS})
    heads, dim, rot_dim, vdim, kv_rank, scale, rot = layer.latent
    rotation = None
    if rot is not None:
        scaling = None if rot.scaling is None else {"kind": "yarn", **dict(rot.scaling)}
        rotation = PartSpec("rope", {"head_dim": rot_dim, "theta": rot.base, "max_positions": positions, "rotary_dim": rot.dims, "scaling": scaling,
                                     "layout": "halves"})
    return PartSpec("latent_attention", {
        "width": config.width, "n_heads": heads, "head_dim": dim, "rot_dim": rot_dim, "value_dim": vdim, "q_rank": None, "kv_rank": kv_rank,
        "norm_eps": config.norm_eps, "scale": scale, "position": rotation, "names": {"q": "q"}, "split_weights": True,
    })


def _feed_forward(config: RirusunConfig, layer: RirusunLayer) -> Optional[PartSpec]:
    mlp = layer.mlp
    if mlp is None:
        return None
    return PartSpec("expert_mixture", {
        "width": config.width, "intermediate": mlp.ff, "experts": mlp.experts, "top": mlp.top, "activation": "gelu", "gated": False,
        "routing": "sigmoid", "correction": True, "groups": mlp.groups, "groups_keep": mlp.groups_keep, "share_eps": SHARE_EPS,
        "shared_intermediate": mlp.shared_ff,
    })


def rirusun_spec(config: RirusunConfig, max_positions: Optional[int] = None) -> ModelSpec:
    positions = MAX_POSITIONS if max_positions is None else int(max_positions)
    norm = PartSpec("dynamic_tanh", {"width": config.width, "weight_name": "", "alpha_name": ".alpha", "bias_name": ".b"})
    layers = []
    for index, layer in enumerate(config.layers):
        block = PartSpec("parallel_sublayers", {"mixer": _mixer(config, layer, index, positions), "feed_forward": _feed_forward(config, layer), "norm": norm})
        layers.append(LayerSpec(f"l{index}.", block))
    return ModelSpec(
        width=config.width,
        vocab_size=config.vocab,
        max_positions=positions,
        embedding_name="embed",
        lm_head_name="head",
        final_norm=norm,
        final_norm_prefix="final.norm",
        layers=tuple(layers),
        order=tuple(RunSpec(index) for index in config.run_order()),
        eos_token_ids=config.eos_token_ids,
        embedding_scale=config.embedding_scale,
    )
