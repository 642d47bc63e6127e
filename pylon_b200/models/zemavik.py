"""Zemavik as a :class:`ModelSpec`.

The embedding rows plus a learnt vector per position enter the residual sum.  The configuration lists the layers; each is
a ``hyper_prenorm`` block over the plain residual sum (RMS norms) around either a ``parallel_mixers`` mixer - a
``gqa_attention`` without positions (no q/k norm, scores times a given factor, inside chunks of positions, values of their
own width) beside a ``state_space`` layer, the two outputs RMS-normed over the width and averaged - or a ``gated_delta``
mixer with a decay per key channel, narrow middles in the decay's and the gate's projections and a sigmoid gate; and a
``gated_unit`` feed-forward (relu, biases), an ``expert_mixture`` (silu, no biases, a router with a bias) or none.  The
run order repeats the loop's span, each pass with caches of its own and entered through the ``loop.in`` map of stream and
embedding output side by side.  The head is the embedding table.  Tensor names: ``embed``, ``pos``, ``loop.in``,
``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from typing import Optional

from pylon_b200.config.model_config import ConfigError, ZemavikConfig, ZemavikLayer
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

UNIT_EPS = 1e-6       # under the root when q and k of the delta rule are made unit vectors


def _mixer(config: ZemavikConfig, layer: ZemavikLayer, index: int) -> PartSpec:
    if layer.kind == "parallel":
        left, right = layer.left, layer.right
        attention = PartSpec("gqa_attention", {
            "width": config.width, "n_heads": left.heads, "n_kv_heads": left.kv_heads, "head_dim": left.dim, "value_dim": left.vdim,
            "scale": left.scale, "chunk": left.chunk, "names": {"q": "q", "k": "k", "v": "v", "o": "o"},
        })
        recurrent = PartSpec("state_space", {
            "width": config.width, "n_heads": right.heads, "value_dim": right.vdim, "state_dim": right.state, "groups": right.groups,
            "norm_groups": right.norm_groups, "conv_taps": right.conv, "norm_eps": config.norm_eps,
        })
        return PartSpec("parallel_mixers", {
            "width": config.width, "mixers": (attention, recurrent), "prefixes": ("left.", "right."), "norm_names": ("left.out", "right.out"),
            "norm_eps": config.norm_eps,
        })
    delta = layer.delta
    if delta.decay_rank is None or delta.gate_rank is None:
        raise ConfigError(f"layer {index}: the widths of the decay's and the gate's middles are not known: the checkpoint's tensor shapes "
                          "give them, or the keys 'decay_rank' and 'gate_rank' of the mixer")
    return PartSpec("gated_delta", {
        "width": config.width, "n_heads": delta.heads, "n_kv_heads": delta.kv_heads, "head_dim": delta.dim, "value_dim": delta.vdim,
        "conv_taps": delta.conv, "norm_eps": config.norm_eps, "unit_eps": UNIT_EPS, "decay": "channel", "decay_rank": delta.decay_rank,
        "gate_rank": delta.gate_rank, "gate_activation": "sigmoid",
        "names": {"decay_in": "a1", "decay": "a2", "gate_in": "g1", "gate": "g2"},
    })


def _feed_forward(config: ZemavikConfig, layer: ZemavikLayer) -> Optional[PartSpec]:
    mlp = layer.mlp
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return PartSpec("gated_unit", {"width": config.width, "intermediate": mlp.ff, "activation": "relu", "bias": True, "bias_suffix": ".b",
                                       "names": {"gate": "gate", "up": "up", "down": "down"}})
    return PartSpec("expert_mixture", {"width": config.width, "intermediate": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                                       "activation": "silu", "router_bias": True})


def zemavik_spec(config: ZemavikConfig, max_positions: Optional[int] = None) -> ModelSpec:
    positions = config.max_positions if max_positions is None else min(config.max_positions, int(max_positions))
    norm = PartSpec("rmsnorm", {"width": config.width, "eps": config.norm_eps, "weight_name": ""})
    layers = []
    for index, layer in enumerate(config.layers):
        feed_forward = _feed_forward(config, layer)
        block = PartSpec("hyper_prenorm", {
            "mixer": _mixer(config, layer, index), "feed_forward": feed_forward, "mixer_norm": norm,
            "ffn_norm": norm if feed_forward is not None else None,
        })
        layers.append(LayerSpec(f"l{index}.", block))
    return ModelSpec(
        width=config.width,
        vocab_size=config.vocab,
        max_positions=positions,
        embedding_name="embed",
        lm_head_name=None,
        final_norm=norm,
        final_norm_prefix="final.norm",
        layers=tuple(layers),
        order=tuple(RunSpec(index, reenter=starts) for index, starts in config.run_order()),
        eos_token_ids=config.eos_token_ids,
        position_name="pos",
        position_rows=config.max_positions,
        reentry_name="loop.in" if any(starts for _, starts in config.run_order()) else None,
    )
