"""Typed model configurations read from a checkpoint's ``config.json``.

Every size and constant of a model comes from here; no part of the engine carries a
size of its own.  A configuration class knows two things: how to read its architecture's
``config.json`` keys (and which options it refuses), and how to describe the model as an
architecture-neutral :class:`~pylon_b200.parts.spec.ModelSpec` that the part builders use.

Reference parity: the field list follows ``src/pylon/model/config.py:20-32`` and the
refusals follow ``src/pylon/model/config.py:35-62``; unlike the reference, no shape is
pinned to the Qwen3-4B checkpoint.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, ClassVar, Mapping, Optional


class ConfigError(ValueError):
    """A config.json that is malformed or asks for something the engine does not build."""


def _require(data: Mapping[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in data:
        raise ConfigError(f"config.json has no '{key}'")
    value = data[key]
    if isinstance(value, bool) and kind is not bool:
        raise ConfigError(f"config.json '{key}' must be {kind}, got a bool")
    if not isinstance(value, kind):
        raise ConfigError(f"config.json '{key}' must be {kind}, got {type(value).__name__}")
    return value


def _positive_int(data: Mapping[str, Any], key: str) -> int:
    value = _require(data, key, int)
    if value < 1:
        raise ConfigError(f"config.json '{key}' must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Qwen3 dense decoder (``Qwen3ForCausalLM``).

    Field names are the checkpoint's own config.json keys.
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"
    model_type: ClassVar[str] = "qwen3"

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)
    torch_dtype: str = "bfloat16"

    def __post_init__(self) -> None:
        for name in (
            "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings",
        ):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        if data.get("model_type", cls.model_type) != cls.model_type:
            raise ConfigError(f"model_type must be '{cls.model_type}', got {data.get('model_type')!r}")
        # Options of the checkpoint format that this architecture's engine does not build.
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {data.get('hidden_act')!r} is not supported (silu only)")
        if data.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported")
        if data.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported")
        if data.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window=true is not supported")
        if data.get("sliding_window") is not None:   # refused as raun6k/Pylon refuses it (src/pylon/model/config.py:48), whatever use_sliding_window says
            raise ConfigError(f"sliding_window={data.get('sliding_window')!r} is not supported (Qwen3 dense attends to every earlier token)")
        heads = _positive_int(data, "num_attention_heads")
        hidden = _positive_int(data, "hidden_size")
        if "head_dim" in data and data["head_dim"] is not None:
            head_dim = _positive_int(data, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        kv_heads = data.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _positive_int(data, "num_key_value_heads")
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(x) for x in eos)
        return cls(
            vocab_size=_positive_int(data, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_positive_int(data, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_positive_int(data, "intermediate_size"),
            max_position_embeddings=_positive_int(data, "max_position_embeddings"),
            rope_theta=float(_require(data, "rope_theta", (int, float))),
            rms_norm_eps=float(_require(data, "rms_norm_eps", (int, float))),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen3Config":
        return cls.from_dict(json.loads(Path(path).read_text()))

    # -- writing -----------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        data = asdict(self)
        eos = data.pop("eos_token_ids")
        data["architectures"] = [self.architecture]
        data["model_type"] = self.model_type
        data["hidden_act"] = "silu"
        data["attention_bias"] = False
        data["rope_scaling"] = None
        data["use_sliding_window"] = False
        data["sliding_window"] = None
        if eos:
            data["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        return data

    # -- derived sizes -----------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim


# ---------------------------------------------------------------------------------------
def _mapping(data: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    value = _require(data, key, dict)
    return value


def _number(data: Mapping[str, Any], key: str) -> float:
    return float(_require(data, key, (int, float)))


@dataclass(frozen=True)
class VopepelLayer:
    """One layer of a Vopepel model: which mixer (``delta`` or ``attention``) with its sizes, and its feed-forward
    (``None``: the layer has none)."""

    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: Optional[int] = None          # delta: taps of the short convolution
    scale: Optional[float] = None       # attention: factor on the scores
    softcap: Optional[float] = None     # attention: scores go through softcap * tanh(score / softcap); None: no cap
    chunk: Optional[int] = None         # attention: a token sees only keys of its own chunk of positions; None: all before it
    v_mix: bool = False                 # attention: values are mixed with those of the first layer that says so
    ff: Optional[int] = None            # feed-forward: inner width; None: no feed-forward
    ff_kind: str = "dense"
    ff_limit: Optional[float] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "VopepelLayer":
        kind = _require(data, "type", str)
        if kind not in ("delta", "attention"):
            raise ConfigError(f"layer {index}: unknown type {kind!r} (delta, attention)")
        mixer = _mapping(data, "mixer")
        fields = dict(kind=kind, heads=_positive_int(mixer, "heads"), kv_heads=_positive_int(mixer, "kv_heads"),
                      dim=_positive_int(mixer, "dim"), vdim=_positive_int(mixer, "vdim"))
        if fields["heads"] % fields["kv_heads"]:
            raise ConfigError(f"layer {index}: {fields['heads']} heads cannot be grouped over {fields['kv_heads']} kv_heads")
        if kind == "delta":
            fields["conv"] = _positive_int(mixer, "conv")
        else:
            fields["scale"] = _number(mixer, "scale")
            if mixer.get("softcap") is not None:
                fields["softcap"] = _number(mixer, "softcap")
                if not fields["softcap"] > 0:
                    raise ConfigError(f"layer {index}: softcap must be positive")
            if mixer.get("mask") is not None:
                fields["chunk"] = _positive_int(_mapping(mixer, "mask"), "size")
            fields["v_mix"] = bool(mixer.get("v_mix", False))
        mlp = data.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"layer {index}: 'mlp' must be an object or null")
            fields["ff_kind"] = str(mlp.get("kind", "dense"))
            if fields["ff_kind"] != "dense":
                raise ConfigError(f"layer {index}: feed-forward kind {fields['ff_kind']!r} is not built (dense)")
            fields["ff"] = _positive_int(mlp, "ff")
            fields["ff_limit"] = _number(mlp, "limit")
            if not fields["ff_limit"] > 0:
                raise ConfigError(f"layer {index}: the feed-forward's limit must be positive")
        return cls(**fields)

    def to_dict(self) -> dict[str, Any]:
        mixer: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim}
        if self.kind == "delta":
            mixer["conv"] = self.conv
        else:
            mixer["scale"] = self.scale
            if self.softcap is not None:
                mixer["softcap"] = self.softcap
            if self.chunk is not None:
                mixer["mask"] = {"size": self.chunk}
            if self.v_mix:
                mixer["v_mix"] = True
        mlp = None if self.ff is None else {"kind": self.ff_kind, "ff": self.ff, "limit": self.ff_limit}
        return {"type": self.kind, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class VopepelConfig:
    """Vopepel: a decoder whose layers are, in an order the configuration lists, gated-delta-rule mixers and chunked
    soft-capped attention without positions, each with a clamped gated feed-forward (or none); layer norm without bias;
    the residual stream optionally kept as several copies (hyper-connections); the sublayers' outputs times a factor.

    ``config.json`` names the model by ``"architecture": "Vopepel"``.  Field names follow its keys.
    """

    architecture: ClassVar[str] = "Vopepel"

    vocab: int
    width: int
    layers: tuple[VopepelLayer, ...]
    norm_eps: float
    residual_mult: float = 1.0
    streams: Optional[int] = None      # copies of the residual stream; None: the plain residual sum
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must be 1 to 8, got {self.streams}")
        mixing = [layer for layer in self.layers if layer.v_mix]
        if any((layer.kv_heads, layer.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for layer in mixing):
            raise ConfigError("layers that mix values must have the same kv_heads and vdim")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "VopepelConfig":
        layers = _require(data, "layers", list)
        eos = data.get("eos_token_id")
        streams = data.get("streams")
        return cls(
            vocab=_positive_int(data, "vocab"),
            width=_positive_int(data, "width"),
            layers=tuple(VopepelLayer.from_dict(layer, index) for index, layer in enumerate(layers)),
            norm_eps=_number(_mapping(data, "norm"), "eps"),
            residual_mult=float(data.get("residual_mult", 1.0)),
            streams=None if streams is None else _positive_int(data, "streams"),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos)),
        )

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
        }
        if self.streams is not None:
            data["streams"] = self.streams
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data


# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RotarySpec:
    """A rotation of query and key by position: the first ``dims`` elements of a head, frequencies ``base^(-2i / dims)``, and
    an optional scaling of the frequencies (its parameters as the configuration names them)."""

    dims: int
    base: float
    scaling: Optional[tuple[tuple[str, float], ...]] = None   # sorted (name, number) pairs: hashable

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str, scaling_keys: tuple[str, ...]) -> "RotarySpec":
        dims = _positive_int(data, "dims")
        if dims % 2:
            raise ConfigError(f"{where}: rot.dims must be even, got {dims}")
        scaling = data.get("scaling")
        pairs = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}: rot.scaling must be an object or null")
            pairs = tuple((key, _number(scaling, key)) for key in sorted(scaling_keys))
        return cls(dims=dims, base=_number(data, "base"), scaling=pairs)

    def to_dict(self) -> dict[str, Any]:
        return {"dims": self.dims, "base": self.base, "scaling": None if self.scaling is None else dict(self.scaling)}


@dataclass(frozen=True)
class FikeraxLayer:
    """One layer of a Fikerax model: its mixer (``lightning``, ``attention`` or ``latent_attention``) with its sizes, and the inner
    width of its feed-forward (``None``: the layer has none)."""

    kind: str
    heads: int
    dim: int
    vdim: int
    decay: Optional[tuple[float, ...]] = None   # lightning: one per head
    kv_heads: Optional[int] = None              # attention
    rot_dim: Optional[int] = None               # latent attention: rotated query/key elements per head, beside ``dim`` others
    q_rank: Optional[int] = None                # latent attention: size of the query latent
    kv_rank: Optional[int] = None               # latent attention: size of the key/value latent
    scale: Optional[float] = None               # both attentions: factor on the scores
    window: Optional[int] = None                # both attentions: a token sees itself and the window - 1 tokens before it; None: all
    rot: Optional[RotarySpec] = None
    ff: Optional[int] = None
    ff_kind: str = "dense"

    KINDS: ClassVar[tuple[str, ...]] = ("lightning", "attention", "latent_attention")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "FikeraxLayer":
        where = f"layer {index}"
        kind = _require(data, "type", str)
        if kind not in cls.KINDS:
            raise ConfigError(f"{where}: unknown type {kind!r} ({', '.join(cls.KINDS)})")
        mixer = _mapping(data, "mixer")
        fields: dict[str, Any] = dict(kind=kind, heads=_positive_int(mixer, "heads"), dim=_positive_int(mixer, "dim"), vdim=_positive_int(mixer, "vdim"))
        if kind == "lightning":
            decay = _require(mixer, "decay", list)
            if len(decay) != fields["heads"] or any(not isinstance(d, (int, float)) or not 0.0 <= d <= 1.0 for d in decay):
                raise ConfigError(f"{where}: 'decay' must list one number in [0, 1] per head")
            fields["decay"] = tuple(float(d) for d in decay)
        else:
            fields["scale"] = _number(mixer, "scale")
            if not fields["scale"] > 0:
                raise ConfigError(f"{where}: scale must be positive")
            if mixer.get("mask") is not None:
                fields["window"] = _positive_int(_mapping(mixer, "mask"), "size")
            if kind == "attention":
                fields["kv_heads"] = _positive_int(mixer, "kv_heads")
                if fields["heads"] % fields["kv_heads"]:
                    raise ConfigError(f"{where}: {fields['heads']} heads cannot be grouped over {fields['kv_heads']} kv_heads")
                if mixer.get("rot") is not None:
                    fields["rot"] = RotarySpec.from_dict(_mapping(mixer, "rot"), where, ("factor", "low", "high", "original"))
                    if fields["rot"].dims > fields["dim"]:
                        raise ConfigError(f"{where}: rot.dims {fields['rot'].dims} exceeds the head's dim {fields['dim']}")
            else:
                for key in ("rot_dim", "q_rank", "kv_rank"):
                    fields[key] = _positive_int(mixer, key)
                if mixer.get("rot") is not None:
                    fields["rot"] = RotarySpec.from_dict(_mapping(mixer, "rot"), where, ("factor", "original", "fast", "slow"))
                    if fields["rot"].dims > fields["rot_dim"]:
                        raise ConfigError(f"{where}: rot.dims {fields['rot'].dims} exceeds rot_dim {fields['rot_dim']}")
        mlp = data.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            fields["ff_kind"] = str(mlp.get("kind", "dense"))
            if fields["ff_kind"] != "dense":
                raise ConfigError(f"{where}: feed-forward kind {fields['ff_kind']!r} is not built (dense)")
            fields["ff"] = _positive_int(mlp, "ff")
        return cls(**fields)

    def to_dict(self) -> dict[str, Any]:
        mixer: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.kind == "lightning":
            mixer["decay"] = list(self.decay)
        else:
            mixer["scale"] = self.scale
            if self.window is not None:
                mixer["mask"] = {"size": self.window}
            if self.rot is not None:
                mixer["rot"] = self.rot.to_dict()
            if self.kind == "attention":
                mixer["kv_heads"] = self.kv_heads
            else:
                mixer.update(rot_dim=self.rot_dim, q_rank=self.q_rank, kv_rank=self.kv_rank)
        return {"type": self.kind, "mixer": mixer, "mlp": None if self.ff is None else {"kind": self.ff_kind, "ff": self.ff}}


@dataclass(frozen=True)
class FikeraxConfig:
    """Fikerax: a decoder whose layers are, in an order the configuration lists, lightning attention (a decayed linear
    recurrence), grouped-query attention (biases, partly rotated heads, q and k made unit vectors behind the rotation) and
    latent attention (one small cached row per token, a sink in the softmax), each over a sliding window where it attends,
    each with a gated feed-forward or none; RMS norms whose checkpoints hold the weight less one; the embedding scaled; and a span
    of layers ``loop_start .. loop_stop - 1`` that runs ``loop_times`` times in a row, the embedding added again before every
    pass but the first.

    ``config.json`` names the model by ``"architecture": "Fikerax"``.  Field names follow its keys.
    """

    architecture: ClassVar[str] = "Fikerax"

    vocab: int
    width: int
    layers: tuple[FikeraxLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers) or self.loop_times < 1:
            raise ConfigError(f"loop {self.loop_start} .. {self.loop_stop} x {self.loop_times} does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FikeraxConfig":
        layers = _require(data, "layers", list)
        eos = data.get("eos_token_id")
        loop = data.get("loop")
        if loop is not None and not isinstance(loop, dict):
            raise ConfigError("'loop' must be an object or null")
        embedding = data.get("embedding")
        return cls(
            vocab=_positive_int(data, "vocab"),
            width=_positive_int(data, "width"),
            layers=tuple(FikeraxLayer.from_dict(layer, index) for index, layer in enumerate(layers)),
            norm_eps=_number(_mapping(data, "norm"), "eps"),
            embedding_scale=1.0 if embedding is None else _number(_mapping(data, "embedding"), "scale"),
            loop_start=0 if loop is None else int(_require(loop, "start", int)),
            loop_stop=0 if loop is None else int(_require(loop, "stop", int)),
            loop_times=1 if loop is None else _positive_int(loop, "times"),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos)),
        )

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "layers": [layer.to_dict() for layer in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}, "norm": {"eps": self.norm_eps},
        }
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding is added before it) for every layer run: the layers before the loop, the loop's span
        ``loop_times`` times, the rest."""
        order = [(index, False) for index in range(self.loop_start)]
        for turn in range(self.loop_times):
            order += [(index, turn > 0 and index == self.loop_start) for index in range(self.loop_start, self.loop_stop)]
        order += [(index, False) for index in range(self.loop_stop, len(self.layers))]
        return order


# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ZemavikAttention:
    """The attending half of a ``parallel`` mixer: grouped-query attention without positions, scores times ``scale``, inside
    chunks of ``chunk`` positions (``None``: every earlier key), values of their own width."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "ZemavikAttention":
        heads, kv_heads = _positive_int(data, "heads"), _positive_int(data, "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads cannot be grouped over {kv_heads} kv_heads")
        mask = data.get("mask")
        return cls(heads, kv_heads, _positive_int(data, "dim"), _positive_int(data, "vdim"), _number(data, "scale"),
                   None if mask is None else _positive_int(_mapping(data, "mask"), "size"))

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.chunk is not None:
            data["mask"] = {"size": self.chunk}
        return data


@dataclass(frozen=True)
class ZemavikStateSpace:
    """The recurrent half of a ``parallel`` mixer: a state-space layer with one decay per head and step, ``heads`` heads of
    ``vdim`` channels, a state of ``state`` rows per head, input and output maps shared by the heads of a group."""

    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "ZemavikStateSpace":
        made = cls(*(_positive_int(data, key) for key in ("heads", "vdim", "state", "groups", "norm_groups", "conv")))
        if made.heads % made.groups:
            raise ConfigError(f"{where}: {made.heads} heads cannot be grouped over {made.groups} groups")
        if (made.heads * made.vdim) % made.norm_groups:
            raise ConfigError(f"{where}: {made.heads * made.vdim} channels cannot be normed in {made.norm_groups} equal parts")
        return made

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "norm_groups": self.norm_groups,
                "conv": self.conv}


@dataclass(frozen=True)
class ZemavikDelta:
    """A ``channel_delta`` mixer: the gated delta rule with a decay per head and key channel.  The decay's and the output
    gate's projections go through a narrow middle whose width the checkpoint's tensor shapes give (``decay_rank``,
    ``gate_rank``; a configuration that was written for random weights names them itself)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "ZemavikDelta":
        heads, kv_heads = _positive_int(data, "heads"), _positive_int(data, "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads cannot be grouped over {kv_heads} kv_heads")
        ranks = [None if data.get(key) is None else _positive_int(data, key) for key in ("decay_rank", "gate_rank")]
        return cls(heads, kv_heads, _positive_int(data, "dim"), _positive_int(data, "vdim"), _positive_int(data, "conv"), *ranks)

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            data["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            data["gate_rank"] = self.gate_rank
        return data


@dataclass(frozen=True)
class ZemavikFeedForward:
    """``dense``: one gated unit of inner width ``ff`` with biases.  ``moe``: ``experts`` gated units of inner width ``ff``
    without biases, of which a token uses ``top``."""

    kind: str
    ff: int
    experts: Optional[int] = None
    top: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "ZemavikFeedForward":
        kind = _require(data, "kind", str)
        if kind == "dense":
            return cls("dense", _positive_int(data, "ff"))
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r} (dense, moe)")
        router = _mapping(data, "router")
        experts, top = _positive_int(router, "experts"), _positive_int(router, "top")
        if top > experts:
            raise ConfigError(f"{where}: a token cannot use {top} of {experts} experts")
        return cls("moe", _positive_int(_mapping(data, "expert"), "ff"), experts, top)

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class ZemavikLayer:
    """One layer: a ``parallel`` mixer (``left`` attends, ``right`` is the state-space layer) or a ``channel_delta`` mixer, and
    its feed-forward, or none."""

    kind: str
    left: Optional[ZemavikAttention] = None
    right: Optional[ZemavikStateSpace] = None
    delta: Optional[ZemavikDelta] = None
    mlp: Optional[ZemavikFeedForward] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "ZemavikLayer":
        kind, where = _require(data, "type", str), f"layer {index}"
        mixer = _mapping(data, "mixer")
        mlp = data.get("mlp")
        if mlp is not None and not isinstance(mlp, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        feed_forward = None if mlp is None else ZemavikFeedForward.from_dict(mlp, where)
        if kind == "parallel":
            return cls(kind, left=ZemavikAttention.from_dict(_mapping(mixer, "left"), where), right=ZemavikStateSpace.from_dict(_mapping(mixer, "right"), where),
                       mlp=feed_forward)
        if kind == "channel_delta":
            return cls(kind, delta=ZemavikDelta.from_dict(mixer, where), mlp=feed_forward)
        raise ConfigError(f"{where}: unknown type {kind!r} (parallel, channel_delta)")

    def to_dict(self) -> dict[str, Any]:
        mixer = {"left": self.left.to_dict(), "right": self.right.to_dict()} if self.kind == "parallel" else self.delta.to_dict()
        return {"type": self.kind, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class ZemavikConfig:
    """Zemavik: a decoder with a learnt vector per position added to the embedding, whose layers are, in an order the
    configuration lists, two mixers side by side (chunked attention without positions and a state-space layer, the mean of
    their normed outputs) or a delta rule with channel-wise decay, each with a dense gated feed-forward with biases, a
    mixture of experts, or none; RMS norms; the head tied to the embedding; and a span of layers ``loop_start ..
    loop_stop - 1`` that runs ``loop_times`` times in a row, every pass entered through a map of the stream and the
    embedding output side by side (``loop`` absent: no span, no map).

    ``config.json`` names the model by ``"architecture": "Zemavik"``.  Field names follow its keys.
    """

    architecture: ClassVar[str] = "Zemavik"

    vocab: int
    width: int
    max_positions: int
    layers: tuple[ZemavikLayer, ...]
    norm_eps: float
    loop: Optional[tuple[int, int, int]] = None    # (start, stop, times)
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start <= stop <= len(self.layers) or times < 1:    # start = stop: an empty span, nothing runs twice
                raise ConfigError(f"loop {start} .. {stop} x {times} does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZemavikConfig":
        layers = _require(data, "layers", list)
        eos = data.get("eos_token_id")
        loop = data.get("loop")
        if loop is not None and not isinstance(loop, dict):
            raise ConfigError("'loop' must be an object or null")
        return cls(
            vocab=_positive_int(data, "vocab"),
            width=_positive_int(data, "width"),
            max_positions=_positive_int(data, "max_positions"),
            layers=tuple(ZemavikLayer.from_dict(layer, index) for index, layer in enumerate(layers)),
            norm_eps=_number(_mapping(data, "norm"), "eps"),
            loop=None if loop is None else (int(_require(loop, "start", int)), int(_require(loop, "stop", int)), _positive_int(loop, "times")),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos)),
        )

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
            "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.norm_eps},
        }
        if self.loop is not None:
            data["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether a pass of the loop starts with it) for every layer run: the layers before the loop, the loop's
        span ``times`` times, the rest."""
        if self.loop is None:
            return [(index, False) for index in range(len(self.layers))]
        start, stop, times = self.loop
        order = [(index, False) for index in range(start)]
        for _ in range(times):
            order += [(index, index == start) for index in range(start, stop)]
        return order + [(index, False) for index in range(stop, len(self.layers))]

    def with_checkpoint_sizes(self, shape_of) -> "ZemavikConfig":
        """The sizes that only tensor shapes give: ``shape_of(name)`` is a checkpoint tensor's shape, or ``None``."""
        from dataclasses import replace

        layers = []
        for index, layer in enumerate(self.layers):
            if layer.kind == "channel_delta":
                decay, gate = shape_of(f"l{index}.mix.a1"), shape_of(f"l{index}.mix.g1")
                layer = replace(layer, delta=replace(
                    layer.delta, decay_rank=layer.delta.decay_rank if decay is None else int(decay[0]),
                    gate_rank=layer.delta.gate_rank if gate is None else int(gate[0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))


# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RirusunAttention:
    """The attending half of a Rirusun ``parallel`` mixer: grouped-query attention without rotation, q and k RMS-normed over their
    whole rows, scores times ``scale`` plus a learnt bias by distance (a table of logarithmic buckets that ends at ``bias_max``),
    a sliding window of ``window`` positions (``None``: every earlier key) that always keeps the first ``keep_first`` positions,
    and a learnt sink per head in the softmax's denominator."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    window: Optional[int] = None
    keep_first: int = 0
    bias_rows: Optional[int] = None    # rows of the bias table: the checkpoint's tensor shape gives them (a configuration written for random weights names them)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RirusunAttention":
        heads, kv_heads = _positive_int(data, "heads"), _positive_int(data, "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads cannot be grouped over {kv_heads} kv_heads")
        mask = data.get("mask")
        window, keep = None, 0
        if mask is not None:
            mask = _mapping(data, "mask")
            window = _positive_int(mask, "size")
            keep = int(mask.get("keep_first") or 0)
            if keep < 0:
                raise ConfigError(f"{where}: mask.keep_first must not be negative")
        far = _number(data, "bias_max")    # a distance; whole in every model seen, but nothing in the table's rule needs that
        if not far > 0:
            raise ConfigError(f"{where}: bias_max must be positive")
        return cls(heads, kv_heads, _positive_int(data, "dim"), _positive_int(data, "vdim"), _number(data, "scale"), int(far) if far == int(far) else far,
                   window, keep, None if data.get("bias_rows") is None else _positive_int(data, "bias_rows"))

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                                "bias_max": self.bias_max}
        if self.window is not None:
            data["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.bias_rows is not None:
            data["bias_rows"] = self.bias_rows
        return data


@dataclass(frozen=True)
class RirusunRecurrent:
    """The recurrent half of a Rirusun ``parallel`` mixer: two branches of ``width`` channels, one through a causal convolution of
    ``conv`` taps and a gated linear recurrence whose gates are maps of ``blocks`` equal parts of the channels."""

    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RirusunRecurrent":
        made = cls(_positive_int(data, "width"), _positive_int(data, "blocks"), _positive_int(data, "conv"))
        if made.width % made.blocks:
            raise ConfigError(f"{where}: {made.width} channels cannot be cut into {made.blocks} equal parts")
        return made

    def to_dict(self) -> dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class RirusunFeedForward:
    """A mixture of ``experts`` ungated feed-forwards of inner width ``ff`` of which a token uses ``top``, chosen by sigmoid scores
    with a correction among the experts of the ``groups_keep`` best of ``groups`` groups, plus (``shared_ff``) one expert that every
    token goes through behind a sigmoid gate."""

    ff: int
    experts: int
    top: int
    groups: Optional[int] = None
    groups_keep: Optional[int] = None
    shared_ff: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RirusunFeedForward":
        kind = _require(data, "kind", str)
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r} (moe)")
        router = _mapping(data, "router")
        experts, top = _positive_int(router, "experts"), _positive_int(router, "top")
        groups = keep = None
        if router.get("groups") is not None:
            groups, keep = _positive_int(_mapping(router, "groups"), "count"), _positive_int(_mapping(router, "groups"), "keep")
            if experts % groups or keep > groups:
                raise ConfigError(f"{where}: {experts} experts in {groups} groups of which {keep} are kept")
        if top > (experts if groups is None else keep * (experts // groups)):
            raise ConfigError(f"{where}: a token cannot use {top} of the experts it may choose from")
        shared = data.get("shared")
        return cls(_positive_int(_mapping(data, "expert"), "ff"), experts, top, groups, keep,
                   None if shared is None else _positive_int(_mapping(data, "shared"), "ff"))

    def to_dict(self) -> dict[str, Any]:
        router: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups, "keep": self.groups_keep}
        data: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff is not None:
            data["shared"] = {"ff": self.shared_ff}
        return data


@dataclass(frozen=True)
class RirusunLayer:
    """One layer: its mixer - ``parallel`` (``left`` attends, ``right`` is the gated linear recurrence, their outputs added with a
    factor each), ``mlstm`` (a matrix memory per head; ``memory`` = (heads, dim, vdim, gate_cap)) or ``latent_attention`` (``latent``
    holds its sizes as a :class:`FikeraxLayer` does) - and its feed-forward, or none."""

    kind: str
    left: Optional[RirusunAttention] = None
    right: Optional[RirusunRecurrent] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    memory: Optional[tuple] = None
    latent: Optional[tuple] = None      # (heads, dim, rot_dim, vdim, kv_rank, scale, RotarySpec or None)
    mlp: Optional[RirusunFeedForward] = None

    KINDS: ClassVar[tuple[str, ...]] = ("parallel", "mlstm", "latent_attention")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "RirusunLayer":
        kind, where = _require(data, "type", str), f"layer {index}"
        if kind not in cls.KINDS:
            raise ConfigError(f"{where}: unknown type {kind!r} ({', '.join(cls.KINDS)})")
        mixer = _mapping(data, "mixer")
        mlp = data.get("mlp")
        if mlp is not None and not isinstance(mlp, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        feed_forward = None if mlp is None else RirusunFeedForward.from_dict(mlp, where)
        if kind == "parallel":
            return cls(kind, left=RirusunAttention.from_dict(_mapping(mixer, "left"), where), right=RirusunRecurrent.from_dict(_mapping(mixer, "right"), where),
                       left_scale=_number(mixer, "left_scale"), right_scale=_number(mixer, "right_scale"), mlp=feed_forward)
        if kind == "mlstm":
            cap = _number(mixer, "gate_cap")
            if not cap > 0:
                raise ConfigError(f"{where}: gate_cap must be positive")
            return cls(kind, memory=(_positive_int(mixer, "heads"), _positive_int(mixer, "dim"), _positive_int(mixer, "vdim"), cap), mlp=feed_forward)
        rot = None
        rot_dim = _positive_int(mixer, "rot_dim")
        if mixer.get("rot") is not None:
            rot = RotarySpec.from_dict(_mapping(mixer, "rot"), where, ("factor", "original", "fast", "slow"))
            if rot.dims > rot_dim:
                raise ConfigError(f"{where}: rot.dims {rot.dims} exceeds rot_dim {rot_dim}")
        return cls(kind, latent=(_positive_int(mixer, "heads"), _positive_int(mixer, "dim"), rot_dim, _positive_int(mixer, "vdim"),
                                 _positive_int(mixer, "kv_rank"), _number(mixer, "scale"), rot), mlp=feed_forward)

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "parallel":
            mixer: dict[str, Any] = {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(), "right_scale": self.right_scale}
        elif self.kind == "mlstm":
            mixer = dict(zip(("heads", "dim", "vdim", "gate_cap"), self.memory))
        else:
            mixer = dict(zip(("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"), self.latent[:6]))
            if self.latent[6] is not None:
                mixer["rot"] = self.latent[6].to_dict()
        return {"type": self.kind, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class RirusunConfig:
    """Rirusun: a decoder whose layers each read one norm - a scaled tanh with weight and bias instead of statistics - and add
    mixer and feed-forward to the stream side by side.  The mixers are, in an order the configuration lists, windowed attention
    with kept first tokens, distance bias and sink beside a gated linear recurrence; a matrix memory with exponential gates; and
    latent attention with YaRN-scaled rotation.  The feed-forward is a mixture of experts with grouped sigmoid routing and a
    gated shared expert.  The embedding is scaled, the head is a tensor of its own, and a span of layers ``loop`` = (start, stop,
    times) runs several times in a row, each pass with caches of its own and nothing between the passes.

    ``config.json`` names the model by ``"architecture": "Rirusun"``.  Field names follow its keys.
    """

    architecture: ClassVar[str] = "Rirusun"

    vocab: int
    width: int
    layers: tuple[RirusunLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    loop: Optional[tuple[int, int, int]] = None
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start <= stop <= len(self.layers) or times < 1:
                raise ConfigError(f"loop {start} .. {stop} x {times} does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RirusunConfig":
        layers = _require(data, "layers", list)
        eos = data.get("eos_token_id")
        loop = data.get("loop")
        if loop is not None and not isinstance(loop, dict):
            raise ConfigError("'loop' must be an object or null")
        return cls(
            vocab=_positive_int(data, "vocab"),
            width=_positive_int(data, "width"),
            layers=tuple(RirusunLayer.from_dict(layer, index) for index, layer in enumerate(layers)),
            norm_eps=_number(_mapping(data, "norm"), "eps"),
            embedding_scale=1.0 if data.get("embedding") is None else _number(_mapping(data, "embedding"), "scale"),
            loop=None if loop is None else (int(_require(loop, "start", int)), int(_require(loop, "stop", int)), _positive_int(loop, "times")),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos)),
        )

    def to_dict(self) -> dict[str, Any]:
        data: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
            "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.norm_eps},
        }
        if self.loop is not None:
            data["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    def run_order(self) -> list[int]:
        """The layer of every run: the layers before the loop, the loop's span ``times`` times, the rest."""
        if self.loop is None:
            return list(range(len(self.layers)))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, len(self.layers)))

    def with_checkpoint_sizes(self, shape_of) -> "RirusunConfig":
        """The sizes that only tensor shapes give: ``shape_of(name)`` is a checkpoint tensor's shape, or ``None``."""
        from dataclasses import replace

        layers = []
        for index, layer in enumerate(self.layers):
            if layer.kind == "parallel":
                table = shape_of(f"l{index}.mix.left.rel")
                if table is not None:
                    layer = replace(layer, left=replace(layer.left, bias_rows=int(table[0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))
