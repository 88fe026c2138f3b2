"""Typed configuration of the Medolorn decoder, read from its ``config.json``.

The document is nested: ``vocab`` and ``width`` at the top, ``norm.eps``, ``canon.taps`` (the
taps of the causal filter in front of every mixer), a list ``layers`` whose entries name the
mixer (``type``: ``delta``, ``latent_attention`` or ``retention``), its sizes (``mixer``) and
the feed-forward (``mlp``, null for none; ``kind`` ``moe`` with ``expert.ff`` and ``router.
{experts, top, scale}``), and an optional ``loop`` (``start``, ``stop``, ``times``): layers
``start`` to ``stop - 1`` run ``times`` times in a row with the same weights, every run with
its own cache and state.  Every size and constant is read from the document; layers may
differ from one another in every one of them.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .keys import COUNT, REAL, TEXT, Key, read_keys
from .rekasun import FACTOR, LoopConfig, _object, _whole

ARCHITECTURE = "Medolorn"
DEFAULT_MAX_POSITIONS = 1 << 17


def _rotation(document: Mapping[str, Any], where: str, most: int) -> Tuple[float, int]:
    rot = _object(document, "rot", where)
    base = read_keys(rot, (Key("base", REAL),), where + "rot.")["base"]
    dims = rot.get("dims")
    if not (_whole(dims) and dims % 2 == 0 and dims <= most):
        raise ConfigError(f"config field '{where}rot.dims' must be even and at most {most}")
    return base, int(dims)


@dataclasses.dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int            # query/key heads; value head h reads h // (heads / kv_heads)
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    conv: int                # taps of the causal filter on q, k and v

    KEYS = (Key("heads", COUNT), Key("kv_heads", COUNT), Key("dim", COUNT), Key("vdim", COUNT),
            Key("conv", COUNT, default=1))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "DeltaMixerConfig":
        values = read_keys(document, cls.KEYS, where)
        if values["heads"] % values["kv_heads"]:
            raise ConfigError(f"config field '{where}heads' must be a multiple of "
                              f"'{where}kv_heads'")
        return cls(**values)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated coordinates of a query / key head
    rot_dim: int             # rotated coordinates behind them
    vdim: int
    kv_rank: int             # the cached latent
    q_rank: int              # the queries' latent
    scale: float
    window: int              # a position sees the last `window` positions, itself included
    rot_base: float
    rot_dims: int            # leading rotated coordinates that are turned

    KEYS = (Key("heads", COUNT), Key("dim", COUNT), Key("rot_dim", COUNT), Key("vdim", COUNT),
            Key("kv_rank", COUNT), Key("q_rank", COUNT), Key("scale", REAL))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        values = read_keys(document, cls.KEYS, where)
        size = _object(document, "mask", where).get("size")
        if not (_whole(size) and size > 0):
            raise ConfigError(f"config field '{where}mask.size' must be a positive integer")
        base, dims = _rotation(document, where, values["rot_dim"])
        return cls(window=int(size), rot_base=base, rot_dims=dims, **values)

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
                "mask": {"size": self.window},
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclasses.dataclass(frozen=True)
class RetentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]     # one constant per head
    rot_base: float
    rot_dims: int

    KEYS = (Key("heads", COUNT), Key("dim", COUNT), Key("vdim", COUNT))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "RetentionMixerConfig":
        values = read_keys(document, cls.KEYS, where)
        decay = document.get("decay")
        if not (isinstance(decay, list) and len(decay) == values["heads"] and all(
                isinstance(d, (int, float)) and not isinstance(d, bool) and math.isfinite(d)
                for d in decay)):
            raise ConfigError(f"config field '{where}decay' must list one number per head")
        base, dims = _rotation(document, where, values["dim"])
        return cls(decay=tuple(float(d) for d in decay), rot_base=base, rot_dims=dims, **values)

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay),
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


# one configuration class per value of a layer's ``type``
MIXER_CONFIGS = {"delta": DeltaMixerConfig, "latent_attention": LatentAttentionConfig,
                 "retention": RetentionMixerConfig}


@dataclasses.dataclass(frozen=True)
class RoutedMlpConfig:
    ff: int                  # of one expert
    experts: int
    top: int
    scale: float
    kind: str = "moe"

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "RoutedMlpConfig":
        kind = read_keys(document, (Key("kind", TEXT, default="moe"),), where)["kind"]
        if kind != "moe":
            raise ConfigError(f"config field '{where}kind' is {kind!r}; this design's "
                              "feed-forwards are 'moe'")
        ff = read_keys(_object(document, "expert", where), (Key("ff", COUNT),),
                       where + "expert.")["ff"]
        router = read_keys(_object(document, "router", where),
                           (Key("experts", COUNT), Key("top", COUNT),
                            Key("scale", FACTOR, default=1.0)), where + "router.")
        if router["top"] > router["experts"]:
            raise ConfigError(f"config field '{where}router.top' is more than "
                              f"'{where}router.experts'")
        return cls(ff=ff, kind=kind, **router)

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": self.kind, "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "scale": self.scale}}


@dataclasses.dataclass(frozen=True)
class MedolornLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[RoutedMlpConfig]

    @classmethod
    def from_dict(cls, document: Any, index: int) -> "MedolornLayerConfig":
        where = f"layers[{index}]."
        if not isinstance(document, dict):
            raise ConfigError(f"config field 'layers[{index}]' must be an object")
        kind = document.get("type")
        if kind not in MIXER_CONFIGS:
            raise ConfigError(f"config field '{where}type' is {kind!r}; known: "
                              + ", ".join(sorted(MIXER_CONFIGS)))
        mixer = MIXER_CONFIGS[kind].from_dict(_object(document, "mixer", where), where + "mixer.")
        mlp = document.get("mlp")
        if mlp is not None and not isinstance(mlp, dict):
            raise ConfigError(f"config field '{where}mlp' must be an object or null")
        return cls(kind, mixer,
                   None if mlp is None else RoutedMlpConfig.from_dict(mlp, where + "mlp."))

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclasses.dataclass(frozen=True)
class MedolornConfig:
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    layers: Tuple[MedolornLayerConfig, ...]
    loop: Optional[LoopConfig] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("config field 'layers' must name at least one layer")
        if self.loop is not None:
            loop = self.loop
            if not 0 <= loop.start < loop.stop <= len(self.layers) or loop.times < 1:
                raise ConfigError(f"config field 'loop' ({loop.start}, {loop.stop}, {loop.times}) "
                                  f"does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "MedolornConfig":
        values = read_keys(document, (Key("vocab", COUNT), Key("width", COUNT),
                                      Key("max_positions", COUNT, default=DEFAULT_MAX_POSITIONS)))
        eps = read_keys(_object(document, "norm"), (Key("eps", REAL),), "norm.")["eps"]
        taps = read_keys(_object(document, "canon"), (Key("taps", COUNT),), "canon.")["taps"]
        layers = document.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a list of layers")
        loop = document.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not all(_whole(loop.get(k))
                                                     for k in ("start", "stop", "times")):
                raise ConfigError("config field 'loop' must give whole numbers start, stop, times")
            loop = LoopConfig(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        return cls(vocab=values["vocab"], width=values["width"], norm_eps=eps, canon_taps=taps,
                   loop=loop, max_positions=values["max_positions"],
                   layers=tuple(MedolornLayerConfig.from_dict(layer, index)
                                for index, layer in enumerate(layers)))

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.loop is not None:
            document["loop"] = dataclasses.asdict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            document["max_positions"] = self.max_positions
        return document

    @staticmethod
    def random_scale(name: str, shape: Tuple[int, ...]):
        """What a model with random weights holds in its vectors and small tables (None: ones):
        norm weights stored around zero stay zero, gates' biases too, learned decays run at rates
        from 1/16 to 1 with steps around 0.1, filters pass the token itself, the steps added
        before the passes of a loop are small."""
        import torch
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm2") or name in ("final.norm", "embed.norm") or leaf == "b":
            return 0.0
        if leaf == "A_log":
            return torch.linspace(math.log(1.0 / 16.0), 0.0, shape[0])
        if leaf == "dt_bias":
            return -2.25
        if leaf == "conv":
            taps = torch.full(shape, 0.1)
            taps[:, -1] = 1.0
            return taps
        if leaf == "canon1":
            return 0.1
        if name == "loop.step":
            return 0.02
        return None

    def layer_runs(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """The layers in the order they run, as ``(layer, pass)``: ``pass`` is the number of the
        pass through the loop that starts with this run, None for every other run."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((layer, None) for layer in range(count))
        loop = self.loop
        runs = [(layer, None) for layer in range(loop.start)]
        for turn in range(loop.times):
            runs.extend((layer, turn if layer == loop.start else None)
                        for layer in range(loop.start, loop.stop))
        runs.extend((layer, None) for layer in range(loop.stop, count))
        return tuple(runs)
