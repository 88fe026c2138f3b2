"""Typed configuration of the Rorovik decoder, read from its ``config.json``.

The document is nested: ``vocab`` and ``width`` at the top, ``norm.eps``, ``residual_mult`` (the
factor on every sublayer's normed result), ``token_side.dim`` (the width of the per-layer piece of
the table of token inputs; the key may be left out: no such input), and a list ``layers`` whose
entries name the mixer (``type``: ``attention`` or ``latent_attention``), its sizes (``mixer``)
and the feed-forward (``mlp``, null for none; ``kind`` ``dense`` with ``ff``, or ``moe`` with
``expert.{ff, limit}`` and ``router.{experts, identity, top}``).  Every size and constant is read
from the document; layers may differ from one another in every one of them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .keys import COUNT, FLAG, REAL, TEXT, Key, read_keys
from .rekasun import FACTOR, _object, _whole

ARCHITECTURE = "Rorovik"
DEFAULT_MAX_POSITIONS = 1 << 17


def _optional_object(document: Mapping[str, Any], name: str, where: str):
    value = document.get(name)
    if value is not None and not isinstance(value, dict):
        raise ConfigError(f"config field {where + name!r} must be an object or null")
    return value


@dataclasses.dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int            # query head h reads key/value head h // (heads / kv_heads)
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float
    window: Optional[int]    # a position sees the last `window` positions, itself included
    temp_coef: Optional[float]   # the query times 1 + coef ln(floor((p + 1) / every) + 1)
    temp_every: Optional[int]
    v_mix: bool              # values blended with the first such layer's

    KEYS = (Key("heads", COUNT), Key("kv_heads", COUNT, default=None), Key("dim", COUNT),
            Key("vdim", COUNT, default=None), Key("scale", REAL),
            Key("v_mix", FLAG, default=False))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "WindowedAttentionConfig":
        values = read_keys(document, cls.KEYS, where)
        values["kv_heads"] = values["kv_heads"] or values["heads"]
        values["vdim"] = values["vdim"] or values["dim"]
        if values["heads"] % values["kv_heads"]:
            raise ConfigError(f"config field '{where}heads' must be a multiple of "
                              f"'{where}kv_heads'")
        window = None
        mask = _optional_object(document, "mask", where)
        if mask is not None:
            window = read_keys(mask, (Key("size", COUNT),), where + "mask.")["size"]
        coef = every = None
        temp = _optional_object(document, "q_temp", where)
        if temp is not None:
            read = read_keys(temp, (Key("coef", FACTOR), Key("every", COUNT)), where + "q_temp.")
            coef, every = read["coef"], read["every"]
        return cls(window=window, temp_coef=coef, temp_every=every, **values)

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {
            "heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
            "scale": self.scale, "v_mix": self.v_mix}
        if self.window is not None:
            document["mask"] = {"size": self.window}
        if self.temp_every is not None:
            document["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return document


@dataclasses.dataclass(frozen=True)
class RotaryScalingConfig:
    factor: float
    original: int
    fast: float
    slow: float

    KEYS = (Key("factor", REAL), Key("original", COUNT), Key("fast", REAL), Key("slow", REAL))


@dataclasses.dataclass(frozen=True)
class CausalLatentAttentionConfig:
    heads: int
    dim: int                 # unrotated coordinates of a query / key head
    rot_dim: int             # rotated coordinates behind them
    vdim: int
    kv_rank: int             # the cached latent
    q_rank: int              # the queries' latent
    scale: float
    rot_base: float
    rot_dims: int            # leading rotated coordinates that are turned
    scaling: Optional[RotaryScalingConfig]

    KEYS = (Key("heads", COUNT), Key("dim", COUNT), Key("rot_dim", COUNT), Key("vdim", COUNT),
            Key("kv_rank", COUNT), Key("q_rank", COUNT), Key("scale", REAL))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "CausalLatentAttentionConfig":
        values = read_keys(document, cls.KEYS, where)
        rot = _object(document, "rot", where)
        base = read_keys(rot, (Key("base", REAL),), where + "rot.")["base"]
        dims = rot.get("dims", values["rot_dim"])
        if not (_whole(dims) and dims % 2 == 0 and dims <= values["rot_dim"]):
            raise ConfigError(f"config field '{where}rot.dims' must be even and at most "
                              f"{values['rot_dim']}")
        scaling = _optional_object(rot, "scaling", where + "rot.")
        if scaling is not None:
            scaling = RotaryScalingConfig(**read_keys(scaling, RotaryScalingConfig.KEYS,
                                                      where + "rot.scaling."))
            if base <= 1.0:
                raise ConfigError(f"config field '{where}rot.base' must exceed 1 with scaling")
        return cls(rot_base=base, rot_dims=int(dims), scaling=scaling, **values)

    def to_dict(self) -> Dict[str, Any]:
        rot: Dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = dataclasses.asdict(self.scaling)
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "rot": rot}


# one configuration class per value of a layer's ``type``
MIXER_CONFIGS = {"attention": WindowedAttentionConfig,
                 "latent_attention": CausalLatentAttentionConfig}


@dataclasses.dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                # dense | moe
    ff: int                  # of the dense layer, or of one expert
    experts: int = 0
    identity: int = 0        # router outputs behind the experts that return their input
    top: int = 0
    limit: float = 0.0       # the experts' clamp

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = read_keys(document, (Key("kind", TEXT),), where)["kind"]
        if kind == "dense":
            return cls(kind=kind, ff=read_keys(document, (Key("ff", COUNT),), where)["ff"])
        if kind != "moe":
            raise ConfigError(f"config field '{where}kind' is {kind!r}; known: dense, moe")
        expert = read_keys(_object(document, "expert", where),
                           (Key("ff", COUNT), Key("limit", REAL)), where + "expert.")
        router = _object(document, "router", where)
        counts = read_keys(router, (Key("experts", COUNT), Key("top", COUNT)), where + "router.")
        identity = router.get("identity", 0)
        if not _whole(identity):
            raise ConfigError(f"config field '{where}router.identity' must be a whole number")
        if counts["top"] > counts["experts"] + identity:
            raise ConfigError(f"config field '{where}router.top' is more than the router's "
                              "outputs")
        return cls(kind=kind, ff=expert["ff"], limit=expert["limit"], experts=counts["experts"],
                   identity=int(identity), top=counts["top"])

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}


@dataclasses.dataclass(frozen=True)
class RorovikLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]

    @classmethod
    def from_dict(cls, document: Any, index: int) -> "RorovikLayerConfig":
        where = f"layers[{index}]."
        if not isinstance(document, dict):
            raise ConfigError(f"config field 'layers[{index}]' must be an object")
        kind = document.get("type")
        if kind not in MIXER_CONFIGS:
            raise ConfigError(f"config field '{where}type' is {kind!r}; known: "
                              + ", ".join(sorted(MIXER_CONFIGS)))
        mixer = MIXER_CONFIGS[kind].from_dict(_object(document, "mixer", where), where + "mixer.")
        mlp = _optional_object(document, "mlp", where)
        return cls(kind, mixer,
                   None if mlp is None else FeedForwardConfig.from_dict(mlp, where + "mlp."))

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclasses.dataclass(frozen=True)
class RorovikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    side_dim: Optional[int]          # None: no per-layer token input
    layers: Tuple[RorovikLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("config field 'layers' must name at least one layer")
        mixing = [layer.mixer.kv_heads * layer.mixer.vdim for layer in self.layers
                  if layer.type == "attention" and layer.mixer.v_mix]
        if len(set(mixing)) > 1:
            raise ConfigError("layers that mix values agree in kv_heads * vdim")

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "RorovikConfig":
        values = read_keys(document, (Key("vocab", COUNT), Key("width", COUNT),
                                      Key("residual_mult", FACTOR, default=1.0),
                                      Key("max_positions", COUNT, default=DEFAULT_MAX_POSITIONS)))
        eps = read_keys(_object(document, "norm"), (Key("eps", REAL),), "norm.")["eps"]
        side = _optional_object(document, "token_side", "")
        side_dim = None if side is None else read_keys(side, (Key("dim", COUNT),),
                                                       "token_side.")["dim"]
        layers = document.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a list of layers")
        return cls(vocab=values["vocab"], width=values["width"], norm_eps=eps,
                   residual_mult=values["residual_mult"], side_dim=side_dim,
                   max_positions=values["max_positions"],
                   layers=tuple(RorovikLayerConfig.from_dict(layer, index)
                                for index, layer in enumerate(layers)))

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.side_dim is not None:
            document["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            document["max_positions"] = self.max_positions
        return document

    @staticmethod
    def random_scale(name: str, shape: Tuple[int, ...]):
        """What a model with random weights holds in its vectors (None: ones): biases, sinks and
        the router's corrections are zero, the values' blend a half."""
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("b", "sink", "correction"):
            return 0.0
        if leaf == "vmix":
            return 0.5
        return None
