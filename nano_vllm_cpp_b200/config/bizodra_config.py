"""Typed view of a Bizodra ``config.json``.

The file lists its layers one by one: ``layers[i] = {"type", "mixer", "mlp"}``.  ``type`` names the mixer
(``mlstm``: a matrix LSTM; ``parallel``: softmax attention with a sink beside a gated delta rule; a numeric suffix,
as in ``mlstm_2``, marks a further set of sizes of the same kind),
``mixer`` holds the mixer's sizes and constants, ``mlp`` the feed-forward (``{"kind": "dense", "ff": n}``) or null.
Top level: ``vocab``, ``width``, ``norm.eps``, ``token_side.dim`` (the per-layer token input; absent: none).
Every size and constant is read from the file; a missing key, a wrong type or an unknown kind is an error that
names the key.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .fields import need as _need, positive as _positive
from .model_config import ConfigError

ARCHITECTURE = "Bizodra"


@dataclass
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[dict] = None        # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RotaryConfig":
        sc = d.get("scaling")
        scaling = None
        if sc is not None:
            scaling = {k: _need(sc, k, float, where + ".scaling") for k in ("factor", "original", "fast", "slow")}
            if scaling["factor"] <= 0 or scaling["original"] <= 0 or scaling["fast"] <= 0 or scaling["slow"] <= 0:
                raise ConfigError(f"config.json: the numbers of '{where}.scaling' must be positive")
        out = cls(_need(d, "dims", int, where), _need(d, "base", float, where), scaling)
        if out.dims < 0 or out.dims % 2:
            raise ConfigError(f"config.json: '{where}.dims' must be even and not negative")
        if out.base <= 0 or out.base == 1.0:
            raise ConfigError(f"config.json: '{where}.base' must be positive and not 1")
        return out


@dataclass
class MatrixLstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MatrixLstmConfig":
        out = cls(_positive(_need(d, "heads", int, where), where + ".heads"),
                  _positive(_need(d, "dim", int, where), where + ".dim"),
                  _positive(_need(d, "vdim", int, where), where + ".vdim"), _need(d, "gate_cap", float, where))
        if out.gate_cap <= 0:
            raise ConfigError(f"config.json: '{where}.gate_cap' must be positive")
        return out


@dataclass
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "SinkAttentionConfig":
        out = cls(_positive(_need(d, "heads", int, where), where + ".heads"),
                  _positive(_need(d, "kv_heads", int, where), where + ".kv_heads"),
                  _positive(_need(d, "dim", int, where), where + ".dim"),
                  _positive(_need(d, "vdim", int, where), where + ".vdim"), _need(d, "scale", float, where),
                  RotaryConfig.from_dict(d["rot"], where + ".rot") if d.get("rot") is not None
                  else RotaryConfig(0, 10000.0, None))          # no 'rot': nothing is turned
        if out.heads % out.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        if out.rot.dims > out.dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' cannot exceed '{where}.dim'")
        return out


@dataclass
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "GatedDeltaConfig":
        out = cls(_positive(_need(d, "heads", int, where), where + ".heads"),
                  _positive(_need(d, "kv_heads", int, where), where + ".kv_heads"),
                  _positive(_need(d, "dim", int, where), where + ".dim"),
                  _positive(_need(d, "vdim", int, where), where + ".vdim"),
                  _positive(_need(d, "conv", int, where), where + ".conv"))
        if out.heads % out.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        return out


@dataclass
class ParallelConfig:
    left: SinkAttentionConfig
    right: GatedDeltaConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ParallelConfig":
        return cls(SinkAttentionConfig.from_dict(_need(d, "left", dict, where), where + ".left"),
                   GatedDeltaConfig.from_dict(_need(d, "right", dict, where), where + ".right"))


MIXER_KINDS = {"mlstm": MatrixLstmConfig, "parallel": ParallelConfig}


def mixer_kind(layer_type: str):
    """The mixer a layer's ``type`` names.  A file numbers the second, third ... set of sizes of a kind
    (``mlstm_2``): the kind is the name without that suffix."""
    base = layer_type
    head, sep, tail = layer_type.rpartition("_")
    if sep and tail.isdigit() and head:
        base = head
    return MIXER_KINDS.get(base)


@dataclass
class BizodraLayer:
    type: str
    mixer: Any
    mlp_kind: Optional[str]           # None: the layer has no feed-forward
    mlp_ff: int = 0


@dataclass
class BizodraConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    eps: float
    side_dim: int                     # 0: no per-layer token input
    layers: list = field(default_factory=list)
    raw: dict = field(default_factory=dict)
    eos_token_id: int = -1

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: dict) -> "BizodraConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            typ = _need(L, "type", str, where)
            kind = mixer_kind(typ)
            if kind is None:
                raise ConfigError(f"config.json: '{where}.type' is {typ!r}; known: {', '.join(sorted(MIXER_KINDS))} "
                                  "(with a numeric suffix for further sets of sizes, as in mlstm_2)")
            mixer = kind.from_dict(_need(L, "mixer", dict, where), where + ".mixer")
            mlp = L.get("mlp")
            mlp_kind, ff = None, 0
            if mlp is not None:
                mlp_kind = _need(mlp, "kind", str, where + ".mlp")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: '{where}.mlp.kind' is {mlp_kind!r}; known: dense")
                ff = _positive(_need(mlp, "ff", int, where + ".mlp"), where + ".mlp.ff")
            layers.append(BizodraLayer(typ, mixer, mlp_kind, ff))
        side = d.get("token_side")
        side_dim = 0
        if side is not None:
            side_dim = _positive(_need(side, "dim", int, "token_side"), "token_side.dim")
        eps = _need(_need(d, "norm", dict, ""), "eps", float, "norm")
        if eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        eos = d.get("eos_token_id", -1)
        return cls(architecture=d.get("architecture", ARCHITECTURE),
                   vocab_size=_positive(_need(d, "vocab", int, ""), "vocab"),
                   hidden_size=_positive(_need(d, "width", int, ""), "width"),
                   eps=eps, side_dim=side_dim, layers=layers, raw=dict(d),
                   eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1)

    def to_dict(self) -> dict:
        return dict(self.raw)
