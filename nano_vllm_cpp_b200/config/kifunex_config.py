"""Typed view of a Kifunex ``config.json``.

The file lists its layers one by one: ``layers[i] = {"type", "mixer", "mlp"}`` and optionally ``"weights_of": j``
(the layer has no tensors of its own and runs with layer j's, keeping a cache entry of its own).  ``type`` names
the mixer (``attention``; a numeric suffix, as in ``attention_2``, marks a further set of sizes of the same kind),
``mixer`` holds its sizes and constants (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``,
``rot.dims``, ``rot.base``, ``rot.scaling.{factor, low, high, original}``), ``mlp`` the feed-forward
(``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}, "shared": {"ff"}}``) or null.
Top level: ``vocab``, ``width``, ``streams``, ``norm.eps``, ``logit_scale``, ``logit_softcap``.
Every size and constant is read from the file; a missing key, a wrong type or an unknown kind is an error that
names the key.  Parts that a file leaves out (``mask``, ``rot``, ``rot.scaling``, ``shared``, ``logit_softcap``) are
switched off.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .fields import need as _need, positive as _positive
from .model_config import ConfigError

ARCHITECTURE = "Kifunex"


@dataclass
class WaveScaling:
    factor: float
    low: float
    high: float
    original: float

    def as_dict(self) -> dict:
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


@dataclass
class KeyValueAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                       # 0: every earlier position is seen
    rot_dims: int                     # 0: nothing is turned
    rot_base: float = 10000.0
    rot_scaling: Optional[WaveScaling] = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "KeyValueAttentionConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        kv = _positive(_need(d, "kv_heads", int, where), where + ".kv_heads")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        if heads % kv:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        if vdim != dim:
            raise ConfigError(f"config.json: '{where}.vdim' must equal '{where}.dim' (the values are the keys)")
        window = 0
        if d.get("mask") is not None:
            window = _positive(_need(d["mask"], "size", int, where + ".mask"), where + ".mask.size")
        dims, base, scaling = 0, 10000.0, None
        rot = d.get("rot")
        if rot is not None:
            dims = _need(rot, "dims", int, where + ".rot")
            if dims < 0 or dims % 2 or dims > dim:
                raise ConfigError(f"config.json: '{where}.rot.dims' must be even, not negative and at most '{where}.dim'")
            base = _need(rot, "base", float, where + ".rot")
            if base <= 0 or base == 1.0:
                raise ConfigError(f"config.json: '{where}.rot.base' must be positive and not 1")
            sc = rot.get("scaling") if isinstance(rot, dict) else None
            if sc is not None:
                w = where + ".rot.scaling"
                scaling = WaveScaling(*(_need(sc, k, float, w) for k in ("factor", "low", "high", "original")))
                if scaling.factor <= 0 or scaling.original <= 0 or scaling.low <= 0 or scaling.high <= 0:
                    raise ConfigError(f"config.json: the numbers of '{w}' must be positive")
                if scaling.low == scaling.high:
                    raise ConfigError(f"config.json: '{w}.low' and '{w}.high' must differ")
        return cls(heads, kv, dim, vdim, _need(d, "scale", float, where), window, dims, base, scaling)


@dataclass
class ScoredMoeConfig:
    experts: int
    top: int
    route_scale: float
    ff: int
    shared_ff: int                    # 0: no shared expert

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ScoredMoeConfig":
        r = _need(d, "router", dict, where)
        experts = _positive(_need(r, "experts", int, where + ".router"), where + ".router.experts")
        top = _positive(_need(r, "top", int, where + ".router"), where + ".router.top")
        if top > experts:
            raise ConfigError(f"config.json: '{where}.router.top' cannot exceed '{where}.router.experts'")
        scale = _need(r, "scale", float, where + ".router", default=1.0, required=False)
        ff = _positive(_need(_need(d, "expert", dict, where), "ff", int, where + ".expert"), where + ".expert.ff")
        shared = 0
        if d.get("shared") is not None:
            shared = _positive(_need(d["shared"], "ff", int, where + ".shared"), where + ".shared.ff")
        return cls(experts, top, scale, ff, shared)


MIXER_KINDS = {"attention": KeyValueAttentionConfig}
MLP_KINDS = {"moe": ScoredMoeConfig}


def _kind_of(name: str, table: dict):
    head, sep, tail = name.rpartition("_")
    if sep and tail.isdigit() and head:
        name = head
    return table.get(name)


@dataclass
class KifunexLayer:
    type: str
    mixer: KeyValueAttentionConfig
    mlp: Optional[ScoredMoeConfig]    # None: the layer has no feed-forward
    weights_of: Optional[int] = None  # the layer whose tensors this one runs with


@dataclass
class KifunexConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    streams: int
    eps: float
    logit_scale: float
    logit_softcap: float              # 0: no cap
    layers: list = field(default_factory=list)
    raw: dict = field(default_factory=dict)
    eos_token_id: int = -1

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def weight_owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with (itself, unless it names another)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: 'layers[{i}].weights_of' runs in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @classmethod
    def from_dict(cls, d: dict) -> "KifunexConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            typ = _need(L, "type", str, where)
            kind = _kind_of(typ, MIXER_KINDS)
            if kind is None:
                raise ConfigError(f"config.json: '{where}.type' is {typ!r}; known: {', '.join(sorted(MIXER_KINDS))} "
                                  "(with a numeric suffix for further sets of sizes)")
            mixer = kind.from_dict(_need(L, "mixer", dict, where), where + ".mixer")
            mlp = None
            if L.get("mlp") is not None:
                mk = _need(L["mlp"], "kind", str, where + ".mlp")
                mlp_kind = _kind_of(mk, MLP_KINDS)
                if mlp_kind is None:
                    raise ConfigError(f"config.json: '{where}.mlp.kind' is {mk!r}; known: {', '.join(sorted(MLP_KINDS))}")
                mlp = mlp_kind.from_dict(L["mlp"], where + ".mlp")
            of = _need(L, "weights_of", int, where, required=False)
            if of is not None and not (0 <= of < len(layers_raw)) or of == i:
                raise ConfigError(f"config.json: '{where}.weights_of' must name another layer")
            layers.append(KifunexLayer(typ, mixer, mlp, of))
        eps = _need(_need(d, "norm", dict, ""), "eps", float, "norm", default=1e-6, required=False)
        cap = _need(d, "logit_softcap", float, "", default=0.0, required=False)
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        eos = d.get("eos_token_id", -1)
        out = cls(architecture=d.get("architecture", ARCHITECTURE),
                  vocab_size=_positive(_need(d, "vocab", int, ""), "vocab"),
                  hidden_size=_positive(_need(d, "width", int, ""), "width"),
                  streams=_positive(_need(d, "streams", int, "", default=1, required=False), "streams"),
                  eps=eps, logit_scale=_need(d, "logit_scale", float, "", default=1.0, required=False),
                  logit_softcap=cap, layers=layers, raw=dict(d),
                  eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1)
        for i in range(len(layers)):
            out.weight_owner(i)
        return out

    def to_dict(self) -> dict:
        return dict(self.raw)
