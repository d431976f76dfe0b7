"""Typed configuration of the Riruzen decoder, read from config.json.

Riruzen is a small decoder of parallel blocks (one grouped RMS norm, then a mixer and a gated feed-forward side by
side), whose mixers are listed layer by layer: `latent_attention` (keys and values from one cached latent, no
positions) or `hgrn2` (a gated linear recurrence with a fixed-size state).  Positions enter once, as learned
vectors added to the embedding; every mixer reads its input through a short causal convolution over time.

config.json of this design:

    architecture   "Riruzen"
    vocab, width, max_positions, logit_scale
    norm           {eps, groups}
    canon          {taps}
    layers         [{type, mixer: {...}, mlp: {kind: "dense", ff} | null}, ...]
        latent_attention mixer: heads, dim, vdim, q_rank, kv_rank, scale
        hgrn2 mixer:            heads, dim, vdim

Every size and constant comes from the file; a missing one is an error, an unknown layer type or
feed-forward kind is refused.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .model_config import ConfigError, _as_float, _as_int

LATENT_ATTENTION = "latent_attention"
HGRN2 = "hgrn2"


def _section(d: Mapping[str, Any], key: str, where: str = "config.json") -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where} lacks the section {key!r}")
    return v


def _need(d: Mapping[str, Any], keys: tuple[str, ...], where: str) -> None:
    missing = [k for k in keys if k not in d or d[k] is None]
    if missing:
        raise ConfigError(f"{where} lacks required key(s): " + ", ".join(missing))


@dataclass(frozen=True)
class RiruzenLayer:
    type: str                       # LATENT_ATTENTION or HGRN2
    heads: int
    dim: int                        # query/key size of a head
    vdim: int                       # value size of a head
    ff: Optional[int]               # inner size of the gated feed-forward; None: the layer has none
    q_rank: int = 0                 # latent_attention only
    kv_rank: int = 0
    scale: float = 0.0


@dataclass(frozen=True)
class RiruzenConfig:
    architecture: str
    vocab: int
    width: int
    max_positions: int
    logit_scale: float
    norm_eps: float
    norm_groups: int
    taps: int
    layers: tuple[RiruzenLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Riruzen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RiruzenConfig":
        _need(d, ("vocab", "width", "max_positions", "logit_scale", "norm", "canon", "layers"), "config.json")
        norm, canon = _section(d, "norm"), _section(d, "canon")
        _need(norm, ("eps", "groups"), "config.json: norm")
        _need(canon, ("taps",), "config.json: canon")
        if not isinstance(d["layers"], (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with one entry a layer")
        layers = []
        for i, entry in enumerate(d["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where} must be an object")
            _need(entry, ("type", "mixer"), where)
            kind, m = entry["type"], _section(entry, "mixer", where)
            _need(m, ("heads", "dim", "vdim"), f"{where}.mixer")
            extra = {}
            if kind == LATENT_ATTENTION:
                _need(m, ("q_rank", "kv_rank", "scale"), f"{where}.mixer")
                extra = dict(q_rank=_as_int(m, "q_rank"), kv_rank=_as_int(m, "kv_rank"), scale=_as_float(m, "scale"))
            elif kind != HGRN2:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {LATENT_ATTENTION}, {HGRN2}")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                _need(mlp, ("kind", "ff"), f"{where}.mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
                ff = _as_int(mlp, "ff")
            layers.append(RiruzenLayer(kind, _as_int(m, "heads"), _as_int(m, "dim"), _as_int(m, "vdim"), ff, **extra))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=cls.ARCHITECTURE, vocab=_as_int(d, "vocab"), width=_as_int(d, "width"),
                  max_positions=_as_int(d, "max_positions"), logit_scale=_as_float(d, "logit_scale"),
                  norm_eps=_as_float(norm, "eps"), norm_groups=_as_int(norm, "groups"), taps=_as_int(canon, "taps"),
                  layers=tuple(layers), eos_token_ids=eos_ids, raw=dict(d))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab", "width", "max_positions", "norm_groups", "taps"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.width % self.norm_groups:
            raise ConfigError(f"width {self.width} is not a multiple of norm.groups {self.norm_groups}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, l in enumerate(self.layers):
            sizes = [l.heads, l.dim, l.vdim] + ([l.q_rank, l.kv_rank] if l.type == LATENT_ATTENTION else []) + ([l.ff] if l.ff is not None else [])
            if any(s <= 0 for s in sizes):
                raise ConfigError(f"layers[{i}]: every size must be positive, got {sizes}")

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for l in self.layers:
            m: dict[str, Any] = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
            if l.type == LATENT_ATTENTION:
                m.update(q_rank=l.q_rank, kv_rank=l.kv_rank, scale=l.scale)
            layers.append({"type": l.type, "mixer": m, "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}})
        d: dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                             "max_positions": self.max_positions, "logit_scale": self.logit_scale,
                             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "canon": {"taps": self.taps},
                             "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
