"""Typed configuration of the Bonolorn decoder, read from config.json.

Bonolorn is a decoder whose blocks norm what a sublayer RETURNS: x += m * ln(mixer(x)), then x += m * ln(ff(x)), with a
layer norm (weight, no bias) and a residual multiplier m.  Positions enter once, as a sinusoidal vector added to the
embedding.  The mixer of a `parallel` layer is two mixers side by side that read the same input: softmax attention with
grouped keys and values, normed queries and keys, a linear distance bias, a sliding window and a sigmoid gate per head
(`left`), and linear attention with a fixed decay per head and a 32-bit state (`right`); their outputs are added with
two weights.  The feed-forward is dense (gelu, tanh form, gated) or a mixture of small clamped-swish experts chosen by a
sigmoid router with a correction, within the best groups, plus an expert every token uses.  The logits use the embedding table.

config.json of this design:

    architecture   "Bonolorn"
    vocab, width, residual_mult
    norm           {eps}
    layers         [{type: "parallel", mixer: {left, left_scale, right, right_scale}, mlp: {...} | null}, ...]
        left:   heads, kv_heads, dim, vdim, scale, mask: {size}
        right:  heads, dim, vdim, decay: [one per head]
        mlp:    {kind: "dense", ff}
                {kind: "moe", expert: {ff, limit}, router: {experts, top, scale, groups: {count, keep}}, shared: {ff, limit} | null}

Every size and constant comes from the file; a missing one is an error, an unknown layer type or feed-forward kind is
refused.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .model_config import ConfigError, _as_float, _as_int
from .riruzen_config import _need, _section

PARALLEL = "parallel"
DENSE, MOE = "dense", "moe"


@dataclass(frozen=True)
class WindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                        # query/key size of a head
    vdim: int                       # value size of a head
    scale: float
    window: int                     # a query sees itself and the window - 1 tokens before it; 0: all


@dataclass(frozen=True)
class DecayAttentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]        # one per head


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                       # DENSE or MOE
    ff: int                         # inner size (of one expert, for MOE)
    limit: float = 0.0              # MOE: the experts' clamp
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    router_scale: float = 1.0
    shared_ff: int = 0              # 0: no expert that every token uses
    shared_limit: float = 0.0


@dataclass(frozen=True)
class BonolornLayer:
    type: str
    left: WindowAttentionSpec
    left_scale: float
    right: DecayAttentionSpec
    right_scale: float
    mlp: Optional[FeedForwardSpec]


@dataclass(frozen=True)
class BonolornConfig:
    architecture: str
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: tuple[BonolornLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Bonolorn"

    @staticmethod
    def _mlp(mlp: Any, where: str) -> Optional[FeedForwardSpec]:
        if mlp is None:
            return None
        if not isinstance(mlp, Mapping):
            raise ConfigError(f"{where} must be an object or null")
        _need(mlp, ("kind",), where)
        if mlp["kind"] == DENSE:
            _need(mlp, ("ff",), where)
            return FeedForwardSpec(DENSE, _as_int(mlp, "ff"))
        if mlp["kind"] != MOE:
            raise ConfigError(f"{where}: unknown kind {mlp['kind']!r}; known: {DENSE}, {MOE}")
        expert, router = _section(mlp, "expert", where), _section(mlp, "router", where)
        _need(expert, ("ff", "limit"), f"{where}.expert")
        _need(router, ("experts", "top", "scale"), f"{where}.router")
        groups, keep = 1, 1
        if router.get("groups") is not None:
            g = _section(router, "groups", f"{where}.router")
            _need(g, ("count", "keep"), f"{where}.router.groups")
            groups, keep = _as_int(g, "count"), _as_int(g, "keep")
        shared_ff, shared_limit = 0, 0.0
        if mlp.get("shared") is not None:
            sh = _section(mlp, "shared", where)
            _need(sh, ("ff", "limit"), f"{where}.shared")
            shared_ff, shared_limit = _as_int(sh, "ff"), _as_float(sh, "limit")
        return FeedForwardSpec(MOE, _as_int(expert, "ff"), _as_float(expert, "limit"), _as_int(router, "experts"), _as_int(router, "top"),
                               groups, keep, _as_float(router, "scale"), shared_ff, shared_limit)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BonolornConfig":
        _need(d, ("vocab", "width", "residual_mult", "norm", "layers"), "config.json")
        norm = _section(d, "norm")
        _need(norm, ("eps",), "config.json: norm")
        if not isinstance(d["layers"], (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with one entry a layer")
        layers = []
        for i, entry in enumerate(d["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where} must be an object")
            _need(entry, ("type", "mixer"), where)
            if entry["type"] != PARALLEL:
                raise ConfigError(f"{where}: unknown layer type {entry['type']!r}; known: {PARALLEL}")
            m = _section(entry, "mixer", where)
            _need(m, ("left", "left_scale", "right", "right_scale"), f"{where}.mixer")
            L, R = _section(m, "left", f"{where}.mixer"), _section(m, "right", f"{where}.mixer")
            _need(L, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}.mixer.left")
            _need(R, ("heads", "dim", "vdim", "decay"), f"{where}.mixer.right")
            window = 0
            if L.get("mask") is not None:
                mask = _section(L, "mask", f"{where}.mixer.left")
                _need(mask, ("size",), f"{where}.mixer.left.mask")
                window = _as_int(mask, "size")
            decay = R["decay"]
            if not isinstance(decay, (list, tuple)):
                raise ConfigError(f"{where}.mixer.right.decay must be a list with one number a head")
            left = WindowAttentionSpec(_as_int(L, "heads"), _as_int(L, "kv_heads"), _as_int(L, "dim"), _as_int(L, "vdim"),
                                       _as_float(L, "scale"), window)
            right = DecayAttentionSpec(_as_int(R, "heads"), _as_int(R, "dim"), _as_int(R, "vdim"), tuple(float(x) for x in decay))
            layers.append(BonolornLayer(PARALLEL, left, _as_float(m, "left_scale"), right, _as_float(m, "right_scale"),
                                        cls._mlp(entry.get("mlp"), f"{where}.mlp")))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=cls.ARCHITECTURE, vocab=_as_int(d, "vocab"), width=_as_int(d, "width"),
                  residual_mult=_as_float(d, "residual_mult"), norm_eps=_as_float(norm, "eps"), layers=tuple(layers),
                  eos_token_ids=eos_ids, raw=dict(d))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab}, {self.width}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, l in enumerate(self.layers):
            where = f"layers[{i}]"
            a, r, f = l.left, l.right, l.mlp
            sizes = [a.heads, a.kv_heads, a.dim, a.vdim, r.heads, r.dim, r.vdim]
            if any(s <= 0 for s in sizes) or a.window < 0:
                raise ConfigError(f"{where}: every size must be positive, got {sizes}, window {a.window}")
            if a.heads % a.kv_heads:
                raise ConfigError(f"{where}: {a.heads} query heads are not a multiple of {a.kv_heads} kv heads")
            if len(r.decay) != r.heads:
                raise ConfigError(f"{where}: {len(r.decay)} decays for {r.heads} heads")
            if f is None:
                continue
            if f.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive, got {f.ff}")
            if f.kind == MOE:
                if f.experts <= 0 or not (0 < f.top <= f.experts) or f.groups <= 0 or f.experts % f.groups or not (0 < f.keep <= f.groups):
                    raise ConfigError(f"{where}.mlp.router: {f.experts} experts, top {f.top}, {f.groups} groups of which {f.keep} are kept do not fit")
                if f.top > f.keep * (f.experts // f.groups):
                    raise ConfigError(f"{where}.mlp.router: top {f.top} exceeds the {f.keep * (f.experts // f.groups)} experts of the kept groups")
                if f.shared_ff < 0:
                    raise ConfigError(f"{where}.mlp.shared: ff must be positive")

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for l in self.layers:
            a, r, f = l.left, l.right, l.mlp
            left: dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.window:
                left["mask"] = {"size": a.window}
            mixer = {"left": left, "left_scale": l.left_scale,
                     "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": list(r.decay)}, "right_scale": l.right_scale}
            if f is None:
                mlp = None
            elif f.kind == DENSE:
                mlp = {"kind": DENSE, "ff": f.ff}
            else:
                mlp = {"kind": MOE, "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.router_scale, "groups": {"count": f.groups, "keep": f.keep}},
                       "shared": {"ff": f.shared_ff, "limit": f.shared_limit} if f.shared_ff else None}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d: dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
