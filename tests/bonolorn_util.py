"""Tiny Bonolorn configurations with weights made here, model folders of them, and the comparison of what the engine
returns with the plain implementation (plain_bonolorn.py)."""
from __future__ import annotations

import json
import random

import torch

from plain_bonolorn import PlainBonolorn


def _left(heads, kv_heads, dim, vdim, scale, window):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        d["mask"] = {"size": window}
    return d


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, groups, keep, ff, limit, scale, shared_ff=None, shared_limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
            "shared": None if shared_ff is None else {"ff": shared_ff, "limit": shared_limit}}


def _layer(left, ls, right, rs, mlp):
    return {"type": "parallel", "mixer": {"left": left, "left_scale": ls, "right": right, "right_scale": rs}, "mlp": mlp}


def _config(vocab, width, mult, eps, layers):
    return {"architecture": "Bonolorn", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps}, "layers": layers}


# A: sizes that are no multiples of 8 (the bfloat16 engine falls back to its plain kernels), values smaller and larger
#    than keys, a window shorter than two pages and one that is no multiple of anything, one kv head for three query
#    heads, experts in three groups, a layer without feed-forward.
# B: everything that can be 1 is 1: one head each, a window of one token (a query sees itself only), one expert chosen,
#    groups of one expert, multiplier and scales of 1, no expert for every token.
# C: sizes at which the bfloat16 engine takes its tensor-core paths (multiples of 64), windows across several pages,
#    as many kv heads as query heads in one layer, a decay of exactly 1, four groups of which two are kept.
# D: heads of 128 with grouped keys, a window longer than any test sequence and a layer without a window, experts
#    whose every group is kept.
CONFIGS = {
    "A": _config(211, 72, 0.3, 1e-5, [
        _layer(_left(3, 1, 20, 12, 0.22, 24), 0.6, _right(2, 20, 40, (0.9, 0.995)), 0.9, _dense(100)),
        _layer(_left(2, 2, 12, 28, 0.3, 37), 1.1, _right(3, 12, 12, (0.5, 0.97, 0.999)), 0.4, _moe(6, 2, 3, 2, 24, 1.5, 1.5, 40, 1.2)),
        _layer(_left(4, 2, 8, 8, 0.35, 5), 0.8, _right(1, 36, 20, (0.98,)), 0.7, None)]),
    "B": _config(97, 40, 1.0, 1e-6, [
        _layer(_left(1, 1, 40, 40, 0.16, 1), 1.0, _right(1, 40, 40, (0.9,)), 1.0, _moe(2, 1, 2, 1, 32, 2.0, 1.0)),
        _layer(_left(1, 1, 16, 24, 0.25, 2), 1.0, _right(1, 8, 56, (0.99,)), 1.0, _dense(64))]),
    "C": _config(331, 256, 0.5, 1e-5, [
        _layer(_left(4, 2, 64, 64, 0.125, 40), 0.7, _right(2, 64, 128, (0.95, 1.0)), 0.8, _dense(512)),
        _layer(_left(4, 4, 32, 32, 0.18, 96), 0.5, _right(4, 32, 32, (0.6, 0.88, 0.97, 0.999)), 1.0, _moe(8, 2, 4, 2, 128, 1.5, 2.5, 256, 1.5)),
        _layer(_left(8, 2, 64, 64, 0.125, 17), 0.9, _right(2, 128, 64, (0.99, 0.9)), 0.6, _moe(16, 4, 2, 1, 64, 7.0, 1.0, 64, 7.0))]),
    "D": _config(150, 256, 0.4, 1e-6, [
        _layer(_left(4, 2, 128, 128, 0.09, 1000), 0.7, _right(4, 128, 64, (0.9, 0.99, 0.999, 0.97)), 0.8, _moe(4, 2, 2, 2, 64, 1.0, 1.0, 128, 2.0)),
        _layer(_left(2, 1, 128, 128, 0.09, 0), 0.7, _right(2, 64, 64, (0.8, 0.995)), 0.8, _dense(256))]),
}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 16}


def make_weights(cfg: dict, seed: int, sharp: float = 1.0, decisive: bool = False) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16 as a checkpoint holds them.  `sharp` multiplies the weights of the query
    norm, so that a few keys carry a query's whole weight and a key that is lost, misplaced or wrongly let through a
    window's edge changes the output by its full size.  `decisive` spreads the router's corrections so far apart that
    the choice of experts does not hang on the last bits of a score (for comparisons in bfloat16, where a near-tie
    decided the other way would change a token's output wholly)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    lin = lambda o, i, gain=1.0: rnd(o, i, std=gain / i ** 0.5)
    w = {"embed": rnd(cfg["vocab"], W), "final.norm": 1 + rnd(W, std=0.2)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        L, R = layer["mixer"]["left"], layer["mixer"]["right"]
        w[p + "norm1"] = 1 + rnd(W, std=0.2)
        H, G, D, Vd = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
        w[p + "mix.left.q"], w[p + "mix.left.k"], w[p + "mix.left.v"] = lin(H * D, W), lin(G * D, W), lin(G * Vd, W)
        w[p + "mix.left.q.norm"], w[p + "mix.left.k.norm"] = (1 + rnd(D, std=0.2)) * sharp, 1 + rnd(D, std=0.2)
        w[p + "mix.left.g"], w[p + "mix.left.o"] = lin(H, W, 2.0), lin(W, H * Vd)
        H, D, Vd = R["heads"], R["dim"], R["vdim"]
        w[p + "mix.right.q"], w[p + "mix.right.k"], w[p + "mix.right.v"] = lin(H * D, W, 2.0), lin(H * D, W, 2.0), lin(H * Vd, W, 2.0)
        w[p + "mix.right.g"], w[p + "mix.right.o"], w[p + "mix.right.norm"] = lin(H * Vd, W, 2.0), lin(W, H * Vd), 1 + rnd(H * Vd, std=0.2)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        w[p + "norm2"] = 1 + rnd(W, std=0.2)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(ff, W, 1.5), lin(ff, W), lin(W, ff)
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            w[p + "mlp.router"] = lin(E, W, 2.0)
            if decisive:
                # scores lie in (0, 1): experts of a group 3 apart, groups 40 apart, so neither the groups' worth nor the
                # experts' order can hang on a score
                G = mlp["router"].get("groups", {}).get("count", 1)
                rank = torch.cat([torch.randperm(E // G, generator=g) for _ in range(G)]).float()
                w[p + "mlp.correction"] = rank * 3.0 + torch.randperm(G, generator=g).float().repeat_interleave(E // G) * 40.0 - 5.0
            else:
                w[p + "mlp.correction"] = rnd(E, std=0.3) - 0.2           # some choice scores are negative
            for j in range(E):
                w[p + f"mlp.e{j}.gate"], w[p + f"mlp.e{j}.up"], w[p + f"mlp.e{j}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
            if mlp.get("shared") is not None:
                ff = mlp["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(folder, cfg: dict, weights: dict[str, torch.Tensor]):
    from lucciola_b200.weights.safetensors_io import write_safetensors
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", weights)
    return folder


def tokens(cfg: dict, n: int, salt: int = 0) -> list[int]:
    g = torch.Generator().manual_seed(7919 * salt + n)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


_plain: dict = {}


def plain_logits(key, cfg: dict, weights: dict, ids: list[int]) -> torch.Tensor:
    """Float64 logits of the whole sequence at every position, by the plain implementation (cached)."""
    k = (key, tuple(ids))
    if k not in _plain:
        _plain[k] = PlainBonolorn(cfg, weights).forward(ids)
    return _plain[k]


# Largest |engine - plain| as a fraction of the sequence's largest |logit| (bfloat16: the most these tests have measured is 3.2e-2, in the
# configuration whose multiplier and scales are all 1).
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def compare(got: dict, key, cfg: dict, weights: dict, reqs: dict[str, list[int]], dtype: str, tol: float | None = None) -> float:
    tol = TOL[dtype] if tol is None else tol
    worst = 0.0
    assert got, "the trace asked for no logits"
    for rid, ids in reqs.items():
        ref = plain_logits(key, cfg, weights, ids)
        scale = ref.abs().max().item()
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert torch.isfinite(row).all(), f"request {rid} position {p}: logits are not finite"
            err = (row - ref[p]).abs().max().item() / scale
            assert err <= tol, f"request {rid}: first wrong position {p} (error {err:.3g} of scale, allowed {tol:.3g})"
            worst = max(worst, err)
    return worst


def rounding_alone(cfg: dict, weights: dict, ids: list[int]) -> float:
    """What rounding alone does to this model's logits: the largest change, as a fraction of the largest |logit|, when
    the plain implementation rounds the input of every mixer and feed-forward to bfloat16 and nothing else.  Any
    bfloat16 engine does at least that; a norm behind a sublayer whose output is small multiplies it."""
    import plain_bonolorn as plain
    exact = PlainBonolorn(cfg, weights).forward(ids)
    r = lambda x: x.to(torch.bfloat16).to(torch.float64)
    names = ("window_attention", "decay_attention", "gelu_feed_forward", "expert_feed_forward")
    saved = [getattr(plain, n) for n in names]
    try:
        for n, f in zip(names, saved):
            setattr(plain, n, (lambda f: lambda h, *a, **k: f(r(h), *a, **k))(f))
        rounded = PlainBonolorn(cfg, weights).forward(ids)
    finally:
        for n, f in zip(names, saved):
            setattr(plain, n, f)
    return ((rounded - exact).abs().max() / exact.abs().max()).item()


def bound(dtype: str, cfg: dict, weights: dict, reqs: dict, base: float | None = None) -> float:
    """The bound of a comparison: the type's own, or for bfloat16 four times what rounding alone does to this model if
    that is more."""
    base = TOL[dtype] if base is None else base
    if dtype != "bfloat16":
        return base
    longest = max(reqs.values(), key=len)
    return max(base, 4 * rounding_alone(cfg, weights, longest))


def random_config(seed: int) -> dict:
    """A configuration whose every size is drawn: widths, the number of layers, head counts and groupings, head sizes
    that are no multiples of 4 or 8, values larger and smaller than keys, windows from one token to none, decays up to
    1, expert counts, groups and choices, layers without feed-forward, experts with and without one for every token."""
    rng = random.Random(seed)
    width = rng.choice([24, 36, 40, 64, 72, 100, 128, 200])
    layers = []
    for _ in range(rng.randint(1, 4)):
        kv = rng.choice([1, 2, 3])
        H = kv * rng.choice([1, 2, 4])
        left = _left(H, kv, rng.choice([4, 8, 10, 16, 24, 64]), rng.choice([4, 8, 12, 20, 32, 72]), rng.choice([0.1, 0.2, 0.3]),
                     rng.choice([0, 1, 2, 7, 16, 33, 64, 150]))
        rh = rng.choice([1, 2, 3, 5])
        right = _right(rh, rng.choice([4, 6, 16, 33, 64, 100]), rng.choice([3, 8, 16, 33, 64, 70]), [rng.choice([0.3, 0.9, 0.99, 0.999, 1.0]) for _ in range(rh)])
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = _dense(rng.choice([24, 64, 100, 128, 192]))
        else:
            groups = rng.choice([1, 2, 3, 4])
            size = rng.choice([1, 2, 3, 5])
            keep = rng.randint(1, groups)
            top = rng.randint(1, min(keep * size, 4))
            mlp = _moe(groups * size, top, groups, keep, rng.choice([8, 24, 64, 100]), rng.choice([0.5, 1.5, 7.0]), rng.choice([1.0, 2.5]),
                       rng.choice([None, 16, 64]), rng.choice([1.0, 3.0]))
        layers.append(_layer(left, rng.choice([0.5, 1.0, 1.3]), right, rng.choice([0.4, 1.0]), mlp))
    return _config(rng.choice([64, 97, 300]), width, rng.choice([0.2, 0.5, 1.0]), rng.choice([1e-5, 1e-6]), layers)
