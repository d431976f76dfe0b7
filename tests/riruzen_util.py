"""Tiny Riruzen configurations with weights made here, model folders of them, and the comparison of what the engine
returns with the plain implementation (plain_riruzen.py)."""
from __future__ import annotations

import json

import torch

from plain_riruzen import PlainRiruzen


def _latent(heads, dim, vdim, q_rank, kv_rank, scale, ff):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _hgrn2(heads, dim, vdim, ff):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, positions, logit_scale, eps, groups, taps, layers):
    return {"architecture": "Riruzen", "vocab": vocab, "width": width, "max_positions": positions, "logit_scale": logit_scale,
            "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps}, "layers": layers}


# P: attention first, two attention layers in a row, a layer without feed-forward, four taps, sizes that are no
#    multiples of 8 (the bfloat16 engine must fall back to its plain kernels there).
# Q: everything that can be 1 is 1 (groups, taps, heads), one layer of each kind.
# R: sizes at which the bfloat16 engine takes its tensor-core paths (multiples of 64 and 128), two taps.
# S: a recurrence only (no pages at all), five taps, many small heads.
# T: twenty heads on a latent of 64, more than a tile of the decode kernels has rows (the engine cuts them into two
#    groups that read the one cached head), beside a recurrence with heads of 16 x 72.
# In P and R the last attention layer has a latent so much wider than a head that the engine keeps the query's two
# maps apart; in the other attention layers it multiplies them out.
CONFIGS = {
    "P": _config(211, 72, 640, 0.5, 1e-6, 3, 4, [_latent(3, 20, 12, 36, 28, 0.3, 100), _latent(2, 16, 24, 24, 40, 0.21, None),
                                                 _hgrn2(2, 20, 40, 56), _latent(5, 8, 8, 32, 48, 0.4, 88), _hgrn2(3, 36, 12, None)]),
    "Q": _config(97, 40, 300, 1.0, 1e-5, 1, 1, [_hgrn2(1, 40, 40, 64), _latent(1, 32, 32, 40, 24, 0.17, 64)]),
    "R": _config(331, 256, 1024, 0.125, 2e-6, 2, 2, [_hgrn2(2, 128, 64, 512), _latent(4, 64, 64, 128, 128, 0.125, 512),
                                                     _hgrn2(4, 64, 128, 256), _latent(8, 32, 48, 64, 128, 0.18, 256)]),
    "S": _config(150, 48, 400, 2.0, 1e-5, 4, 5, [_hgrn2(6, 8, 8, 96), _hgrn2(3, 12, 16, None)]),
    "T": _config(257, 128, 600, 0.3, 1e-6, 8, 3, [_latent(20, 16, 24, 48, 64, 0.25, 192), _hgrn2(2, 16, 72, 128)]),
}
PAGE = {"P": 16, "Q": 8, "R": 16, "S": 16, "T": 16}


def make_weights(cfg: dict, seed: int, sharp: float = 1.0, keep: float | None = None) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16 as a checkpoint holds them.  `sharp` multiplies the maps that make the
    attention's queries, so that a few keys (anywhere in the sequence) carry a query's whole weight and a key that is
    lost or misplaced changes the output by its full size.  `keep` moves the recurrence's lower bounds up to at least
    that value, so that what entered the state hundreds of tokens ago still shows."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    lin = lambda o, i, gain=1.0: rnd(o, i, std=gain / i ** 0.5)
    w = {"embed": rnd(cfg["vocab"], W), "pos": rnd(cfg["max_positions"], W, std=0.5), "final.norm": 1 + rnd(W, std=0.2)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, D, Vd = m["heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = 1 + rnd(W, std=0.2)
        w[p + "canon1"] = rnd(W, cfg["canon"]["taps"], std=0.4)
        if layer["type"] == "latent_attention":
            w[p + "mix.dq"], w[p + "mix.dq.norm"] = lin(m["q_rank"], W), 1 + rnd(m["q_rank"], std=0.2)
            w[p + "mix.uq"] = lin(H * D, m["q_rank"], sharp)
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = lin(m["kv_rank"], W), 1 + rnd(m["kv_rank"], std=0.2)
            w[p + "mix.uk"], w[p + "mix.uv"] = lin(H * D, m["kv_rank"], 2.0), lin(H * Vd, m["kv_rank"])
            w[p + "mix.g"], w[p + "mix.o"] = lin(H * Vd, W, 2.0), lin(W, H * Vd)
        else:
            w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"] = lin(H * D, W, 2.0), lin(H * D, W, 2.0), lin(H * Vd, W)
            w[p + "mix.f.b"] = rnd(H * D)
            low = torch.rand(H * D, generator=g)
            w[p + "mix.lower"] = low if keep is None else keep + (1 - keep) * low
            w[p + "mix.norm"], w[p + "mix.o"] = 1 + rnd(Vd, std=0.2), lin(W, H * Vd)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(ff, W, 1.5), lin(ff, W), lin(W, ff)
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
        _plain[k] = PlainRiruzen(cfg, weights).forward(ids)
    return _plain[k]


# Largest |engine - plain| as a fraction of the sequence's largest |logit|.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


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
    bfloat16 engine does at least that; models with tiny heads behind a norm multiply it many times."""
    import plain_riruzen as plain
    exact = PlainRiruzen(cfg, weights).forward(ids)
    r = lambda x: x.to(torch.bfloat16).to(torch.float64)
    saved = plain.hgrn2, plain.latent_attention, plain.gated_feed_forward
    try:
        plain.hgrn2 = lambda u, *a, **k: saved[0](r(u), *a, **k)
        plain.latent_attention = lambda u, *a, **k: saved[1](r(u), *a, **k)
        plain.gated_feed_forward = lambda h, *a, **k: saved[2](r(h), *a, **k)
        rounded = PlainRiruzen(cfg, weights).forward(ids)
    finally:
        plain.hgrn2, plain.latent_attention, plain.gated_feed_forward = saved
    return ((rounded - exact).abs().max() / exact.abs().max()).item()


def random_config(seed: int) -> dict:
    """A configuration whose every size is drawn: widths, group counts, taps, the order and number of layers, head
    counts (above 16 too), head sizes that are no multiples of 4 or 8, layers without feed-forward."""
    import random
    rng = random.Random(seed)
    groups = rng.choice([1, 2, 3, 4, 5, 6, 8])
    width = groups * rng.choice([4, 6, 8, 10, 16, 24, 32, 40])
    layers = []
    for _ in range(rng.randint(1, 6)):
        ff = rng.choice([None, 24, 64, 100, 128, 192])
        if rng.random() < 0.5:
            layers.append(_latent(rng.choice([1, 2, 3, 4, 6, 8, 12, 18]), rng.choice([4, 8, 10, 16, 24, 48, 64]), rng.choice([4, 8, 12, 20, 32, 80]),
                                  rng.choice([8, 12, 32, 40, 128]), rng.choice([8, 12, 16, 24, 32, 64, 96, 128]), rng.choice([0.1, 0.125, 0.3]), ff))
        else:
            layers.append(_hgrn2(rng.choice([1, 2, 3, 4, 8]), rng.choice([4, 6, 16, 33, 48, 64, 100]), rng.choice([3, 8, 16, 33, 64, 70]), ff))
    return _config(rng.choice([64, 97, 300, 577]), width, 400, rng.choice([0.5, 1.0, 3.0]), rng.choice([1e-5, 1e-6]), groups,
                   rng.choice([1, 2, 3, 4, 6]), layers)
