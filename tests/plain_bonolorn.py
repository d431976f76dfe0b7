"""The Bonolorn decoder, plainly: one slow function per mechanism, on the CPU, in float64 unless told otherwise.

This file is what the engine's kernels are compared with.  It shares no code with the package: it takes a
configuration as the dictionary of config.json and the weights as a dictionary of tensors by checkpoint name,
and runs one sequence at a time, either whole or token by token with an explicit state.

Notation.  x: residual stream [T, width].  A layer computes x <- x + m * ln1(mixer(x)), then x <- x + m * ln2(ff(x)):
the sublayers read the stream itself, the norms sit on their outputs.  Linear weights are [out, in].
"""
from __future__ import annotations

import math

import torch


def sinusoid_positions(positions: torch.Tensor, width: int, base: float = 10000.0) -> torch.Tensor:
    """[T, width]: entry 2i is sin(p * base^(-2i / width)), entry 2i + 1 the cosine of the same angle."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / width)[None, :]
    out = torch.zeros(positions.shape[0], 2 * i.shape[0], dtype=torch.float64)
    out[:, 0::2] = torch.sin(angle)
    out[:, 1::2] = torch.cos(angle)
    return out[:, :width]                    # an odd width ends on a sine


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight, var the mean of the squared deviations; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt(d.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def distance_slopes(heads: int) -> torch.Tensor:
    """slope of head h = 2^(-8 (h + 1) / heads)"""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def window_attention(h: torch.Tensor, w: dict, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, window: int,
                     eps: float, start: int = 0, keys_before: torch.Tensor | None = None,
                     values_before: torch.Tensor | None = None):
    """Grouped-query softmax attention with normed queries and keys, a linear distance bias, a sliding window (0: none)
    and a sigmoid gate per head.  w: q, k, v, q.norm, k.norm, g, o.  The tokens of h stand at positions start, start + 1, ...;
    keys_before / values_before [start, kv_heads, *] are the normed keys and the values of the positions before.
    Returns (output [T, width], all keys, all values)."""
    T = h.shape[0]
    q = rms_norm((h @ w["q"].T).reshape(T, heads, dim), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).reshape(T, kv_heads, dim), w["k.norm"], eps)
    v = (h @ w["v"].T).reshape(T, kv_heads, vdim)
    if keys_before is not None:
        k, v = torch.cat([keys_before, k], dim=0), torch.cat([values_before, v], dim=0)
    slopes = distance_slopes(heads)
    gate = torch.sigmoid(h @ w["g"].T)                                     # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    per = heads // kv_heads
    for t in range(T):
        i = start + t
        lo = max(0, i - window + 1) if window > 0 else 0                  # 0 <= i - j < window; no window: every key before
        js = torch.arange(lo, i + 1)
        for hd in range(heads):
            g = hd // per
            s = (k[lo:i + 1, g] @ q[t, hd]) * scale - slopes[hd] * (i - js).to(h.dtype)
            p = torch.softmax(s, dim=0)
            out[t, hd] = (p[:, None] * v[lo:i + 1, g]).sum(dim=0) * gate[t, hd]
    return out.reshape(T, heads * vdim) @ w["o"].T, k, v


def decay_attention(h: torch.Tensor, w: dict, heads: int, dim: int, vdim: int, decay, eps: float,
                    state: torch.Tensor | None = None):
    """Linear attention with a fixed decay per head: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v
    passed through silu; the heads' outputs are normed together, gated elementwise and projected.
    w: q, k, v, g, o, norm.  state [heads, dim, vdim] (zeros if None).  Returns (output [T, width], state)."""
    T = h.shape[0]
    q = silu(h @ w["q"].T).reshape(T, heads, dim)
    k = silu(h @ w["k"].T).reshape(T, heads, dim)
    v = silu(h @ w["v"].T).reshape(T, heads, vdim)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    d = torch.as_tensor(decay, dtype=h.dtype)
    o = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        S = d[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    y = rms_norm(o.reshape(T, heads * vdim), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return y @ w["o"].T, S


def gelu_feed_forward(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down( g * sigmoid(1.702 g) * (u + 1) )"""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """For each token the `top` experts and their weights.  Scores are sigmoid(router h); the choice is made on
    score + correction, among the experts of the `keep` best of `groups` equal groups of neighbours (a group is worth
    the sum of its two largest choice scores); the weights are the plain scores of the chosen, normed to sum 1, times scale."""
    s = torch.sigmoid(h @ router.T)                                        # [T, E]
    c = s + correction
    T, E = s.shape
    size = E // groups
    cg = c.reshape(T, groups, size)
    worth = cg.topk(min(2, size), dim=-1).values.sum(dim=-1)               # [T, groups]
    best = worth.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(T, groups, size).reshape(T, E), c, torch.full_like(c, -math.inf))
    chosen = masked.topk(top, dim=-1).indices                             # [T, top]
    picked = s.gather(1, chosen)
    weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * scale
    return chosen, weights


def expert_feed_forward(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    """w: router, correction, e<j>.{gate,up,down}, shared.{gate,up,down}."""
    r = mlp["router"]
    chosen, weights = route(h, w["router"], w["correction"].to(h.dtype), r["top"], r["groups"]["count"], r["groups"]["keep"], r["scale"])
    out = torch.zeros_like(h)
    limit = mlp["expert"]["limit"]
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"])
    return out


class PlainBonolorn:
    """The whole model on one sequence.  forward(tokens) runs a whole prompt; step(tokens, state) runs the next
    tokens from an explicit state (keys, values and recurrent state per layer, and the position)."""

    def __init__(self, cfg: dict, weights: dict[str, torch.Tensor], dtype: torch.dtype = torch.float64):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}

    def _sub(self, prefix: str) -> dict:
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self) -> dict:
        return {"pos": 0, "layers": [{"k": None, "v": None, "S": None} for _ in self.cfg["layers"]]}

    def step(self, tokens, state: dict, trace: list | None = None) -> torch.Tensor:
        """Logits [T, vocab] of the next tokens; `state` is updated in place.  `trace`, if a list, receives the
        residual stream after every layer."""
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(tokens, dtype=torch.long)
        T, start = ids.shape[0], state["pos"]
        eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
        x = w["embed"][ids] + sinusoid_positions(torch.arange(start, start + T), cfg["width"]).to(self.dtype)
        for i, layer in enumerate(cfg["layers"]):
            if layer["type"] != "parallel":
                raise ValueError(f"unknown layer type {layer['type']!r}")
            mx, st = layer["mixer"], state["layers"][i]
            L, R = mx["left"], mx["right"]
            a, st["k"], st["v"] = window_attention(x, self._sub(f"l{i}.mix.left."), L["heads"], L["kv_heads"], L["dim"], L["vdim"],
                                                   L["scale"], (L.get("mask") or {}).get("size", 0), eps, start, st["k"], st["v"])
            b, st["S"] = decay_attention(x, self._sub(f"l{i}.mix.right."), R["heads"], R["dim"], R["vdim"], R["decay"], eps, st["S"])
            x = x + m * layer_norm(mx["left_scale"] * a + mx["right_scale"] * b, w[f"l{i}.norm1"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                sub = self._sub(f"l{i}.mlp.")
                if mlp["kind"] == "dense":
                    f = gelu_feed_forward(x, sub["gate"], sub["up"], sub["down"])
                elif mlp["kind"] == "moe":
                    f = expert_feed_forward(x, sub, mlp)
                else:
                    raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
                x = x + m * layer_norm(f, w[f"l{i}.norm2"], eps)
            if trace is not None:
                trace.append(x.clone())
        state["pos"] = start + T
        return layer_norm(x, w["final.norm"], eps) @ w["embed"].T

    def forward(self, tokens, trace: list | None = None) -> torch.Tensor:
        return self.step(tokens, self.new_state(), trace)
