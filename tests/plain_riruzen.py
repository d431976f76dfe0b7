"""The Riruzen decoder, plainly: one slow function per mechanism, on the CPU, in float64 unless told otherwise.

This file is what the engine's kernels are compared with.  It shares no code with the package: it takes a
configuration as the dictionary of config.json and the weights as a dictionary of tensors by checkpoint name,
and runs one sequence at a time, either whole or token by token with an explicit state.

Notation.  x: residual stream [T, width].  A layer computes h = gnorm(x), u = h + canon(h), and
x <- x + mixer(u) + ff(h).  Linear weights are [out, in].
"""
from __future__ import annotations

import torch


def group_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Each of `groups` equal consecutive parts of a row is divided by sqrt(mean(part^2) + eps); then times weight."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, W) * weight


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def causal_taps(h: torch.Tensor, w: torch.Tensor, history: torch.Tensor | None = None) -> torch.Tensor:
    """out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zero before the sequence's start.  `history`: the
    taps - 1 inputs that came before h (oldest first), zeros if None."""
    T, W = h.shape
    taps = w.shape[1]
    if history is None:
        history = h.new_zeros((taps - 1, W))
    ext = torch.cat([history, h], dim=0)                 # ext[taps - 1 + t] = h_t
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            out[t] += w[:, j] * ext[t + j]
    return out


def gated_feed_forward(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """down( relu(gate h) * (up h) )"""
    return (torch.relu(h @ gate.T) * (h @ up.T)) @ down.T


def latent_attention(u: torch.Tensor, w: dict, heads: int, dim: int, vdim: int, scale: float, eps: float,
                     latents_before: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Attention whose keys and values are both made from one normed latent per token; no positions.

    w: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o.  Returns (output [T, width], latents [T0 + T, kv_rank]) where
    the latents include `latents_before` (those of the T0 earlier tokens of the sequence)."""
    T = u.shape[0]
    cq = rms_norm(u @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, heads, dim)
    c_new = rms_norm(u @ w["dkv"].T, w["dkv.norm"], eps)
    c = c_new if latents_before is None else torch.cat([latents_before, c_new], dim=0)
    n = c.shape[0]
    k = (c @ w["uk"].T).reshape(n, heads, dim)
    v = (c @ w["uv"].T).reshape(n, heads, vdim)
    out = u.new_zeros((T, heads, vdim))
    first = n - T
    for t in range(T):
        see = first + t + 1                               # keys 0 .. own position
        for hd in range(heads):
            s = (k[:see, hd] @ q[t, hd]) * scale
            p = torch.softmax(s, dim=0)
            out[t, hd] = p @ v[:see, hd]
    gated = out.reshape(T, heads * vdim) * torch.sigmoid(u @ w["g"].T)
    return gated @ w["o"].T, c


def hgrn2(u: torch.Tensor, w: dict, heads: int, dim: int, vdim: int, eps: float,
          state: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Gated linear recurrence: per head S <- diag(f) S + (1 - f) v^T, o = S^T q, with q = silu(Wq u),
    v = Wv u, f = l + (1 - l) sigmoid(Wf u + b).  w: q, f, f.b, lower, v, norm, o.
    state [heads, dim, vdim] (zeros if None).  Returns (output [T, width], state after the last token)."""
    T = u.shape[0]
    q = torch.nn.functional.silu(u @ w["q"].T).reshape(T, heads, dim)
    v = (u @ w["v"].T).reshape(T, heads, vdim)
    low = w["lower"]
    f = (low + (1 - low) * torch.sigmoid(u @ w["f"].T + w["f.b"])).reshape(T, heads, dim)
    S = u.new_zeros((heads, dim, vdim)) if state is None else state.clone()
    o = u.new_zeros((T, heads, vdim))
    for t in range(T):
        S = f[t].unsqueeze(-1) * S + (1 - f[t]).unsqueeze(-1) * v[t].unsqueeze(1)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = o / torch.sqrt(o.pow(2).mean(dim=-1, keepdim=True) + eps) * w["norm"]
    return o.reshape(T, heads * vdim) @ w["o"].T, S


class PlainRiruzen:
    """The whole model on one sequence.  `forward(tokens)` continues from what earlier calls left, so a prompt may
    be given whole, in portions or token by token; `reset()` starts a new sequence."""

    def __init__(self, config: dict, weights: dict, dtype: torch.dtype = torch.float64):
        self.cfg = config
        self.w = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in weights.items()}
        self.dtype = dtype
        self.reset()

    def reset(self) -> None:
        self.pos = 0
        n = len(self.cfg["layers"])
        self.history = [None] * n          # the last taps - 1 normed inputs of each layer
        self.state = [None] * n            # recurrent state or latents of each layer

    def _mixer_weights(self, i: int) -> dict:
        p = f"l{i}.mix."
        return {k[len(p):]: v for k, v in self.w.items() if k.startswith(p)}

    def forward(self, tokens, layer_outputs: list | None = None) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        T = len(tokens)
        eps, groups, taps = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["canon"]["taps"]
        ids = torch.as_tensor(tokens, dtype=torch.long)
        x = w["embed"][ids] + w["pos"][self.pos:self.pos + T]
        for i, layer in enumerate(cfg["layers"]):
            h = group_rms_norm(x, w[f"l{i}.norm1"], groups, eps)
            u = h + causal_taps(h, w[f"l{i}.canon1"], self.history[i])
            past = h if self.history[i] is None else torch.cat([self.history[i], h], dim=0)
            if past.shape[0] < taps - 1:
                past = torch.cat([h.new_zeros((taps - 1 - past.shape[0], h.shape[1])), past], dim=0)
            self.history[i] = past[past.shape[0] - (taps - 1):]
            m, mw = layer["mixer"], self._mixer_weights(i)
            if layer["type"] == "latent_attention":
                a, self.state[i] = latent_attention(u, mw, m["heads"], m["dim"], m["vdim"], m["scale"], eps, self.state[i])
            elif layer["type"] == "hgrn2":
                a, self.state[i] = hgrn2(u, mw, m["heads"], m["dim"], m["vdim"], eps, self.state[i])
            else:
                raise ValueError(f"unknown layer type {layer['type']!r}")
            if layer["mlp"] is not None:
                if layer["mlp"]["kind"] != "dense":
                    raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
                a = a + gated_feed_forward(h, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
            x = x + a
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        self.pos += T
        h = group_rms_norm(x, w["final.norm"], groups, eps)
        return (h @ w["embed"].T) * cfg["logit_scale"]
