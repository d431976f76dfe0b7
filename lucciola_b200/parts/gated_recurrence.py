"""HGRN2: linear attention whose forget gate also decides what is written.  Per head, with a state S [dim, vdim]:

    q = silu(W_q u)    v = W_v u    f = l + (1 - l) * sigmoid(W_f u + b)        (l: a lower bound per channel)
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        o_t = S_t^T q_t
    out = W_o concat_h( rmsnorm(o_t,h) * w )          (w [vdim], shared by the heads)

The state is 32-bit, one slot a request, zero for a new request, and is all this mixer keeps of the past:
prompts, portions and decoded tokens go through the same kernel, which walks a sequence's tokens of the
step in order from the state the step before left.  W_q | W_f | W_v are one product with 32-bit output; the
gates, the recurrence and the output are computed in 32-bit.
"""
from __future__ import annotations

from typing import Callable

import torch

from .. import ops
from .base import Mixer, ParamSpec, Part, Runtime, StateCacheView, StateSlot, StepContext
from .linear import Linear


class GatedLinearRecurrence(Mixer):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, dim: int, vdim: int, eps: float):
        self.rt, self.prefix = rt, prefix
        self.width, self.heads, self.dim, self.vdim, self.eps = width, heads, dim, vdim, float(eps)
        self.qfv = Linear(rt, [f"{prefix}.q", f"{prefix}.f", f"{prefix}.v"], width, [heads * dim, heads * dim, heads * vdim])
        self.o = Linear(rt, f"{prefix}.o", heads * vdim, width)
        self.bias: torch.Tensor | None = None
        self.lower: torch.Tensor | None = None
        self.norm_w: torch.Tensor | None = None

    def children(self) -> list[Part]:
        return [self.qfv, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p, n = self.prefix, self.heads * self.dim
        return [ParamSpec(f"{p}.f.b", (n,), "linear"), ParamSpec(f"{p}.lower", (n,), "unit"), ParamSpec(f"{p}.norm", (self.vdim,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        self.bias = get(f"{p}.f.b").to(torch.float32).contiguous()
        self.lower = get(f"{p}.lower").to(torch.float32).contiguous()
        self.norm_w = get(f"{p}.norm").to(torch.float32).contiguous()

    def cache_request(self) -> StateSlot:
        return StateSlot((self.heads, self.dim, self.vdim), torch.float32)

    def forward(self, u: torch.Tensor, step: StepContext, cache: StateCacheView, write_cache: bool = True) -> torch.Tensor:
        rt = self.rt
        T, H, n = u.shape[0], self.heads, self.heads * self.dim
        if not write_cache:
            raise ops.KernelError("a recurrent mixer has no cache another call could have written")
        pre = self.qfv.forward(u, out_dtype=torch.float32)                    # [T, 2 * H * dim + H * vdim]
        o = rt.empty((T, H * self.vdim), torch.float32)
        ops.gated_recurrence(pre, 0, n, 2 * n, self.bias, self.lower, cache.state, o, step, H, self.dim, self.vdim, rt.stream,
                             max_tokens_a_seq=step.max_q_len)
        normed = rt.empty((T * H, self.vdim))
        ops.add_rmsnorm(normed, o.view(T * H, self.vdim), None, self.norm_w, self.eps, rt.stream)
        return self.o.forward(normed.view(T, H * self.vdim))
