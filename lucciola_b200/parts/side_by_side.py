"""Two mixers side by side: both read the same input, and the result is a * left(x) + b * right(x).

What each mixer keeps of the past stays its own: the pair asks for (left's cache, right's cache) and hands each its view.
Mixers that offer their steps apart (in_names / in_sizes, inner, `o`, as GatedBiasAttention and DecayLinearAttention do)
are run with stacked products: ONE input product over the rows of both (32-bit output), each mixer's inner step writing
its scaled result into its columns of one matrix, and ONE output product over that matrix with the two output maps laid
side by side along the input, which is the weighted sum: [W_l | W_r] [a y_l ; b y_r] = a W_l y_l + b W_r y_r.  The
weights a and b multiply in 32-bit inside the inner steps' last kernels, before the one rounding there, so they cost
neither a kernel nor a rounding.
"""
from __future__ import annotations

from typing import Callable, Hashable, Optional

import torch

from .base import BatchShape, Mixer, ParamSpec, Part, Runtime, StepContext, StepPlan
from .linear import Linear


class SideBySideMixer(Mixer):
    def __init__(self, rt: Runtime, width: int, left: Mixer, right: Mixer, left_scale: float, right_scale: float):
        for m in (left, right):
            if not all(hasattr(m, a) for a in ("in_names", "in_sizes", "inner", "inner_size", "o")):
                raise ValueError(f"{type(m).__name__} does not offer its steps apart (in_names, in_sizes, inner, inner_size, o)")
        self.rt, self.width = rt, width
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.n_left = sum(left.in_sizes())
        self.proj = Linear(rt, left.in_names() + right.in_names(), width, left.in_sizes() + right.in_sizes())
        self.o = Linear(rt, [left.o.names[0], right.o.names[0]], [left.inner_size, right.inner_size], width)

    @property
    def recordable(self) -> bool:
        return bool(self.left.recordable and self.right.recordable)

    def children(self) -> list[Part]:
        return [self.proj, self.o]

    def param_specs(self) -> list[ParamSpec]:
        # the two mixers' own tensors (norm weights and the like); their products' tensors are this part's
        return list(self.left.param_specs()) + list(self.right.param_specs())

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.left.bind(get)
        self.right.bind(get)

    def cache_request(self) -> tuple:
        return (self.left.cache_request(), self.right.cache_request())

    def plan_key(self) -> Optional[Hashable]:
        a, b = self.left.plan_key(), self.right.plan_key()
        if a is not None and b is not None and a != b:
            raise NotImplementedError("two mixers side by side that both plan work on the host")
        return a if a is not None else b

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        return (self.left if self.left.plan_key() is not None else self.right).plan(batch)

    def forward(self, h: torch.Tensor, step: StepContext, cache, write_cache: bool = True) -> torch.Tensor:
        left_cache, right_cache = cache
        pre = self.proj.forward(h, out_dtype=torch.float32)
        kl = self.left.inner_size
        inner = self.rt.empty((h.shape[0], kl + self.right.inner_size))
        self.left.inner(pre[:, :self.n_left], step, left_cache, inner[:, :kl], self.left_scale, write_cache)
        self.right.inner(pre[:, self.n_left:], step, right_cache, inner[:, kl:], self.right_scale, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)
