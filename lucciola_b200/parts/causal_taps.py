"""A short causal convolution over time, added to its input: u_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j).

One weight per channel and tap ([width, taps], no bias), zeros before a sequence's start.  The last taps - 1
inputs of a sequence are its state (a slot of [taps - 1, width] in the activation type, zero for a new
request), so a portion of a prompt or a single decoded token continues where the step before stopped.
With one tap there is no state and u = (1 + w) * h.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from .base import ParamSpec, Part, Runtime, StateCacheView, StateSlot, StepContext


class CausalTaps(Part):
    recordable = True

    def __init__(self, rt: Runtime, name: str, width: int, taps: int):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.rt, self.name, self.width, self.taps = rt, name, width, int(taps)
        self.weight: torch.Tensor | None = None     # float32 [taps, width]: the checkpoint's tensor, transposed

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.width, self.taps), "linear")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).to(torch.float32).t().contiguous()

    def cache_request(self) -> Optional[StateSlot]:
        return StateSlot((self.taps - 1, self.width), self.rt.act_dtype) if self.taps > 1 else None

    def forward(self, h: torch.Tensor, step: StepContext, cache: Optional[StateCacheView]) -> torch.Tensor:
        """u for this step's tokens; the sequences' states move on to the end of the step."""
        out = self.rt.empty(h.shape, h.dtype)
        state = cache.state if self.taps > 1 else None
        ops.causal_taps(out, h, self.weight, state, step, self.rt.stream)
        if state is not None:
            ops.causal_taps_state(state, h, self.taps, step, self.rt.stream)
        return out
