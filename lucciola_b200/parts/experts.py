"""A feed-forward of many small experts of which each token uses a few, plus (optionally) one that every token uses.

    z = W_router h (32-bit)         s = sigmoid(z)         choice score c = s + correction
    experts form `groups` equal groups of neighbours; a group is worth the sum of its two largest c; only experts of the
    `keep` best groups can be chosen; the `top` experts with the largest c are
    weights = s of the chosen / (their sum + 1e-20) * scale          (the correction steers the choice only)
    out = sum_k weight_k * expert_k(h) [+ shared(h)]

An expert is a gated feed-forward (GATE_ACTS of ops, e.g. "clamped_swish" with its limit) without biases.  The
checkpoint holds each expert's three matrices under <prefix>.e<j>.{gate,up,down}; they are stacked when bound
([experts, 2 ff, width] gate rows then up rows, and [experts, width, ff]).

Everything runs on the device with launches that do not depend on the choices (the pairs of token and choice are
sorted by expert by a kernel; the products walk a list of row tiles that the same kernel writes), so a step through
this part can be recorded.

Steps with many tokens (bfloat16 engine, `GROUPED_FROM` pairs an expert and more) take the tensor-memory product
instead: every expert's run of pairs is padded to whole tiles of 128 places, the tokens are gathered into that order,
and `gemm_tcgen05_grouped` multiplies every tile with its expert's matrix.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from .base import FeedForward, ParamSpec, Part, Runtime, StepContext
from .linear import Linear


# From this many pairs of token and choice an expert (on average) the padded runs of the tensor-memory product cost
# less than they gain: the padding is 64 places an expert on average, 127 at most, and the product several times faster.
GROUPED_FROM = 96


class RoutedExperts(FeedForward):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, experts: int, top: int, ff: int, act: str, limit: float,
                 router_scale: float, groups: int = 1, keep: int = 1, shared: Optional[FeedForward] = None,
                 correction: bool = True, out_dtype: Optional[torch.dtype] = None):
        if act not in ops.GATE_ACTS:
            raise ValueError(f"activation {act!r} of an expert is not one of {sorted(ops.GATE_ACTS)}")
        if experts % groups or not (0 < keep <= groups) or not (0 < top <= keep * (experts // groups)):
            raise ValueError(f"{experts} experts, top {top}, {groups} groups of which {keep} are kept do not fit")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.experts, self.top, self.ff, self.act, self.limit = experts, top, ff, act, float(limit)
        self.router_scale, self.groups, self.keep = float(router_scale), groups, keep
        self.shared, self.has_correction = shared, correction
        self.out_dtype = out_dtype          # type of the result (None: the activation type)
        self.router = Linear(rt, f"{prefix}.router", width, experts)
        self.correction: torch.Tensor | None = None
        self.interleaved = False
        self.gate_up: torch.Tensor | None = None        # [experts, 2 * ff, width]
        self.down: torch.Tensor | None = None           # [experts, width, ff]

    def children(self) -> list[Part]:
        return [self.router] + ([self.shared] if self.shared is not None else [])

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        specs = [ParamSpec(f"{p}.correction", (self.experts,), "linear")] if self.has_correction else []
        for j in range(self.experts):
            specs += [ParamSpec(f"{p}.e{j}.gate", (self.ff, self.width)), ParamSpec(f"{p}.e{j}.up", (self.ff, self.width)),
                      ParamSpec(f"{p}.e{j}.down", (self.width, self.ff))]
        return specs

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        if self.has_correction:
            self.correction = get(f"{p}.correction").to(torch.float32).contiguous()
        # gate and up rows of an expert: interleaved in blocks of 64 where the products with the activation in their epilogue
        # want them so (both kinds of product then read that one copy), else all gate rows and then all up rows
        gates, ups = [get(f"{p}.e{j}.gate") for j in range(self.experts)], [get(f"{p}.e{j}.up") for j in range(self.experts)]
        self.interleaved = bool(self.rt.fast_kernels and gates[0].is_cuda and gates[0].dtype == torch.bfloat16 and self.ff % 64 == 0
                                and self.width % 8 == 0)
        if self.interleaved:
            self.gate_up = torch.stack([ops.interleave_gate_up(g, u) for g, u in zip(gates, ups)]).contiguous()
        else:
            self.gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()
        self.down = torch.stack([get(f"{p}.e{j}.down") for j in range(self.experts)]).contiguous()

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        rt, E, top = self.rt, self.experts, self.top
        T = h.shape[0]
        pairs = T * top
        logits = self.router.forward(h, out_dtype=torch.float32)
        ids, weights = rt.empty((T, top), torch.int32), rt.empty((T, top), torch.float32)
        ops.route_topk(ids, weights, logits, self.correction, self.groups, self.keep, self.router_scale, rt.stream)
        always = self.shared.forward(h, step) if self.shared is not None else None
        out = rt.empty((T, self.width), self.out_dtype)
        if self.interleaved and pairs >= GROUPED_FROM * E and self.ff % 8 == 0 and h.dtype == torch.bfloat16:
            places = ops.expert_padded_places(pairs, E)
            pair_at, place_of = rt.empty((places,), torch.int32), rt.empty((pairs,), torch.int32)
            tile_group = rt.empty((places // ops.GROUP_TILE,), torch.int32)
            ops.expert_dispatch_padded(ids, E, pair_at, place_of, tile_group, rt.stream)
            xs = rt.empty((places, self.width))
            ops.expert_gather_rows(xs, h, pair_at, top, rt.stream)
            inner = rt.empty((places, self.ff))
            ops.gemm_tcgen05_grouped(inner, xs, self.gate_up, tile_group, rt.stream, act=self.act, limit=self.limit)
            y = rt.empty((places, self.width), torch.float32)
            ops.gemm_tcgen05_grouped(y, inner, self.down, tile_group, rt.stream)
            ops.expert_combine(out, y, weights, place_of, rt.stream, always=always)
            return out
        offsets, pair_at, place_of = rt.empty((E + 1,), torch.int32), rt.empty((pairs,), torch.int32), rt.empty((pairs,), torch.int32)
        meta = rt.empty((4 + 3 * ops.expert_max_tiles(pairs, E),), torch.int32)
        ops.expert_dispatch(ids, E, offsets, pair_at, place_of, meta, rt.stream)
        inner = rt.empty((pairs, self.ff))
        ops.expert_gemm(inner, h, self.gate_up, meta, pair_at, top, True, rt.stream, act=self.act, limit=self.limit, fast=rt.fast_kernels,
                        interleaved=self.interleaved)
        y = rt.empty((pairs, self.width), torch.float32)
        ops.expert_gemm(y, inner, self.down, meta, pair_at, top, False, rt.stream, fast=rt.fast_kernels)
        ops.expert_combine(out, y, weights, place_of, rt.stream, always=always)
        return out
