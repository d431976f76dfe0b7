"""Latent attention without positions: keys and values of all heads are linear maps of ONE normed latent
vector per token, and only that latent is kept.

    c_q = rmsnorm(W_dq u) * w_q         q_h = W_uq[h] c_q                       (heads x dim)
    c   = rmsnorm(W_dkv u) * w_kv       k_h = W_uk[h] c,  v_h = W_uv[h] c        (dim, vdim a head)
    o_h = softmax_j<=i( q_h . k_h,j * scale ) v_h,j ;  out = W_o ( concat_h o_h * sigmoid(W_g u) )

Because k and v are linear in c, the head's key map moves to the query and its value map behind the sum:
q_h . (W_uk[h] c_j) = (W_uk[h]^T q_h) . c_j and sum_j p_j W_uv[h] c_j = W_uv[h] (sum_j p_j c_j).  So the
attention itself runs as `heads` query heads of size kv_rank over one shared "head" whose keys and values
are both the cached latents, through the same paged attention kernels as grouped-query attention
(KVPages(1, kv_rank, shared=True): one vector a token, half the memory of separate keys and values), for
prompts and for decoding alike.  The three maps that read u (W_dq | W_dkv | W_g) are one product with
32-bit output; the two norms and the write into the pages are one kernel; the per-head maps are one
batched product each, the second with the sigmoid gate in its epilogue.

Where it costs no more multiplications than the two maps apart (kv_rank * q_rank <= dim * (q_rank + kv_rank):
latents no wider than about a head), the query's two maps are multiplied out once when the weights are bound,
W_qc[h] = W_uk[h]^T W_uq[h] ([kv_rank, q_rank], formed in 32-bit), and the query in latent space is one product
of the normed query latent with the stacked W_qc.
"""
from __future__ import annotations

from typing import Callable, Hashable, Optional

import torch

from .. import ops
from .attention import DECODE_ROWS, TILE_ROWS, plan_tiles
from .base import BatchShape, KVCacheView, KVPages, Mixer, ParamSpec, Part, Runtime, StepContext, StepPlan
from .linear import Linear


class LatentAttention(Mixer):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float):
        self.rt, self.prefix = rt, prefix
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.eps = q_rank, kv_rank, float(scale), float(eps)
        # one product for everything that reads the mixer's input: query latent | key/value latent | gate
        self.down = Linear(rt, [f"{prefix}.dq", f"{prefix}.dkv", f"{prefix}.g"], width, [q_rank, kv_rank, heads * vdim])
        self.uq = Linear(rt, f"{prefix}.uq", q_rank, heads * dim)
        self.o = Linear(rt, f"{prefix}.o", heads * vdim, width)
        self.q_norm_w: torch.Tensor | None = None
        self.kv_norm_w: torch.Tensor | None = None
        self.uk_t: torch.Tensor | None = None       # [heads, kv_rank, dim]: W_uk[h]^T, the key map moved to the query
        self.uv: torch.Tensor | None = None         # [heads, vdim, kv_rank]
        # the query's two maps as one, where that is no more work (see the module's text)
        self.merge_query_maps = kv_rank * q_rank <= dim * (q_rank + kv_rank)
        self.qc: Linear | None = None               # [heads * kv_rank, q_rank] when merged

    def children(self) -> list[Part]:
        return [self.down, self.uq, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        return [ParamSpec(f"{p}.dq.norm", (self.q_rank,), "norm"), ParamSpec(f"{p}.dkv.norm", (self.kv_rank,), "norm"),
                ParamSpec(f"{p}.uk", (self.heads * self.dim, self.kv_rank)), ParamSpec(f"{p}.uv", (self.heads * self.vdim, self.kv_rank))]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        self.q_norm_w = get(f"{p}.dq.norm").to(torch.float32).contiguous()
        self.kv_norm_w = get(f"{p}.dkv.norm").to(torch.float32).contiguous()
        self.uk_t = get(f"{p}.uk").view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = get(f"{p}.uv").view(self.heads, self.vdim, self.kv_rank).contiguous()

    def bind_all(self, get) -> None:
        super().bind_all(get)
        if self.merge_query_maps:
            uq = self.uq.weight.view(self.heads, self.dim, self.q_rank)
            merged = torch.bmm(self.uk_t.float(), uq.float()).reshape(self.heads * self.kv_rank, self.q_rank)
            self.qc = Linear(self.rt, f"{self.prefix}.uk^T.uq", self.q_rank, self.heads * self.kv_rank)
            self.qc.bind_tensor(merged.to(self.uq.weight.dtype).contiguous())
            self.uq.weight = None                   # the two maps are not needed apart
            self.uk_t = None

    def cache_request(self) -> KVPages:
        return KVPages(1, self.kv_rank, 0, shared=True)

    # The tile lists of the tensor-core attention kernels, as grouped-query attention makes them for a group of query
    # heads on one key/value head.  All heads read the one cached "head"; more than 16 of them are cut into `share`
    # equal groups of at most 16 (the rows of the decode kernels' tiles), each of which reads it on its own.  The work
    # items of the prompt kernel ("big") stay those of all heads together.
    @property
    def share(self) -> int:
        if self.heads <= DECODE_ROWS:
            return 1
        return next((s for s in range(2, self.heads + 1) if self.heads % s == 0 and self.heads // s <= DECODE_ROWS), 1)

    def plan_key(self) -> Optional[Hashable]:
        if not self.rt.fast_kernels or self.heads // self.share > TILE_ROWS:
            return None
        return ("attention tiles", self.heads, self.share)

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        share = self.share
        key = (self.heads, share, len(batch.q_lens)) if batch.max_q_len == 1 else None
        if key is not None and key in self._plans_of_single_tokens:
            return self._plans_of_single_tokens[key]
        plan = plan_tiles(batch, self.heads // share)
        if share > 1 and "big" in plan.arrays:
            whole = plan_tiles(batch, self.heads)
            plan.arrays["big"] = whole.arrays["big"]
            plan.host["rows"]["big"] = whole.host["rows"]["big"]
        if key is not None:
            self._plans_of_single_tokens[key] = plan
        return plan

    _plans_of_single_tokens: dict = {}

    def forward(self, u: torch.Tensor, step: StepContext, cache: KVCacheView, write_cache: bool = True) -> torch.Tensor:
        rt = self.rt
        T, H = u.shape[0], self.heads
        if not write_cache:
            raise ops.KernelError("latent attention always writes its own latents")
        table = step.block_tables[cache.group]
        pre = self.down.forward(u, out_dtype=torch.float32)                  # [T, q_rank + kv_rank + H * vdim]
        c_q = rt.empty((T, self.q_rank))
        ops.latent_norm(pre, 0, self.q_rank, self.q_rank, self.kv_rank, self.q_norm_w, self.kv_norm_w, c_q, cache.k,
                        step, table, cache.page_size, self.eps, rt.stream)
        if self.qc is not None:
            q_lat = self.qc.forward(c_q).view(T, H, self.kv_rank)
        else:
            q = self.uq.forward(c_q).view(T, H, self.dim)
            q_lat = rt.empty((T, H, self.kv_rank))
            ops.gemm_heads(q_lat, q, self.uk_t, rt.stream)                   # the head's key map, applied to the query
        mix = rt.empty((T, H, self.kv_rank))
        ops.attention(q_lat, mix, cache.k, cache.v, step, cache.group, H, 1, self.kv_rank, cache.page_size, 0,
                      self.scale, rt.stream, plan=step.plans.get(self.plan_key()), kv_share=self.share)
        gated = rt.empty((T, H, self.vdim))
        ops.gemm_heads(gated, mix, self.uv, rt.stream, gate=pre[:, self.q_rank + self.kv_rank:])
        return self.o.forward(gated.view(T, H * self.vdim))
