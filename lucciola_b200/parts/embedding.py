"""Token embedding and output head."""
from __future__ import annotations

from typing import Callable

import torch

from .. import ops
from .base import ParamSpec, Part, Runtime
from .linear import Linear


class TokenEmbedding(Part):
    """residual[t, :] = table[id_t, :], unscaled (src/kernels/embedding.cu:22-38 of lucciola), as float32.
    With `positions_name` the model has a table of learned position vectors [max_positions, hidden], and
    residual[t, :] += positions[p_t, :] (unscaled, added in 32-bit); forward() then takes the tokens' positions."""
    recordable = True

    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int, positions_name: str | None = None,
                 max_positions: int = 0):
        self.rt, self.name, self.vocab_size, self.hidden_size = rt, name, vocab_size, hidden_size
        self.positions_name, self.max_positions = positions_name, max_positions
        if positions_name is not None and max_positions <= 0:
            raise ValueError("a table of position vectors needs its number of rows")
        self.weight: torch.Tensor | None = None
        self.position_table: torch.Tensor | None = None

    @property
    def uses_positions(self) -> bool:
        return self.positions_name is not None

    def param_specs(self) -> list[ParamSpec]:
        specs = [ParamSpec(self.name, (self.vocab_size, self.hidden_size), "embedding")]
        if self.positions_name is not None:
            specs.append(ParamSpec(self.positions_name, (self.max_positions, self.hidden_size), "embedding"))
        return specs

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).contiguous()
        if self.positions_name is not None:
            self.position_table = get(self.positions_name).to(self.weight.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        out = self.rt.empty((token_ids.shape[0], self.hidden_size), torch.float32)
        if self.positions_name is not None:
            if positions is None:
                raise ValueError("this embedding adds position vectors and needs the tokens' positions")
            ops.embedding(out, token_ids, self.weight, self.rt.stream, pos_table=self.position_table, positions=positions)
        else:
            ops.embedding(out, token_ids, self.weight, self.rt.stream)
        return out


class OutputHead(Part):
    """logits = h . W^T in float32; W is its own tensor or the embedding table when tied
    (src/qwen.cc:80-84 of lucciola falls back to a second copy of the table; here the table is shared)."""
    recordable = True


    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None,
                 scale: float = 1.0):
        self.rt, self.name, self.tied_to = rt, name, tied_to
        self.vocab_size = vocab_size
        self.scale = float(scale)           # the logits are multiplied by this, in 32-bit
        self.proj = Linear(rt, name, hidden_size, vocab_size)

    def param_specs(self) -> list[ParamSpec]:
        return [] if self.tied_to is not None else self.proj.param_specs()

    def ignored_names(self) -> list[str]:
        """A tied head does not need its own tensor; a checkpoint may carry one all the same."""
        return [self.name] if self.tied_to is not None else []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.tied_to is not None:
            self.proj.bind_tensor(self.tied_to.weight)
        else:
            self.proj.bind(get)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.proj.forward(h, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_(logits, self.scale, self.rt.stream)
        return logits
