"""What a layer adds for the token itself, behind its sublayers.

``gated_token_rows``: a row ``e`` of a table per token (its columns ``[column, column + dim)``: one table
may serve every layer, each with columns of its own), gated by the residual stream: ``proj(gelu_tanh(gate x)
* e)``.  The block puts the result through a norm of its own on the way into the residual.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from ..kernels import grouped
from .base import TOKEN_SIDES, PartEnv, StepContext, TokenSide, WeightInfo


@TOKEN_SIDES.register("gated_token_rows")
class GatedTokenRows(TokenSide):
    """params: ``vocab_size``, ``dim``, ``column`` (first column of this layer's part of a table row),
    ``table_width`` (columns of the table), ``table_name`` (default ``/side.embed``: a leading ``/`` marks
    a tensor's whole name, outside the part's prefix), ``weight_names`` (gate ``[dim, hidden]``, proj
    ``[hidden, dim]``; default ``gate``, ``proj``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.dim = int(params["dim"])
        self.column = int(params.get("column", 0))
        self.table_width = int(params.get("table_width", self.dim))
        if self.column < 0 or self.column + self.dim > self.table_width:
            raise ValueError(f"columns {self.column} to {self.column + self.dim} of a table of {self.table_width}")
        self.table_name = str(params.get("table_name", "/side.embed"))
        self.names = tuple(params.get("weight_names", ("gate", "proj")))
        self.table = self.gate = self.proj = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        gate, proj = self.names
        return {self.table_name: WeightInfo((self.vocab_size, self.table_width)),
                gate: WeightInfo((self.dim, self.env.hidden_size)), proj: WeightInfo((self.env.hidden_size, self.dim))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, proj = self.names
        self.table = tensors[self.table_name]           # the very tensor every layer holds
        self.gate, self.proj = tensors[gate].contiguous(), tensors[proj].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if ctx.token_ids is None:
            raise ValueError("a token side needs the step's token ids (StepContext.token_ids)")
        tokens = x.shape[0]
        gate = torch.empty((tokens, self.dim), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.gate, gate)
        gated = torch.empty_like(gate)
        grouped.gelu_gate_rows(gate, self.table, ctx.token_ids, gated, self.column)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(gated, self.proj, out)
        return out
