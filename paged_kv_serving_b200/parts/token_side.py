"""A per-layer input that depends on the token itself, added to the stream behind a layer."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm, mixer_ops
from paged_kv_serving_b200.parts.base import ParamSpec, Part, StepContext

__all__ = ["TokenSideInput", "TokenSideTable"]


class TokenSideTable(Part):
    """The table all layers share: row ``token`` holds ``layers * dim`` numbers, layer ``i``
    reads ``[i * dim, (i + 1) * dim)``."""

    graph_safe = True

    def __init__(self, vocab_size: int, columns: int) -> None:
        self.vocab_size, self.columns = int(vocab_size), int(columns)
        self.table: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"table": ParamSpec((self.vocab_size, self.columns))}


@register_part("mixer", "token_side_input")
class TokenSideInput(Part):
    """``x <- x + rmsnorm(proj(gelu_tanh(gate x) * e)) * weight`` with ``e`` the layer's slice of
    the token's row in a ``TokenSideTable``; ``gate [dim, width]``, ``proj [width, dim]``, an
    ordinary RMS norm weight ``[width]``. ``x`` is the stream itself (not a norm of it): the
    pending update of the layer is added first. ``forward`` returns the new pending update."""

    graph_safe = True
    #: Steps of at most this many tokens run the whole side input as one kernel (a block a token)
    #: instead of two library products with the element-wise kernels between them. Off (0): measured
    #: inside captured decode steps of 8 requests the one kernel is slower than the five launches it
    #: replaces (0.68 against 0.60 ms a step at width 2,048, 1.37 against 1.20 at 4,096): a block a
    #: token leaves the two matrices to eight SMs. Tests run it.
    FUSED_ROWS = 0

    def __init__(self, width: int, dim: int, slice_index: int, table: TokenSideTable, eps: float) -> None:
        self.width, self.dim, self.slice_index, self.table, self.eps = int(width), int(dim), int(slice_index), table, float(eps)
        self.gate: torch.Tensor | None = None
        self.proj: torch.Tensor | None = None
        self.norm: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"gate": ParamSpec((self.dim, self.width)), "proj": ParamSpec((self.width, self.dim)),
                "norm": ParamSpec((self.width,), "vector")}

    def forward(self, hidden: torch.Tensor, pending: torch.Tensor | None, ctx: StepContext,
                bias: torch.Tensor | None = None) -> torch.Tensor:
        fed_back_at = ctx.ints(ctx.TOKEN_FEEDBACK) if ctx.fed_back_ids is not None else None
        if hidden.shape[0] <= self.FUSED_ROWS:
            return mixer_ops.token_side(hidden, pending, bias, self.gate, self.proj, self.table.table, ctx.ints(ctx.TOKEN_IDS),
                                        self.slice_index * self.dim, self.norm, self.eps, "gelu_tanh", ctx.status,
                                        ctx.fed_back_ids if fed_back_at is not None else None, fed_back_at)
        x = mixer_ops.residual_add(hidden, pending, bias, out_dtype=ctx.dtype)
        z = gemm.linear(x, self.gate)
        g = mixer_ops.act_times_table(z, self.table.table, ctx.ints(ctx.TOKEN_IDS), self.slice_index * self.dim, "gelu_tanh",
                                      ctx.status, ctx.fed_back_ids if fed_back_at is not None else None, fed_back_at)
        y = gemm.linear(g, self.proj, out_dtype=torch.float32)
        # the norm of y itself (not of the stream): the add-and-norm kernel without an addend
        return ops.add_rmsnorm(y, None, self.norm, self.eps, torch.float32)
