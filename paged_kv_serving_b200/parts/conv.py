"""A short causal convolution over time in front of a mixer."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext

__all__ = ["ResidualCausalConv"]


@register_part("mixer", "residual_causal_conv")
class ResidualCausalConv(Part):
    """``h <- h + conv(h)``: per channel, ``conv(h)[t] = sum_j w[:, j] * h[t - taps + 1 + j]`` with
    zeros before the start of the sequence (``weight [width, taps]``, no bias; the last tap is on
    the token itself). The last ``taps - 1`` inputs of a request are its state, named ``tail`` in
    the layer call's binding (``state_requests``), so that a sequence may arrive in portions."""

    graph_safe = True
    STATE = "conv_tail"

    def __init__(self, width: int, taps: int) -> None:
        if taps < 1 or taps > 16:
            raise ValueError("the convolution takes 1 to 16 taps")
        self.width, self.taps = int(width), int(taps)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width, self.taps), "vector")}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"].contiguous()
        self.weight_t = self.weight.t().contiguous()          # [taps, width], what the 16-byte kernel reads

    def state_requests(self) -> dict[str, StateRequest]:
        if self.taps == 1:
            return {}
        return {self.STATE: StateRequest((self.taps - 1, self.width), "compute")}

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        state = ctx.states[binding.extra[self.STATE]] if self.taps > 1 else None
        return mixer_ops.conv_residual(x, self.weight, state, ctx.ints(ctx.TOKEN_SEQ), ctx.ints(ctx.SEQ_STARTS),
                                       ctx.ints(ctx.STATE_SLOTS), self.weight_t)
