"""The selective-scan recurrent mixer of Mamba."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import arena, gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext

__all__ = ["Mamba1"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part("mixer", "mamba1")
class Mamba1(Part):
    """Selective state-space mixer (Gu and Dao, "Mamba: Linear-Time Sequence Modeling with
    Selective State Spaces"). With ``h`` the input:

    ``[x | z] = W_in h`` (``inner`` channels each); ``x <- silu(conv(x) + b_conv)``, a causal
    convolution per channel over ``taps`` tokens (the last tap on the token itself, zeros before
    the sequence); ``[dt_low | B | C] = W_x x`` (``dt_rank``, ``state``, ``state`` numbers); ``dt =
    softplus(W_dt dt_low + b_dt)`` per channel; ``A = -exp(A_log)``. Per channel ``c`` and state
    coordinate ``n``: ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``, ``y_c = sum_n S[c, n]
    C_n + D_c x_c``; the output is ``W_o (y * silu(z))``.

    ``S`` (float32, zero at the start of a sequence) and the convolution's last ``taps - 1``
    inputs are states of the layer call (``state_requests``), so a sequence may arrive in portions
    or token by token; the scan applies the same operations in the same order however it is cut.
    Step sizes, decays, ``B``, ``C`` and the state are float32; the projections take operands in
    the compute type and keep float32 results where the recurrence reads them.
    """

    graph_safe = True
    STATE, TAIL = "mamba_state", "mamba_conv_tail"

    def __init__(self, width: int, inner: int, state: int, dt_rank: int, taps: int) -> None:
        if min(width, inner, state, dt_rank, taps) < 1:
            raise ValueError("every size of the mixer must be >= 1")
        if taps > 16 or state > 256:
            raise ValueError("the kernels take up to 16 taps and 256 state coordinates per channel")
        self.width, self.inner, self.state, self.dt_rank, self.taps = int(width), int(inner), int(state), int(dt_rank), int(taps)
        # rows of the fused low-rank projection: dt_low padded to a multiple of 8 (the product that
        # reads it wants rows of 16 bytes), then B, then C
        self.rank_padded = _round_up(self.dt_rank, 8)
        self.b_at, self.c_at = self.rank_padded, self.rank_padded + self.state
        self.low_rows = _round_up(self.rank_padded + 2 * self.state, 8)

    def param_specs(self) -> dict[str, ParamSpec]:
        return {
            "in_proj": ParamSpec((2 * self.inner, self.width)),
            "conv": ParamSpec((self.inner, self.taps), "vector", init=(0.0, 0.4)),
            "conv_b": ParamSpec((self.inner,), "vector", init=(0.0, 0.1)),
            "x_proj": ParamSpec((self.dt_rank + 2 * self.state, self.inner)),
            "dt_proj": ParamSpec((self.inner, self.dt_rank)), "dt_b": ParamSpec((self.inner,), "vector", init=(-2.0, 0.5)),
            "A_log": ParamSpec((self.inner, self.state), "vector", init=(0.0, 0.5)),
            "D": ParamSpec((self.inner,), "vector", init=(1.0, 0.1)),
            "o": ParamSpec((self.width, self.inner)),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.in_proj = params["in_proj"].contiguous()
        self.conv = params["conv"].contiguous()
        self.conv_t = self.conv.t().contiguous()
        self.conv_b = params["conv_b"].contiguous()
        x_proj = params["x_proj"]
        low = torch.zeros((self.low_rows, self.inner), dtype=x_proj.dtype, device=x_proj.device)
        low[:self.dt_rank] = x_proj[:self.dt_rank]
        low[self.b_at:self.b_at + 2 * self.state] = x_proj[self.dt_rank:]
        self.x_proj = low
        dt_proj = torch.zeros((self.inner, self.rank_padded), dtype=x_proj.dtype, device=x_proj.device)
        dt_proj[:, :self.dt_rank] = params["dt_proj"]
        self.dt_proj = dt_proj
        self.dt_b = params["dt_b"].contiguous()
        self.A = (-torch.exp(params["A_log"].to(torch.float32))).contiguous()       # the decay rates, float32
        self.D = params["D"].contiguous()
        self.o = params["o"].contiguous()

    def state_requests(self) -> dict[str, StateRequest]:
        requests = {self.STATE: StateRequest((self.inner, self.state))}
        if self.taps > 1:
            requests[self.TAIL] = StateRequest((self.taps - 1, self.inner), "compute")
        return requests

    def forward(self, h: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        starts, slots = ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS)
        xz = gemm.linear(h, self.in_proj, chain=True)                                           # [tokens, 2 inner]
        tail = ctx.states[binding.extra[self.TAIL]] if self.taps > 1 else None
        x = mixer_ops.conv_residual(xz[:, :self.inner], self.conv, tail, ctx.ints(ctx.TOKEN_SEQ), starts, slots, self.conv_t,
                                    bias=self.conv_b, residual=False, act="silu")
        low = gemm.linear(x, self.x_proj, out_dtype=torch.float32, few_rows_f32=True, chain=True)                  # [tokens, dt_low | B | C]
        if ctx.dtype == torch.float32:
            dt_low = low[:, :self.rank_padded]
            dt_pre = gemm.matmul(dt_low, self.dt_proj.t())
        else:
            dt_low = arena.empty((low.shape[0], self.rank_padded), ctx.dtype, low.device)
            dt_low.copy_(low[:, :self.rank_padded])
            dt_pre = gemm.linear(dt_low, self.dt_proj, out_dtype=torch.float32, few_rows_f32=True, chain=True)     # [tokens, inner], before bias and softplus
        y = mixer_ops.selective_scan(x, xz[:, self.inner:], dt_pre, self.dt_b, low, self.b_at, self.c_at, self.A, self.D,
                                     ctx.states[binding.extra[self.STATE]], starts, slots)
        # the float32 result of the last product goes to a norm
        return gemm.linear(y, self.o, out_dtype=torch.float32, few_rows_f32=True, chain=True)
