"""The matrix-memory recurrent mixer of xLSTM."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext

__all__ = ["MLSTM"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part("mixer", "mlstm")
class MLSTM(Part):
    """Matrix memory (mLSTM): per head a state ``S [dim, vdim]``, a normaliser ``n [dim]`` and a
    running maximum ``m`` of the log gates, all float32 and all starting at zero.

    ``q = W_q h * dim^-1/2``, ``k = W_k h``, ``v = W_v h``; log input gate ``i = cap * tanh((W_i h +
    b_i) / cap)``, log forget gate ``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``. Per token:
    ``m' = max(f + m, i)``, ``S' = exp(f + m - m') S + exp(i - m') k v^T``, ``n'`` likewise with
    ``k`` alone, ``o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)``. Each head's ``o`` is divided
    by its root mean square, the heads are multiplied by ``norm`` and ``sigmoid(W_g h)`` and go
    through ``W_o``. The three states are further states of the layer call (``state_requests``);
    the recurrence runs token by token in the kernels whether the tokens arrive as a prompt, in
    portions or one at a time, so the result does not depend on the cut.
    """

    graph_safe = True
    #: The output projection may carry the caller's residual add and norm (``finish``, see ``Part``).
    fuses_last_linear = True
    chains_last_linear = False

    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float) -> None:
        if dim > 1024:
            raise ValueError("the mLSTM kernels take a key size of up to 1024")
        self.width, self.heads, self.dim, self.vdim = int(width), int(heads), int(dim), int(vdim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        self.offsets = {"q": 0, "k": qk, "v": 2 * qk, "g": 2 * qk + vg, "i": 2 * qk + 2 * vg, "f": 2 * qk + 2 * vg + self.heads}
        self.fused_rows = _round_up(2 * qk + 2 * vg + 2 * self.heads, 8)

    def param_specs(self) -> dict[str, ParamSpec]:
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        return {
            "q": ParamSpec((qk, self.width)), "k": ParamSpec((qk, self.width)), "v": ParamSpec((vg, self.width)),
            "g": ParamSpec((vg, self.width)), "o": ParamSpec((self.width, vg)), "norm": ParamSpec((vg,), "vector"),
            "i": ParamSpec((self.heads, self.width)), "i_b": ParamSpec((self.heads,), "vector"),
            "f": ParamSpec((self.heads, self.width)), "f_b": ParamSpec((self.heads,), "vector"),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        q = params["q"]
        fused = torch.zeros((self.fused_rows, self.width), dtype=q.dtype, device=q.device)
        for name in ("q", "k", "v", "g", "i", "f"):
            fused[self.offsets[name]:self.offsets[name] + params[name].shape[0]] = params[name]
        self.fused = fused
        self.o = params["o"].contiguous()
        self.norm, self.i_b, self.f_b = params["norm"], params["i_b"], params["f_b"]

    def state_requests(self) -> dict[str, StateRequest]:
        return {"mlstm_S": StateRequest((self.heads, self.vdim, self.dim)), "mlstm_n": StateRequest((self.heads, self.dim)),
                "mlstm_m": StateRequest((self.heads,))}

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, finish=None) -> torch.Tensor:
        # the gates' pre-activations and everything else that enters the recurrence stay float32
        proj = gemm.linear(x, self.fused, out_dtype=torch.float32)
        states = ctx.states
        out = mixer_ops.mlstm(proj, self.offsets, self.i_b, self.f_b, self.norm, self.gate_cap, self.dim ** -0.5, self.eps,
                              states[binding.extra["mlstm_S"]], states[binding.extra["mlstm_n"]],
                              states[binding.extra["mlstm_m"]], ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS),
                              self.heads, self.dim, self.vdim, ctx.dtype)
        return finish(out, self.o) if finish is not None else gemm.linear(out, self.o)
