"""A plain, slow implementation of the Tiburax design in float64, one function per mechanism.

It shares no code with the package: plain PyTorch on the CPU, whole sequences at once, no cache,
no state carried between calls (``mamba`` walks the tokens in a Python loop). The tests compare
the engine with it. ``tensors`` maps the names of a model folder to tensors; ``config`` is the
nested dictionary of ``config.json``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is centred on zero: the factor is ``1 + weight``."""
    return rms_unit(x, eps) * (1.0 + weight.to(F64))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Angular frequency of every rotated pair and the factor on cos and sin.

    Without ``scaling`` the frequencies are ``base^(-2i/dims)`` and the factor is 1. With it the
    frequencies of slowly turning pairs are divided by ``factor``, those of fast pairs stay, and
    a linear ramp over the pair index blends the two between the pairs that make ``fast`` and
    ``slow`` turns over ``original`` positions."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """Rotate the first ``rot.dims`` coordinates of every head of ``x [tokens, heads, dim]``;
    coordinate ``i`` pairs with ``i + dims/2``."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, factor = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None, None] * freq[None, None, :]
    cos, sin = torch.cos(angle) * factor, torch.sin(angle) * factor
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def visible(n: int, size: int, keep_first: int) -> torch.Tensor:
    """``[queries, keys]`` mask of a sliding window that also keeps the first tokens."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention(h: torch.Tensor, p: dict, m: dict, eps: float, v_first: torch.Tensor | None):
    """The attention mixer on a whole sequence ``h [tokens, width]``. ``p``: the layer's mixer
    tensors by short name. ``v_first``: the values of the first value-mixing layer, or ``None``
    when this layer is that one or does not mix. Returns ``(output, values as cached)``."""
    n = h.shape[0]
    heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = torch.arange(n)
    q = (h @ p["q"].to(F64).T).view(n, heads, dim)
    k = (h @ p["k"].to(F64).T).view(n, groups, dim)
    v = (h @ p["v"].to(F64).T).view(n, groups, vdim)
    rot = m.get("rot") or {}
    if int(rot.get("dims") or 0):
        q, k = rotate(q, positions, rot), rotate(k, positions, rot)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    if v_first is not None:
        lam = p["vmix"].to(F64)
        v = (1.0 - lam) * v + lam * v_first
    k_of_head = k.repeat_interleave(heads // groups, dim=1)
    v_of_head = v.repeat_interleave(heads // groups, dim=1)
    score = torch.einsum("ihd,jhd->hij", q, k_of_head) * float(m["scale"])
    cap = float(m.get("softcap") or 0.0)
    if cap:
        score = cap * torch.tanh(score / cap)
    window = (m.get("mask") or {}).get("size")
    mask = visible(n, int(window) if window else n, int((m.get("mask") or {}).get("keep_first") or 0))
    score = score.masked_fill(~mask[None], float("-inf"))
    weight = torch.softmax(score, dim=-1)
    out = torch.einsum("hij,jhd->ihd", weight, v_of_head).reshape(n, heads * vdim)
    return out @ p["o"].to(F64).T, v


def mamba(h: torch.Tensor, p: dict, m: dict) -> torch.Tensor:
    """The selective-scan mixer on a whole sequence, token by token."""
    n = h.shape[0]
    inner, state, rank, taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
    xz = h @ p["in"].to(F64).T
    x, z = xz[:, :inner], xz[:, inner:]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=F64), x], dim=0)
    w = p["conv"].to(F64)                                           # [inner, taps], last column = current token
    conv = sum(padded[j:j + n] * w[:, j][None, :] for j in range(taps)) + p["conv.b"].to(F64)
    x = silu(conv)
    low = x @ p["x"].to(F64).T
    dt_low, B, C = low[:, :rank], low[:, rank:rank + state], low[:, rank + state:]
    dt = softplus(dt_low @ p["dt"].to(F64).T + p["dt.b"].to(F64))   # [tokens, inner]
    A = -torch.exp(p["A_log"].to(F64))                              # [inner, state]
    S = torch.zeros(inner, state, dtype=F64)
    ys = []
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + p["D"].to(F64) * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ p["o"].to(F64).T


def gated_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.to(F64).T) * (h @ up.to(F64).T)) @ down.to(F64).T


def routed_feed_forward(h: torch.Tensor, p: dict, mlp: dict) -> torch.Tensor:
    """Mixture of gated experts: the ``top`` largest router logits choose, the softmax over the
    chosen logits weighs; a shared expert is added for every token."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ p["router"].to(F64).T + p["router.b"].to(F64)
    best, index = torch.topk(logits, top, dim=-1)
    weight = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for e in range(experts):
        share = (weight * (index == e)).sum(dim=-1, keepdim=True)
        out = out + share * gated_expert(h, p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])
    if mlp.get("shared"):
        out = out + gated_expert(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


def _layer_tensors(tensors: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """Logits ``[tokens, vocab]`` (float64) of one whole sequence; with ``return_layers`` also the
    residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = tensors["embed"].to(F64)[torch.tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    v_first = None
    streams = []
    for index, layer in enumerate(config["layers"]):
        mix = _layer_tensors(tensors, f"l{index}.mix.")
        if layer["type"] == "attention":
            mixes = bool(layer["mixer"].get("v_mix"))
            update, values = attention(x, mix, layer["mixer"], eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = values
        elif layer["type"] == "mamba1":
            update = mamba(x, mix, layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(update, tensors[f"l{index}.norm1"], eps)
        if layer.get("mlp"):
            update = routed_feed_forward(x, _layer_tensors(tensors, f"l{index}.mlp."), layer["mlp"])
            x = x + offset_norm(update, tensors[f"l{index}.norm2"], eps)
        streams.append(x)
    logits = offset_norm(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T
    return (logits, torch.stack(streams)) if return_layers else logits
