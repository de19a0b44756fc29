"""A plain, slow implementation of the Revupel design: one function per mechanism, written from
the design's equations in float64 on the CPU, token by token where a mechanism has a state.

It shares no code with the product path. ``forward`` runs whole sequences and returns the logits
of every position (and, on request, the residual stream after every layer run). Notation:
``x`` the residual stream ``[tokens, width]``, ``h`` what a mixer or feed-forward reads,
weights ``[out, in]`` applied as ``h @ W.T``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(tensors, name):
    return tensors[name].to(F64)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is one number for all coordinates."""
    return rms(x, eps) * g.reshape(())


def input_convolution(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h + conv(h): per channel, conv(h)[t] = sum_j w[:, j] h[t - taps + 1 + j], zeros before 0."""
    tokens, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(tokens):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary positions on the first ``dims`` coordinates of the last axis: coordinate i pairs
    with i + dims/2; v is [tokens, ..., size], positions [tokens]."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]                      # [tokens, half]
    while angle.dim() < v.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, w = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = u * cos - w * sin
    out[..., half:dims] = w * cos + u * sin
    return out


def latent_attention(h: torch.Tensor, tensors, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    heads, dim, rot_dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    c_q = rms(h @ _w(tensors, prefix + "dq").T, eps) * _w(tensors, prefix + "dq.norm")
    q = (c_q @ _w(tensors, prefix + "uq").T).view(tokens, heads, dim + rot_dim)
    down = h @ _w(tensors, prefix + "dkv").T
    c = rms(down[:, :rank], eps) * _w(tensors, prefix + "dkv.norm")
    k_rot = rotate_half(down[:, rank:], positions, mixer["rot"]["dims"], mixer["rot"]["base"])
    q_plain = q[..., :dim]
    q_rot = rotate_half(q[..., dim:], positions, mixer["rot"]["dims"], mixer["rot"]["base"])
    k_plain = (c @ _w(tensors, prefix + "uk").T).view(tokens, heads, dim)
    v = (c @ _w(tensors, prefix + "uv").T).view(tokens, heads, vdim)
    gate = torch.sigmoid(h @ _w(tensors, prefix + "g").T)                  # [tokens, heads]
    out = torch.zeros(tokens, heads, vdim, dtype=F64)
    for t in range(tokens):
        for a in range(heads):
            score = (k_plain[:t + 1, a] @ q_plain[t, a] + k_rot[:t + 1] @ q_rot[t, a]) * mixer["scale"]
            weight = torch.softmax(score, dim=0)
            out[t, a] = (weight[:, None] * v[:t + 1, a]).sum(dim=0) * gate[t, a]
    return out.reshape(tokens, heads * vdim) @ _w(tensors, prefix + "o").T


def mlstm(h: torch.Tensor, tensors, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    heads, dim, vdim, cap = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["gate_cap"]
    tokens = h.shape[0]
    q = (h @ _w(tensors, prefix + "q").T).view(tokens, heads, dim) * dim ** -0.5
    k = (h @ _w(tensors, prefix + "k").T).view(tokens, heads, dim)
    v = (h @ _w(tensors, prefix + "v").T).view(tokens, heads, vdim)
    log_i = cap * torch.tanh((h @ _w(tensors, prefix + "i").T + _w(tensors, prefix + "i.b")) / cap)
    log_f = torch.nn.functional.logsigmoid(
        cap * torch.tanh((h @ _w(tensors, prefix + "f").T + _w(tensors, prefix + "f.b")) / cap))
    out = torch.zeros(tokens, heads, vdim, dtype=F64)
    for a in range(heads):
        S = torch.zeros(dim, vdim, dtype=F64)
        n = torch.zeros(dim, dtype=F64)
        m = 0.0
        for t in range(tokens):
            i, f = float(log_i[t, a]), float(log_f[t, a])
            m_new = max(f + m, i)
            keep, take = math.exp(f + m - m_new), math.exp(i - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            m = m_new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(float(n @ q[t, a])), math.exp(-m)) + 1e-6)
    out = rms(out, eps).reshape(tokens, heads * vdim) * _w(tensors, prefix + "norm")
    out = out * torch.sigmoid(h @ _w(tensors, prefix + "g").T)
    return out @ _w(tensors, prefix + "o").T


def dense_feed_forward(h: torch.Tensor, tensors, prefix: str) -> torch.Tensor:
    inner = gelu_erf(h @ _w(tensors, prefix + "up").T + _w(tensors, prefix + "up.b"))
    return inner @ _w(tensors, prefix + "down").T + _w(tensors, prefix + "down.b")


def _expert(h, tensors, prefix):
    return torch.relu(h @ _w(tensors, prefix + "up").T) ** 2 @ _w(tensors, prefix + "down").T


def routed_feed_forward(h: torch.Tensor, tensors, prefix: str, mlp: dict) -> torch.Tensor:
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    score = torch.softmax(h @ _w(tensors, prefix + "router").T, dim=-1)
    out = torch.zeros(h.shape[0], _w(tensors, prefix + "e0.down").shape[0], dtype=F64)
    for t in range(h.shape[0]):
        chosen = sorted(range(experts), key=lambda e: (-float(score[t, e]), e))[:top]
        for e in chosen:
            out[t] += score[t, e] * _expert(h[t:t + 1], tensors, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        share = torch.sigmoid(h @ _w(tensors, prefix + "shared.sg").T)          # [tokens, 1]
        out = out + share * _expert(h, tensors, prefix + "shared.")
    return out


def token_side_input(x: torch.Tensor, tokens: torch.Tensor, tensors, layer: int, dim: int, eps: float) -> torch.Tensor:
    """The update the per-layer token input adds to the stream."""
    e = _w(tensors, "side.embed")[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ _w(tensors, f"l{layer}.side.gate").T) * e
    y = g @ _w(tensors, f"l{layer}.side.proj").T
    return rms(y, eps) * _w(tensors, f"l{layer}.side.norm")


def run_order(config: dict) -> list[int]:
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def forward(config: dict, tensors: dict, token_ids, return_layers: bool = False):
    """Logits [tokens, vocab] of one sequence run from position 0 (float64)."""
    tokens = torch.as_tensor(token_ids, dtype=torch.long)
    eps = config["norm"]["eps"]
    x = _w(tensors, "embed")[tokens]
    after = []
    for layer in run_order(config):
        spec, p = config["layers"][layer], f"l{layer}."
        h = scalar_norm(x, _w(tensors, p + "norm1"), eps)
        if config.get("canon"):
            h = input_convolution(h, _w(tensors, p + "canon1"))
        if spec["type"] == "latent_attention":
            x = x + latent_attention(h, tensors, p + "mix.", spec["mixer"], eps)
        elif spec["type"] == "mlstm":
            x = x + mlstm(h, tensors, p + "mix.", spec["mixer"], eps)
        else:
            raise ValueError(spec["type"])
        mlp = spec.get("mlp")
        if mlp:
            h = scalar_norm(x, _w(tensors, p + "norm2"), eps)
            if mlp["kind"] == "dense":
                x = x + dense_feed_forward(h, tensors, p + "mlp.")
            else:
                x = x + routed_feed_forward(h, tensors, p + "mlp.", mlp)
        if config.get("token_side"):
            x = x + token_side_input(x, tokens, tensors, layer, config["token_side"]["dim"], eps)
        after.append(x.clone())
    logits = scalar_norm(x, _w(tensors, "final.norm"), eps) @ _w(tensors, "head").T
    if return_layers:
        return logits, torch.stack(after)
    return logits
