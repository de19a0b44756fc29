"""Position-encoding parts."""

from __future__ import annotations

import numpy as np
import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.parts.base import Part

__all__ = ["NoPositionEncoding", "PositionEncoding", "RotaryEncoding", "ScaledRotaryFrequencies"]


class PositionEncoding(Part):
    """Interface of a position encoding used by an attention mixer.

    ``fused_tables`` returns ``(cos, sin)`` float32 tables ``[positions, rotated/2]`` when the
    encoding is a half-split rotation of queries and keys that the attention kernels apply
    themselves; an encoding of another kind returns ``None`` and implements ``apply_qk``, which
    rewrites the query and key columns of the fused ``qkv`` buffer in place before the keys are
    stored. Keys are cached after encoding, so an encoding must depend on a key's own absolute
    position only.
    """

    graph_safe = True

    def fused_tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor] | None:
        return None

    def apply_qk(self, qkv: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv: int, head_dim: int) -> None:
        return None


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    """Rotary encoding, half-split form: ``inv_freq_j = theta^(-2j/hd)``, ``angle = p * inv_freq_j``
    computed in float64 and cast to float32 tables, as the reference does
    (src/paged_kv_serving/engine/model.py:60-81)."""

    def __init__(self, head_dim: int, theta: float, max_positions: int) -> None:
        if head_dim % 2:
            raise ValueError("head_dim must be even for rotary position encoding")
        if not theta > 1.0:
            raise ValueError("rope theta must be > 1")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._tables: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}

    def host_tables(self) -> tuple[np.ndarray, np.ndarray]:
        half = self.head_dim // 2
        inv_freq = 1.0 / (self.theta ** (np.arange(half, dtype=np.float64) * 2.0 / self.head_dim))
        angles = np.outer(np.arange(self.max_positions, dtype=np.float64), inv_freq)
        return np.cos(angles).astype(np.float32), np.sin(angles).astype(np.float32)

    def fused_tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        key = str(device)
        if key not in self._tables:
            cos, sin = self.host_tables()
            self._tables[key] = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        return self._tables[key]


@register_part("position", "scaled_rotary")
class ScaledRotaryFrequencies(PositionEncoding):
    """A half-split rotation of the first ``dims`` coordinates of a head (coordinate ``i`` pairs
    with ``i + dims / 2``) by ``position * f_i`` with ``f_i = base^(-2i / dims)``, optionally
    stretched for contexts longer than the ``original`` one (YaRN; Peng, Quesnelle, Fan and
    Shippole, "YaRN: Efficient Context Window Extension of Large Language Models"):

    * pair ``i`` makes ``original * f_i / (2 pi)`` turns over the original context; the pair that
      makes ``t`` turns has the (real-valued) index ``pair(t) = dims * ln(original / (2 pi t)) / (2
      ln base)``;
    * with ``lo = max(floor(pair(fast)), 0)`` and ``hi = min(ceil(pair(slow)), dims - 1)`` the ramp
      ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` blends ``f_i`` (fast pairs, ``r = 0``)
      into ``f_i / factor`` (slow pairs, ``r = 1``);
    * cos and sin are multiplied by ``0.1 * ln(factor) + 1``.

    There is no table and no bound on positions: the kernels form ``float(position) * f_i`` in
    float32 and take accurate sines and cosines. ``frequencies`` are computed in float64 and
    rounded to float32 once.
    """

    def __init__(self, dims: int, base: float, factor: float | None = None, original: float | None = None,
                 fast: float | None = None, slow: float | None = None) -> None:
        if dims < 0 or dims % 2:
            raise ValueError("the number of rotated coordinates must be even")
        if dims and not base > 1.0:
            raise ValueError("the rotation's base must be > 1")
        self.dims, self.base = int(dims), float(base)
        self.scaling = None
        if factor is not None:
            if None in (original, fast, slow) or not factor >= 1.0:
                raise ValueError("a stretched rotation needs factor >= 1, original, fast and slow")
            self.scaling = (float(factor), float(original), float(fast), float(slow))
        self._device: dict[str, torch.Tensor] = {}

    @property
    def amplitude(self) -> float:
        """The factor on cos and sin."""
        return 0.1 * float(np.log(self.scaling[0])) + 1.0 if self.scaling else 1.0

    def frequencies(self) -> np.ndarray:
        half = self.dims // 2
        i = np.arange(half, dtype=np.float64)
        freq = self.base ** (-2.0 * i / max(self.dims, 1))
        if self.scaling is None:
            return freq
        factor, original, fast, slow = self.scaling

        def pair(turns: float) -> float:
            return self.dims * np.log(original / (2.0 * np.pi * turns)) / (2.0 * np.log(self.base))

        lo = max(int(np.floor(pair(fast))), 0)
        hi = min(int(np.ceil(pair(slow))), self.dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp)

    def device_frequencies(self, device: torch.device) -> torch.Tensor | None:
        if not self.dims:
            return None
        key = str(device)
        if key not in self._device:
            self._device[key] = torch.from_numpy(self.frequencies().astype(np.float32)).to(device)
        return self._device[key]
