"""Typed configuration of the Revupel design, read from the ``config.json`` of a model folder.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``layers`` (each with ``type``, ``mixer``
and ``mlp``), and the optional sections ``canon.taps`` (input convolution), ``token_side.dim``
(per-layer token input) and ``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop - 1``
run ``times`` times in a row). The class keeps the file's content as it is (``to_dict`` returns
it) and checks that every key it meets is one the design knows.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

__all__ = ["RevupelConfig"]

_TOP = {"architecture", "vocab", "width", "norm", "layers", "canon", "token_side", "loop", "max_positions"}
_MIXERS = {
    "latent_attention": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"},
    "mlstm": {"heads", "dim", "vdim", "gate_cap"},
}
#: Positions an engine may be asked for when the file sets no bound of its own: the rotation's
#: angles are computed from the position, no table limits them.
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be an integer >= 1, found {value!r}")
    return value


@dataclass(frozen=True)
class RevupelConfig:
    data: dict = field(repr=False)
    architecture: str = "Revupel"

    def __post_init__(self) -> None:
        d = self.data
        unknown = sorted(set(d) - _TOP)
        if unknown:
            raise ValueError(f"unknown model config fields: {', '.join(unknown)}")
        for key in ("vocab", "width", "norm", "layers"):
            if key not in d:
                raise ValueError(f"missing model config field: {key}")
        _positive_int(d["vocab"], "vocab")
        _positive_int(d["width"], "width")
        if not float(d["norm"]["eps"]) > 0.0:
            raise ValueError("norm.eps must be > 0")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ValueError("layers must be a non-empty list")
        for i, layer in enumerate(d["layers"]):
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
            mixer = layer.get("mixer") or {}
            bad = sorted(set(mixer) - _MIXERS[kind])
            lacking = sorted(_MIXERS[kind] - set(mixer))
            if bad or lacking:
                raise ValueError(f"layer {i} ({kind}): unknown keys {bad}, missing keys {lacking}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
                elif mlp.get("kind") == "moe":
                    _positive_int(mlp["expert"]["ff"], f"layer {i}: mlp.expert.ff")
                    experts = _positive_int(mlp["router"]["experts"], f"layer {i}: mlp.router.experts")
                    top = _positive_int(mlp["router"]["top"], f"layer {i}: mlp.router.top")
                    if top > experts:
                        raise ValueError(f"layer {i}: a token cannot use more experts than there are")
                    if mlp.get("shared"):
                        _positive_int(mlp["shared"]["ff"], f"layer {i}: mlp.shared.ff")
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        if d.get("canon"):
            _positive_int(d["canon"]["taps"], "canon.taps")
        if d.get("token_side"):
            _positive_int(d["token_side"]["dim"], "token_side.dim")
        loop = d.get("loop")
        if loop:
            start, stop, times = loop["start"], loop["stop"], _positive_int(loop["times"], "loop.times")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start <= stop <= len(d["layers"])):
                raise ValueError("loop.start and loop.stop must bound a range of layers")
        if "max_positions" in d:
            _positive_int(d["max_positions"], "max_positions")

    # --- what the engine and the command line ask of any configuration ---------------------

    @property
    def vocab_size(self) -> int:
        return self.data["vocab"]

    @property
    def d_model(self) -> int:
        return self.data["width"]

    @property
    def max_seq_len(self) -> int:
        return int(self.data.get("max_positions", DEFAULT_MAX_POSITIONS))

    @property
    def n_layers(self) -> int:
        return len(self.data["layers"])

    def run_order(self) -> list[int]:
        """Layer numbers in the order they run."""
        count = len(self.data["layers"])
        loop = self.data.get("loop")
        if not loop:
            return list(range(count))
        start, stop, times = loop["start"], loop["stop"], loop["times"]
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))

    def to_dict(self) -> dict[str, Any]:
        out = copy.deepcopy(self.data)
        out["architecture"] = self.architecture
        return out

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "RevupelConfig":
        data = copy.deepcopy(dict(data))
        name = data.get("architecture", "Revupel")
        return cls(data, architecture=name)
