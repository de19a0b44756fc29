"""Typed configuration of the Tiburax design, read from the ``config.json`` of a model folder.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``, each
layer with ``type`` ("attention" or "mamba1"), the mixer's sizes and constants under ``mixer``, and
``mlp`` (a routed feed-forward, or null for none). The class keeps the file's content as it is
(``to_dict`` returns it) and checks that every key it meets is one the design knows.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

__all__ = ["TiburaxConfig"]

_TOP = {"architecture", "vocab", "width", "norm", "embedding", "layers", "max_positions"}
_REQUIRED = {
    "attention": {"heads", "kv_heads", "dim", "vdim", "scale"},
    "mamba1": {"inner", "state", "dt_rank", "conv"},
}
#: (no mask: every earlier position is visible; no rot: no rotation; no softcap: scores as they are)
_OPTIONAL = {"attention": {"mask", "rot", "softcap", "v_mix"}, "mamba1": set()}
#: Positions an engine may be asked for when the file sets no bound of its own: the rotation's
#: angles are computed from the position, no table limits them.
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be an integer >= 1, found {value!r}")
    return value


@dataclass(frozen=True)
class TiburaxConfig:
    data: dict = field(repr=False)
    architecture: str = "Tiburax"

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
        if d.get("embedding") is not None and not float(d["embedding"].get("scale", 1.0)) > 0.0:
            raise ValueError("embedding.scale must be > 0")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ValueError("layers must be a non-empty list")
        for i, layer in enumerate(d["layers"]):
            kind = layer.get("type")
            if kind not in _REQUIRED:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(sorted(_REQUIRED))}")
            mixer = layer.get("mixer") or {}
            bad = sorted(set(mixer) - _REQUIRED[kind] - _OPTIONAL[kind])
            lacking = sorted(_REQUIRED[kind] - set(mixer))
            if bad or lacking:
                raise ValueError(f"layer {i} ({kind}): unknown keys {bad}, missing keys {lacking}")
            if kind == "attention":
                heads = _positive_int(mixer["heads"], f"layer {i}: heads")
                groups = _positive_int(mixer["kv_heads"], f"layer {i}: kv_heads")
                if heads % groups:
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
                dim = _positive_int(mixer["dim"], f"layer {i}: dim")
                _positive_int(mixer["vdim"], f"layer {i}: vdim")
                mask = mixer.get("mask") or {}
                if mask.get("size") is not None:
                    _positive_int(mask["size"], f"layer {i}: mask.size")
                if int(mask.get("keep_first") or 0) < 0:
                    raise ValueError(f"layer {i}: mask.keep_first must be >= 0")
                rot = mixer.get("rot") or {}
                dims = int(rot.get("dims") or 0)
                if dims < 0 or dims % 2 or dims > dim:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
                if rot.get("scaling"):
                    for key in ("factor", "original", "fast", "slow"):
                        if key not in rot["scaling"]:
                            raise ValueError(f"layer {i}: rot.scaling lacks {key}")
            else:
                for key in ("inner", "state", "dt_rank", "conv"):
                    _positive_int(mixer[key], f"layer {i}: {key}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                _positive_int(mlp["expert"]["ff"], f"layer {i}: mlp.expert.ff")
                experts = _positive_int(mlp["router"]["experts"], f"layer {i}: mlp.router.experts")
                top = _positive_int(mlp["router"]["top"], f"layer {i}: mlp.router.top")
                if top > experts:
                    raise ValueError(f"layer {i}: a token cannot use more experts than there are")
                if mlp.get("shared"):
                    _positive_int(mlp["shared"]["ff"], f"layer {i}: mlp.shared.ff")
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

    @property
    def embedding_scale(self) -> float:
        return float((self.data.get("embedding") or {}).get("scale", 1.0))

    def to_dict(self) -> dict[str, Any]:
        out = copy.deepcopy(self.data)
        out["architecture"] = self.architecture
        return out

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "TiburaxConfig":
        data = copy.deepcopy(dict(data))
        name = data.get("architecture", "Tiburax")
        return cls(data, architecture=name)
