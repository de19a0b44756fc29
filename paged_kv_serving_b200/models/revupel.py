"""The Revupel design: a decoder whose layers alternate, in an order the configuration lists,
between attention over a cached latent and a matrix-memory recurrence (mLSTM), each behind a
short causal convolution of the mixer's input, with dense or routed feed-forwards, a per-layer
input that depends on the token itself, norms whose weight is one number, and a span of layers
that runs several times with the same weights (every pass with its own cache and state).

This module is all that is specific to the design: which parts a layer has, with which numbers
of the configuration, the run order, and the tensor names of a model folder (``embed``, ``head``,
``final.norm``, ``side.embed``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``).
"""

from __future__ import annotations

from paged_kv_serving_b200.config.registry import register_architecture
from paged_kv_serving_b200.config.revupel_config import RevupelConfig
from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
from paged_kv_serving_b200.parts import (
    MLSTM, BiasedDense, ConvSideBlock, LatentAttention, ResidualCausalConv, RoutedExperts, ScalarRMSNorm, TokenSideInput,
    TokenSideTable,
)

__all__ = ["Revupel"]


def _mixer(kind: str, sizes: dict, width: int, eps: float):
    """The mixer of a layer and the map from its tensors' names in the file to the part's."""
    if kind == "latent_attention":
        part = LatentAttention(width, sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["q_rank"],
                               sizes["kv_rank"], sizes["scale"], sizes["rot"]["base"], sizes["rot"]["dims"], eps)
        names = {"dq": "dq", "dq.norm": "dq_norm", "uq": "uq", "dkv": "dkv", "dkv.norm": "dkv_norm", "uk": "uk", "uv": "uv",
                 "g": "g", "o": "o"}
    elif kind == "mlstm":
        part = MLSTM(width, sizes["heads"], sizes["dim"], sizes["vdim"], sizes["gate_cap"], eps)
        names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "i.b": "i_b", "f": "f",
                 "f.b": "f_b"}
    else:
        raise ValueError(f"unknown mixer type {kind!r}")
    return part, names


def _feed_forward(mlp: dict, width: int):
    if mlp["kind"] == "dense":
        part = BiasedDense(width, mlp["ff"], "gelu_erf")
        return part, {"up": "up", "up.b": "up_b", "down": "down", "down.b": "down_b"}
    shared = mlp.get("shared") or {}
    experts = mlp["router"]["experts"]
    part = RoutedExperts(width, experts, mlp["router"]["top"], mlp["expert"]["ff"], shared.get("ff", 0), "relu_squared")
    names = {"router": "router"}
    for e in range(experts):
        names[f"e{e}.up"], names[f"e{e}.down"] = f"e{e}_up", f"e{e}_down"
    if shared:
        names.update({"shared.up": "shared_up", "shared.down": "shared_down", "shared.sg": "shared_sg"})
    return part, names


@register_architecture("Revupel")
class Revupel:
    config_class = RevupelConfig

    @staticmethod
    def layout(config: RevupelConfig) -> ModelLayout:
        d = config.data
        width, vocab, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        taps = d["canon"]["taps"] if d.get("canon") else 0
        side_dim = d["token_side"]["dim"] if d.get("token_side") else 0
        names: dict = {}
        side_table = None
        if side_dim:
            side_table = TokenSideTable(vocab, len(d["layers"]) * side_dim)
            names["side.embed"] = (side_table, "table")
        blocks = []
        for index, layer in enumerate(d["layers"]):
            prefix = f"l{index}."
            norm1 = ScalarRMSNorm(width, eps)
            names[prefix + "norm1"] = (norm1, "weight")
            mixer, mixer_names = _mixer(layer["type"], layer["mixer"], width, eps)
            for stored, local in mixer_names.items():
                names[f"{prefix}mix.{stored}"] = (mixer, local)
            conv = None
            if taps:
                conv = ResidualCausalConv(width, taps)
                names[prefix + "canon1"] = (conv, "weight")
            norm2 = feed_forward = None
            if layer.get("mlp"):
                norm2 = ScalarRMSNorm(width, eps)
                names[prefix + "norm2"] = (norm2, "weight")
                feed_forward, ff_names = _feed_forward(layer["mlp"], width)
                for stored, local in ff_names.items():
                    names[f"{prefix}mlp.{stored}"] = (feed_forward, local)
            side = None
            if side_dim:
                side = TokenSideInput(width, side_dim, index, side_table, eps)
                for stored in ("gate", "proj", "norm"):
                    names[f"{prefix}side.{stored}"] = (side, stored)
            blocks.append(ConvSideBlock(norm1, mixer, norm2, feed_forward, input_conv=conv, side=side))
        final_norm = ScalarRMSNorm(width, eps)
        names["final.norm"] = (final_norm, "weight")
        optional = {f"l{index}.norm2" for index, layer in enumerate(d["layers"]) if not layer.get("mlp")}
        return ModelLayout(
            width=width, vocab_size=vocab, max_positions=config.max_seq_len, blocks=blocks,
            order=[LayerCall(index) for index in config.run_order()],      # every call gets a cache and states of its own
            final_norm=final_norm, names=names, embedding_name="embed", head_name="head", optional_names=optional,
        )
