"""The Tiburax design: a decoder whose layers, in an order the configuration lists, mix tokens
either by attention over a sliding window that also keeps a sequence's first tokens (rotated,
unit-norm queries and keys, capped scores, values blended with those of the first such layer) or
by a Mamba selective scan, each followed by a routed feed-forward of gated experts with a shared
expert. The norms sit on the sublayers' outputs (``x += norm(sublayer(x))``) and store their
weights around zero; the embedding is scaled.

This module is all that is specific to the design: which parts a layer has, with which numbers
of the configuration, and the tensor names of a model folder (``embed``, ``head``, ``final.norm``,
and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``).
"""

from __future__ import annotations

from paged_kv_serving_b200.config.registry import register_architecture
from paged_kv_serving_b200.config.tiburax_config import TiburaxConfig
from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
from paged_kv_serving_b200.parts import (
    GatedRoutedExperts, Mamba1, OffsetRMSNorm, PostNormBlock, ScaledRotaryFrequencies, SinkWindowAttention, TokenEmbedding,
)

__all__ = ["Tiburax"]


def _attention(sizes: dict, width: int, eps: float, value_share: str | None):
    rot = sizes.get("rot") or {}
    rotary = None
    if int(rot.get("dims") or 0):
        scaling = rot.get("scaling") or {}
        rotary = ScaledRotaryFrequencies(int(rot["dims"]), float(rot["base"]), scaling.get("factor"), scaling.get("original"),
                                         scaling.get("fast"), scaling.get("slow"))
    mask = sizes.get("mask") or {}
    part = SinkWindowAttention(width, sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"], float(sizes["scale"]),
                               rotary=rotary, unit_norm=True, eps=eps, softcap=float(sizes.get("softcap") or 0.0),
                               window=mask.get("size"), keep_first=int(mask.get("keep_first") or 0), value_share=value_share)
    names = {"q": "q", "k": "k", "v": "v", "o": "o"}
    if value_share is not None:
        names["vmix"] = "vmix"
    return part, names


def _mamba(sizes: dict, width: int):
    part = Mamba1(width, sizes["inner"], sizes["state"], sizes["dt_rank"], sizes["conv"])
    names = {"in": "in_proj", "conv": "conv", "conv.b": "conv_b", "x": "x_proj", "dt": "dt_proj", "dt.b": "dt_b",
             "A_log": "A_log", "D": "D", "o": "o"}
    return part, names


def _feed_forward(mlp: dict, width: int):
    shared = mlp.get("shared") or {}
    experts = mlp["router"]["experts"]
    part = GatedRoutedExperts(width, experts, mlp["router"]["top"], mlp["expert"]["ff"], shared.get("ff", 0), "silu",
                              router_bias=True, renormalise=True)
    names = {"router": "router", "router.b": "router_b"}
    for e in [f"e{e}" for e in range(experts)] + (["shared"] if shared else []):
        for kind in ("gate", "up", "down"):
            names[f"{e}.{kind}"] = f"{e}_{kind}"
    return part, names


@register_architecture("Tiburax")
class Tiburax:
    config_class = TiburaxConfig

    @staticmethod
    def layout(config: TiburaxConfig) -> ModelLayout:
        d = config.data
        width, vocab, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        names: dict = {}
        optional: set = set()
        blocks = []
        value_source_seen = False
        for index, layer in enumerate(d["layers"]):
            prefix = f"l{index}."
            if layer["type"] == "attention":
                share = None
                if layer["mixer"].get("v_mix"):
                    # the first layer that mixes values is the one the later ones mix with
                    share = "blend" if value_source_seen else "source"
                    value_source_seen = True
                else:
                    optional.add(prefix + "mix.vmix")
                mixer, mixer_names = _attention(layer["mixer"], width, eps, share)
            else:
                mixer, mixer_names = _mamba(layer["mixer"], width)
            for stored, local in mixer_names.items():
                names[f"{prefix}mix.{stored}"] = (mixer, local)
            norm1 = OffsetRMSNorm(width, eps)
            names[prefix + "norm1"] = (norm1, "weight")
            norm2 = feed_forward = None
            if layer.get("mlp"):
                norm2 = OffsetRMSNorm(width, eps)
                names[prefix + "norm2"] = (norm2, "weight")
                feed_forward, ff_names = _feed_forward(layer["mlp"], width)
                for stored, local in ff_names.items():
                    names[f"{prefix}mlp.{stored}"] = (feed_forward, local)
            else:
                optional.add(prefix + "norm2")
            blocks.append(PostNormBlock(norm1, mixer, norm2, feed_forward))
        final_norm = OffsetRMSNorm(width, eps)
        names["final.norm"] = (final_norm, "weight")
        embedding = TokenEmbedding(vocab, width, scale=config.embedding_scale)
        names["embed"] = (embedding, "table")
        return ModelLayout(
            width=width, vocab_size=vocab, max_positions=config.max_seq_len, blocks=blocks,
            order=[LayerCall(index) for index in range(len(blocks))], final_norm=final_norm, names=names,
            embedding=embedding, embedding_name="embed", head_name="head", optional_names=optional,
        )
