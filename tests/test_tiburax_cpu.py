"""What of the Tiburax design runs without a GPU: its configuration, its layout and tensor names,
the rotation's frequencies against the plain formula, and the cache manager's rule for a window
that keeps a sequence's first positions."""

from __future__ import annotations

import copy

import numpy as np
import pytest

import plain_tiburax as plain

CONFIG = {
    "architecture": "Tiburax", "vocab": 90, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 24, "state": 6, "dt_rank": 3, "conv": 3}, "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "softcap": 20.0, "v_mix": False,
                   "mask": {"size": 9, "keep_first": 2}, "rot": {"base": 100.0, "dims": 8}},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 2}}},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "softcap": 20.0, "v_mix": True,
                   "mask": {"size": 9, "keep_first": 2},
                   "rot": {"base": 100.0, "dims": 12, "scaling": {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 1}, "shared": {"ff": 16}}},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "v_mix": True,
                   "mask": {"size": 5, "keep_first": 0}, "rot": {"base": 100.0, "dims": 6}},
         "mlp": None},
    ],
}


def _layout(config=CONFIG):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.tiburax_config import TiburaxConfig

    typed = TiburaxConfig.from_dict(config)
    return typed, registry.architecture("Tiburax").layout(typed)


def test_config_round_trip_and_refusals():
    from paged_kv_serving_b200.config.tiburax_config import TiburaxConfig

    typed = TiburaxConfig.from_dict(CONFIG)
    assert TiburaxConfig.from_dict(typed.to_dict()).to_dict() == typed.to_dict()
    assert typed.vocab_size == 90 and typed.d_model == 40 and typed.n_layers == 4 and typed.embedding_scale == 2.5
    for change in (lambda c: c["layers"][1]["mixer"].update(window=5), lambda c: c["layers"][0].update(type="something"),
                   lambda c: c["layers"][1]["mixer"].pop("dim"), lambda c: c["layers"][1]["mixer"].update(heads=3),
                   lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), lambda c: c["layers"][1]["mlp"]["router"].update(top=4),
                   lambda c: c.update(extra=1), lambda c: c["layers"][0]["mixer"].update(state=0)):
        bad = copy.deepcopy(CONFIG)
        change(bad)
        with pytest.raises(ValueError):
            TiburaxConfig.from_dict(bad)


def test_config_is_found_by_its_architecture_name(tmp_path):
    import json

    from paged_kv_serving_b200.config import load_config
    from paged_kv_serving_b200.config.tiburax_config import TiburaxConfig

    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    assert isinstance(load_config(tmp_path), TiburaxConfig)


def test_layout_names_roles_and_cache_requests():
    from paged_kv_serving_b200.cache.manager import plan_groups
    from paged_kv_serving_b200.parts import Mamba1, PostNormBlock, SinkWindowAttention

    _, layout = _layout()
    names = set(layout.tensor_specs())
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.in", "l0.mix.conv.b", "l0.mix.A_log", "l1.mix.q", "l1.mlp.router.b",
            "l1.mlp.e2.gate", "l2.mlp.shared.down", "l2.mix.vmix", "l3.mix.vmix"} <= names
    assert "l1.mix.vmix" not in names and "l0.norm2" not in names and "l3.norm2" not in names
    assert {"l1.mix.vmix", "l0.norm2", "l3.norm2"} <= layout.optional_names
    assert all(isinstance(block, PostNormBlock) for block in layout.blocks)
    mixers = [block.mixer for block in layout.blocks]
    assert isinstance(mixers[0], Mamba1)
    assert [m.value_share for m in mixers[1:]] == [None, "source", "blend"]
    assert isinstance(mixers[1], SinkWindowAttention) and mixers[1].rotary.scaling is None and mixers[2].rotary.scaling is not None
    assert mixers[3].softcap == 0.0 and mixers[3].keep_first == 0 and mixers[3].window == 5
    bare = copy.deepcopy(CONFIG)
    for key in ("mask", "rot"):
        bare["layers"][3]["mixer"].pop(key)
    bare["layers"][1]["mixer"]["mask"] = None
    bare["layers"][2]["mixer"]["mask"] = {"size": None, "keep_first": 3}
    bare["layers"][2]["mlp"]["shared"] = None
    del bare["embedding"]
    _, plain_layout = _layout(bare)
    plain_mixers = [block.mixer for block in plain_layout.blocks]
    assert plain_mixers[3].window is None and plain_mixers[3].rotary is None and plain_mixers[1].window is None
    assert plain_mixers[2].window is None and plain_mixers[2].cache_request().keep_first == 0
    assert plain_layout.blocks[2].feed_forward.shared_inner == 0 and plain_layout.embedding.scale == 1.0
    groups, states = plan_groups(layout.cache_entries())
    assert len(groups) == 2 and len(states) == 2
    by_dim = {g.head_dim: g for g in groups}
    assert by_dim[12].value_dim == 10 and by_dim[12].keep_first == 2 and by_dim[12].window == 9 and len(by_dim[12].entries) == 2
    assert by_dim[6].value_dim == 10 and by_dim[6].keep_first == 0
    assert layout.parameter_count() == sum(int(np.prod(spec.shape)) for spec in layout.tensor_specs().values())


@pytest.mark.parametrize("rot", [
    {"base": 10000.0, "dims": 32}, {"base": 500.0, "dims": 6},
    {"base": 50000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 24.0, "slow": 2.0}},
    {"base": 100.0, "dims": 16, "scaling": {"factor": 2.0, "original": 64, "fast": 4.0, "slow": 0.5}},
    {"base": 1e6, "dims": 128, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"base": 50.0, "dims": 4, "scaling": {"factor": 1.0, "original": 16, "fast": 1.0, "slow": 1.0}},
])
def test_rotation_frequencies_and_amplitude_against_the_plain_formula(rot):
    from paged_kv_serving_b200.parts import ScaledRotaryFrequencies

    scaling = rot.get("scaling") or {}
    part = ScaledRotaryFrequencies(rot["dims"], rot["base"], scaling.get("factor"), scaling.get("original"), scaling.get("fast"),
                                   scaling.get("slow"))
    want, amplitude = plain.rotary_frequencies(rot)
    np.testing.assert_allclose(part.frequencies(), want.numpy(), rtol=1e-13)
    assert abs(part.amplitude - amplitude) < 1e-15
    if scaling and scaling["factor"] > 1:
        plainly = rot["base"] ** (-2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        assert (part.frequencies() <= plainly + 1e-18).all() and (part.frequencies() >= plainly / scaling["factor"] - 1e-18).all()


class _Seq:
    def __init__(self, groups):
        self.token_ids, self.num_computed_tokens = [], 0
        self.block_tables, self.block_hashes = [[] for _ in range(groups)], []
        self.cached_prefix_blocks, self.state_slot = 0, None

    @property
    def num_tokens(self):
        return len(self.token_ids)


@pytest.mark.parametrize("keep,kept_pages", [(0, 0), (1, 1), (4, 1), (5, 2), (8, 2), (9, 3)])
def test_pages_behind_the_window_go_back_but_those_of_the_kept_first_positions_stay(keep, kept_pages):
    from paged_kv_serving_b200.cache.manager import GroupSpec, KVCacheManager
    from paged_kv_serving_b200.cache.pages import NULL_PAGE

    page, window = 4, 6
    groups = [GroupSpec((0,), 2, 8, window, True, 5, keep), GroupSpec((1,), 2, 8, None)]
    cache = KVCacheManager(groups, num_blocks=40, block_size=page, enable_prefix_cache=False)
    seq = _Seq(2)
    for total in (3, 4, 9, 10, 31, 32, 33, 70):
        seq.token_ids = list(range(total))
        cache.reserve(seq, total)
        seq.num_computed_tokens = total
        cache.release_behind_window(seq)
        table = seq.block_tables[0]
        first_live = max(0, total - window + 1)            # the oldest position the next query still reads
        for index, entry in enumerate(table):
            needed = index < kept_pages or (index + 1) * page > first_live
            assert (entry != NULL_PAGE) == needed, f"{total} tokens, page {index}"
        assert all(entry != NULL_PAGE for entry in seq.block_tables[1])
        cache.check_invariants()
    cache.free(seq)
    assert cache.num_free_blocks == 40


def test_groups_differ_by_value_size_and_kept_positions_only_where_it_matters():
    from paged_kv_serving_b200.cache.manager import plan_groups
    from paged_kv_serving_b200.parts import PagedKVRequest

    entries = [(0, PagedKVRequest(2, 16, 8, value_dim=16, keep_first=0)), (1, PagedKVRequest(2, 16, 8)),
               (2, PagedKVRequest(2, 16, 8, value_dim=12)), (3, PagedKVRequest(2, 16, 8, keep_first=3)),
               (4, PagedKVRequest(2, 16, None, keep_first=3)), (5, PagedKVRequest(2, 16, None))]
    groups, _ = plan_groups(entries)
    assert sorted(g.entries for g in groups) == [(0, 1), (2,), (3,), (4, 5)]
