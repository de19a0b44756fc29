"""The Revupel design in the engine against the plain implementation of ``plain_revupel`` (``-m gpu``).

Small configurations with random weights, none of them a model anyone serves: they differ from
each other in every size and option (head counts, ranks, rotated coordinates fewer than the
rotated part, taps, experts and how many a token uses, with and without shared expert, loop,
side input, feed-forward), and some tests build weights or inputs so that one key, one window of
taps or one expert decides the result.
"""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

import plain_revupel as plain

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


def _attention(heads=3, dim=24, rot_dim=8, vdim=20, q_rank=40, kv_rank=48, rot_dims=None, base=10000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}}


def _mlstm(heads=2, dim=16, vdim=24, cap=15.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _dense(ff=72):
    return {"kind": "dense", "ff": ff}


def _moe(experts=6, top=2, ff=24, shared=40):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _layer(mixer, mlp):
    return {**mixer, "mlp": mlp}


#: "A": every mechanism, a loop in the middle, rotation on fewer coordinates than the rotated part.
CONFIG_A = {
    "architecture": "Revupel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
    "token_side": {"dim": 12}, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [_layer(_mlstm(), _dense()), _layer(_attention(rot_dims=4), _moe()), _layer(_mlstm(3, 40, 16, 8.0), _moe(4, 4, 16, 0)),
               _layer(_attention(2, 16, 16, 32, 24, 72), None)],
}
#: "B": no loop, no side input, two taps, one expert per token, heads and sizes that are no powers of two.
CONFIG_B = {
    "architecture": "Revupel", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [_layer(_attention(5, 12, 4, 12, 16, 20, base=500.0), _moe(5, 1, 20, 8)), _layer(_mlstm(1, 48, 40, 10.0), _dense(50))],
}
#: "C": no convolution, a loop over everything, a single attention layer.
CONFIG_C = {
    "architecture": "Revupel", "vocab": 130, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 5},
    "loop": {"start": 0, "stop": 1, "times": 3},
    "layers": [_layer(_attention(2, 8, 8, 8, 8, 16), _dense(32))],
}
#: "D": sizes that are no multiples of 8, some of them odd (nothing may rest on alignment).
CONFIG_D = {
    "architecture": "Revupel", "vocab": 77, "width": 100, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "token_side": {"dim": 3},
    "layers": [_layer(_attention(3, 10, 6, 7, 18, 21, rot_dims=4), _moe(3, 2, 10, 6)), _layer(_mlstm(3, 10, 7, 11.0), _dense(30)),
               _layer(_attention(2, 9, 2, 5, 11, 13), _moe(5, 3, 9, 0))],
}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}
PAGE = {"A": 8, "B": 4, "C": 16, "D": 16}


def _specs(config):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.revupel_config import RevupelConfig

    typed = RevupelConfig.from_dict(config)
    return typed, registry.architecture("Revupel").layout(typed).tensor_specs()


def random_tensors(config, seed, scale=1.0):
    """Random tensors, rounded to bfloat16 so that both number formats hold the same values.
    Matrices are drawn at ``scale / sqrt(inputs)``, norm weights around one, biases small."""
    _, specs = _specs(config)
    rng = np.random.default_rng(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].shape
        if name.endswith(("norm1", "norm2", "final.norm")) or name.endswith(".norm"):
            values = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith(".b"):
            values = 0.5 * rng.standard_normal(shape)
        elif name.endswith("canon1"):
            values = 0.4 * rng.standard_normal(shape)
        elif name in ("embed", "side.embed"):
            values = rng.standard_normal(shape)
        else:
            values = scale * rng.standard_normal(shape) / math.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.bfloat16)
    return out


def build(config, tensors, dtype):
    from paged_kv_serving_b200.models.decoder import DecoderModel

    typed, _ = _specs(config)
    return DecoderModel.from_tensors(typed, tensors, dtype=dtype, device="cuda")


def session_for(config, tensors, dtype, max_tokens=512, page=8, max_live=4):
    from paged_kv_serving_b200.engine.replay import ReplaySession

    session = ReplaySession(build(config, tensors, dtype), max_tokens=max_tokens, block_size=page, max_live=max_live)
    session.runner.storage.fill(float("nan"))        # a page that was never written must never be read
    return session


def tokens_for(config, count, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, config["vocab"], size=count)]


def close(got, want, dtype, what):
    """Rows of logits against the plain ones: the gap with its mean taken off, as a share of the
    spread of the plain logits. float32: every row within 1e-4. bfloat16: rounding moves a row by
    about half a percent, but where two experts' router scores nearly tie it may pick the other one,
    which moves that token's row by tens of percent and, through the caches and states, the rows
    after it by a few. So the typical row must stay within 5 %, at most one row in six may
    exceed 10 %, and none 150 % (with two of three experts in use a swap replaces half of the routed
    output); the float32 runs of the same schedules are the sharp test."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shapes {got.shape} and {want.shape}"
    gap = got - want
    gap = gap - gap.mean(axis=-1, keepdims=True)
    spread = max(float(want.std()), 1e-6)
    error = np.sqrt((gap ** 2).mean(axis=-1)) / spread
    assert np.isfinite(got).all(), f"{what}: the engine's logits are not finite"
    worst = f"{what}: row {int(error.argmax())} is off by {error.max():.3e} of the spread"
    if dtype == "float32":
        assert float(error.max()) <= 1e-4, worst
    else:
        assert float(np.median(error)) <= 0.05, f"{what}: the typical row is off by {np.median(error):.3e} of the spread"
        assert int((error > 0.1).sum()) <= max(1, error.size // 6), worst
        assert float(error.max()) <= 1.5, worst


def plain_logits(config, tensors, tokens):
    return plain.forward(config, tensors, tokens).numpy()


# --- whole models: prompts, decoding, portions, batches --------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_every_position_first_tokens_included(name, dtype):
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=3)
    tokens = tokens_for(config, 70, seed=1)
    session = session_for(config, tensors, dtype, page=PAGE[name])
    got = session.step([{"id": "r", "tokens": tokens, "want": list(range(len(tokens)))}], end=["r"])
    close(got, plain_logits(config, tensors, tokens), dtype, f"{name} whole prompt")
    session.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=4)
    tokens = tokens_for(config, 61, seed=2)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=PAGE[name])
    bulk = 21
    rows = [session.step([{"id": "r", "tokens": tokens[:bulk], "want": [bulk - 1]}])]
    for t in tokens[bulk:]:
        rows.append(session.step([{"id": "r", "tokens": [t], "want": [0]}]))
    close(np.concatenate(rows), want[bulk - 1:], dtype, f"{name} prompt then decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_from_the_very_first_token_and_for_long(dtype):
    """Every token alone from position 0 (the convolution's zeros, the recurrence's start) for 150
    steps: decode steps replay a captured graph, pages fill and follow each other."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=5)
    tokens = tokens_for(config, 150, seed=3)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=4)
    rows = [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens]
    close(np.concatenate(rows), want, dtype, "decoding from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=6)
    tokens = tokens_for(config, 90, seed=4)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=PAGE[name])
    rows, at = [], 0
    sizes = [2, 3, 1, 2, 17, 2, 1, 1, 31, 5, 2, 9, 2, 2, 10]
    for size in sizes:
        part = tokens[at:at + size]
        rows.append(session.step([{"id": "r", "tokens": part, "want": list(range(len(part)))}]))
        at += len(part)
    assert at == len(tokens)
    close(np.concatenate(rows), want, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("A", "B"))
def test_unequal_requests_in_one_batch_equal_each_alone_and_slots_and_pages_are_used_again(name, dtype):
    """Three requests of different lengths advance side by side in portions and single tokens, in
    a pool of two state slots and few pages: a fourth and a fifth request start in the slot and on
    the pages a finished one gave back."""
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=7)
    lengths = {"a": 50, "b": 23, "c": 9, "d": 41, "e": 30}
    tokens = {k: tokens_for(config, n, seed=10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: plain_logits(config, tensors, v) for k, v in tokens.items()}
    session = session_for(config, tensors, dtype, max_tokens=128, page=PAGE[name], max_live=2)
    got = {k: [] for k in tokens}
    at = {k: 0 for k in tokens}

    def step(plan):
        entries, order, end = [], [], []
        for key, count in plan:
            part = tokens[key][at[key]:at[key] + count]
            entries.append({"id": key, "tokens": part, "want": list(range(len(part)))})
            order.append((key, len(part)))
            at[key] += len(part)
            if at[key] == len(tokens[key]):
                end.append(key)
        out = session.step(entries, end=end)
        row = 0
        for key, n in order:
            got[key].append(out[row:row + n])
            row += n
        session.check_invariants()

    step([("a", 13), ("b", 2)])
    step([("a", 1), ("b", 19)])
    step([("a", 30), ("b", 1)])
    step([("a", 1), ("b", 1)])            # b ends: its slot and pages go back
    step([("a", 1), ("c", 7)])            # c takes them
    step([("a", 1), ("c", 1)])
    step([("c", 1), ("a", 3)])            # both end
    step([("d", 2), ("e", 30)])           # e is whole in one step and ends
    step([("d", 39)])
    for key in tokens:
        close(np.concatenate(got[key]), want[key], dtype, f"{name} request {key} in a batch")
    assert session.cache.num_free_blocks == session.num_blocks and session.cache.state_slots.num_free == 2


def test_logits_do_not_depend_on_the_cut_in_float32():
    """The same tokens whole, in portions and one by one: rows agree far below the bound against
    the plain implementation (recurrences run token by token whatever the cut)."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=8)
    tokens = tokens_for(config, 40, seed=9)
    whole = session_for(config, tensors, "float32").step([{"id": "r", "tokens": tokens, "want": list(range(40))}])
    session = session_for(config, tensors, "float32")
    parts = [session.step([{"id": "r", "tokens": tokens[i:i + 1], "want": [0]}]) for i in range(40)]
    assert np.abs(np.concatenate(parts) - whole).max() <= 2e-5 * np.abs(whole).max()


# --- greedy generation through the entry point and the scheduler ------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    from paged_kv_serving_b200.api import generate
    from paged_kv_serving_b200.weights.random_init import write_model_folder

    config = CONFIGS["A"]
    typed, _ = _specs(config)
    tensors = random_tensors(config, seed=11, scale=1.5)
    write_model_folder(tmp_path, typed, tensors)
    prompts = [tokens_for(config, n, seed=20 + n) for n in (5, 33, 18)]
    new = 10
    got = generate(tmp_path, prompts, max_new_tokens=new, dtype=dtype, block_size=8, max_batched_tokens=24, max_running_seqs=4)
    for prompt, samples in zip(prompts, got):
        ids = samples[0]
        assert len(ids) == new
        rows = plain_logits(config, tensors, list(prompt) + ids[:-1])[len(prompt) - 1:]
        for place, (token, row) in enumerate(zip(ids, rows)):
            if dtype == "float32":
                assert token == int(row.argmax()) or row[token] >= row.max() - 1e-4, f"token {place} is not the plain choice"
            else:
                assert row[token] >= row.max() - 0.08 * row.std(), f"token {place}: far from the plain maximum"


def test_config_round_trip_and_refusals():
    from paged_kv_serving_b200.config.revupel_config import RevupelConfig

    typed = RevupelConfig.from_dict(CONFIG_A)
    assert RevupelConfig.from_dict(typed.to_dict()).to_dict() == typed.to_dict()
    assert typed.run_order() == [0, 1, 2, 1, 2, 3]
    bad = copy.deepcopy(CONFIG_A)
    bad["layers"][1]["mixer"]["window"] = 5
    with pytest.raises(ValueError):
        RevupelConfig.from_dict(bad)
    bad = copy.deepcopy(CONFIG_A)
    bad["layers"][0]["type"] = "something"
    with pytest.raises(ValueError):
        RevupelConfig.from_dict(bad)


# --- mechanisms alone ---------------------------------------------------------------------------


def _single(mixer, mlp=None, **extra):
    return {"architecture": "Revupel", "vocab": 60, "width": 32, "norm": {"eps": 1e-6}, "layers": [_layer(mixer, mlp)], **extra}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("what", ("attention", "attention_partly_rotated", "mlstm", "mlstm_wide_keys", "mlstm_very_wide_keys",
                                  "dense", "routed_top_all", "routed_no_shared", "conv", "conv_one_tap", "side"))
def test_each_mechanism_alone(what, dtype):
    config = {
        "attention": _single(_attention(2, 8, 8, 16, 8, 24)),
        "attention_partly_rotated": _single(_attention(4, 4, 12, 4, 12, 8, rot_dims=6)),
        "mlstm": _single(_mlstm(2, 8, 12, 6.0)),
        "mlstm_wide_keys": _single(_mlstm(1, 72, 8, 20.0)),
        "mlstm_very_wide_keys": _single(_mlstm(2, 288, 6, 20.0)),          # the kernels' form for keys beyond 256
        "dense": _single(_attention(1, 8, 4, 8, 8, 8), _dense(20)),
        "routed_top_all": _single(_attention(1, 8, 4, 8, 8, 8), _moe(3, 3, 8, 8)),
        "routed_no_shared": _single(_attention(1, 8, 4, 8, 8, 8), _moe(7, 2, 8, 0)),
        "conv": _single(_mlstm(2, 8, 8, 9.0), canon={"taps": 5}),
        "conv_one_tap": _single(_mlstm(2, 8, 8, 9.0), canon={"taps": 1}),     # no tail, no state
        "side": _single(_mlstm(2, 8, 8, 9.0), token_side={"dim": 7}),
    }[what]
    tensors = random_tensors(config, seed=31, scale=2.0)
    tokens = tokens_for(config, 37, seed=5)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=4)
    got = [session.step([{"id": "r", "tokens": tokens[:5], "want": list(range(5))}]),
           session.step([{"id": "r", "tokens": tokens[5:30], "want": list(range(25))}])]
    got += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[30:]]
    close(np.concatenate(got), want, dtype, what)


def test_convolution_sees_exactly_its_taps_across_portion_edges():
    """A weight that is one on a single tap: the output is the input plus the input that many
    tokens back, whatever the cut; just outside the taps nothing arrives."""
    from paged_kv_serving_b200.ops import mixer_ops

    width, taps, slots = 8, 4, 3
    x = torch.arange(1, 1 + 11 * width, dtype=torch.float32, device="cuda").view(11, width)
    for back in range(taps):
        weight = torch.zeros((width, taps), device="cuda")
        weight[:, taps - 1 - back] = 1.0
        want = x.clone()
        want[back:] += x[:11 - back]
        for cuts in ([11], [1, 1, 1, 8], [2, 9], [5, 1, 5], [3, 3, 3, 2]):
            state = torch.zeros((slots, taps - 1, width), device="cuda")
            state[0] = float("nan")                        # another request's slot is never read
            rows, at = [], 0
            for n in cuts:
                part = x[at:at + n].contiguous()
                rows.append(mixer_ops.conv_residual(part, weight, state, torch.zeros(n, dtype=torch.int32, device="cuda"),
                                                    torch.tensor([0, n], dtype=torch.int32, device="cuda"),
                                                    torch.tensor([2], dtype=torch.int32, device="cuda")))
                at += n
            assert torch.equal(torch.cat(rows), want), f"tap {back} back, cuts {cuts}"


def _latent_reference(q_lat, q_rot, cache, first, scale, rank, window=0):
    """Plain absorbed attention of one entry: q_lat [heads, n, rank], q_rot [heads, n, rot] (already
    rotated), cache [keys, rank + rot] with key j at position j; query i sits at position first + i."""
    heads, n, _ = q_lat.shape
    out = np.zeros((heads, n, rank))
    for a in range(heads):
        for i in range(n):
            hi = first + i + 1
            lo = max(0, hi - window) if window else 0
            q = np.concatenate([q_lat[a, i], q_rot[a, i]])
            score = cache[lo:hi] @ q * scale
            weight = np.exp(score - score.max())
            weight /= weight.sum()
            out[a, i] = weight @ cache[lo:hi, :rank]
    return out


@pytest.mark.parametrize("page", (4, 16))
@pytest.mark.parametrize("far_key", (0, 1, 3, 4, 15, 16, 17, 255, 256, 300))
def test_latent_attention_finds_one_far_key_among_hundreds(far_key, page):
    """One key is made to match the query (its score stands out by a wide margin); the result must
    be that key's latent, wherever the key lies: first tokens, either side of a page border, far
    back. Queries: a run of prompt tokens and a single decoded token."""
    from paged_kv_serving_b200.ops import mixer_ops

    rng = np.random.default_rng(far_key)
    heads, rank, rot, keys = 2, 16, 4, 320
    cache = rng.standard_normal((keys, rank + rot)).astype(np.float32)
    direction = cache[far_key] / np.linalg.norm(cache[far_key])
    for n_queries in (1, 7):
        first = keys - n_queries
        q = np.tile(direction * 40.0, (heads, n_queries, 1)).astype(np.float32)
        q_lat, q_rot = q[..., :rank].copy(), q[..., rank:].copy()
        pages = keys // page
        order = rng.permutation(pages + 3)[:pages]                     # pages lie scattered in the pool
        pool = torch.full((pages + 3, 1, page, rank + rot), float("nan"), device="cuda")
        for p in range(pages):
            pool[order[p], 0] = torch.from_numpy(cache[p * page:(p + 1) * page]).cuda()
        table = torch.tensor(order[None, :], dtype=torch.int32, device="cuda")
        # the kernel reads the rotated part from the query projection's rows [tokens, heads * (0 + rot)]
        rows = torch.from_numpy(np.ascontiguousarray(q_rot.transpose(1, 0, 2).reshape(n_queries, heads * rot))).cuda()
        per_block = mixer_ops.latent_rows_per_block()
        blocks = -(-n_queries * heads // per_block)
        got = mixer_ops.latent_attention(
            torch.from_numpy(q_lat).cuda(), rows, 0, rot, pool, table, torch.tensor([0, n_queries], dtype=torch.int32, device="cuda"),
            torch.tensor([first], dtype=torch.int32, device="cuda"), torch.zeros(blocks, dtype=torch.int32, device="cuda"),
            torch.arange(blocks, dtype=torch.int32, device="cuda") * per_block, torch.zeros(1, device="cuda"), None, heads,
            rank, rot, 0, page, 0, 1.0, torch.zeros(1, dtype=torch.int32, device="cuda")).cpu().numpy()
        want = _latent_reference(q_lat, q_rot, cache, first, 1.0, rank)
        assert np.abs(got - want).max() <= 1e-4
        assert np.abs(got - cache[far_key, :rank]).max() <= 1e-3, "the far key did not decide the result"


@pytest.mark.parametrize("window", (1, 5, 32, 33))
def test_latent_attention_window_edges(window):
    """The kernel's optional window: the key just inside it decides, the key just outside is not seen."""
    from paged_kv_serving_b200.ops import mixer_ops

    rng = np.random.default_rng(window)
    heads, rank, rot, keys, page = 1, 8, 2, 100, 8
    cache = rng.standard_normal((keys, rank + rot)).astype(np.float32)
    for inside in (True, False):
        qpos = keys - 1
        target = qpos - window + 1 if inside else qpos - window
        direction = cache[target] / np.linalg.norm(cache[target]) * 50.0
        q_lat = direction[None, None, :rank].astype(np.float32).copy()
        q_rot = direction[None, None, rank:].astype(np.float32).copy()
        pages = -(-keys // page)
        padded = np.full((pages * page, rank + rot), np.nan, dtype=np.float32)
        padded[:keys] = cache
        pool = torch.from_numpy(padded).cuda().view(pages, 1, page, rank + rot)
        got = mixer_ops.latent_attention(
            torch.from_numpy(q_lat).cuda(), torch.from_numpy(q_rot[0]).cuda(), 0, rot, pool,
            torch.arange(pages, dtype=torch.int32, device="cuda")[None, :].contiguous(),
            torch.tensor([0, 1], dtype=torch.int32, device="cuda"), torch.tensor([qpos], dtype=torch.int32, device="cuda"),
            torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
            torch.zeros(1, device="cuda"), None, heads, rank, rot, 0, page, window, 1.0,
            torch.zeros(1, dtype=torch.int32, device="cuda")).cpu().numpy()
        want = _latent_reference(q_lat, q_rot, cache, qpos, 1.0, rank, window)
        assert np.abs(got - want).max() <= 1e-4
        decided = np.abs(got[0, 0] - cache[target, :rank]).max() <= 1e-3
        assert decided == inside


def test_mlstm_kernels_remember_a_token_from_far_back():
    """The forget gate is held open (log f near 0) and one early token gets a large input gate: a
    later query that matches its key reads its value back, across many portions."""
    from paged_kv_serving_b200.ops import mixer_ops

    heads, dim, vdim, tokens = 2, 8, 12, 200
    rng = np.random.default_rng(0)
    offsets = {"q": 0, "k": heads * dim, "v": 2 * heads * dim, "g": 2 * heads * dim + heads * vdim,
               "i": 2 * heads * dim + 2 * heads * vdim, "f": 2 * heads * dim + 2 * heads * vdim + heads}
    ld = offsets["f"] + heads
    proj = (0.1 * rng.standard_normal((tokens, ld))).astype(np.float32)
    proj[:, offsets["i"]:offsets["i"] + heads] = -8.0
    proj[:, offsets["f"]:offsets["f"] + heads] = 30.0
    marked, asking = 3, tokens - 1
    proj[marked, offsets["i"]:offsets["i"] + heads] = 8.0
    key = rng.standard_normal((heads, dim)).astype(np.float32)
    proj[marked, offsets["k"]:offsets["k"] + heads * dim] = key.reshape(-1)
    proj[asking, offsets["q"]:offsets["q"] + heads * dim] = key.reshape(-1) * 3.0
    value = proj[marked, offsets["v"]:offsets["v"] + heads * vdim].reshape(heads, vdim).copy()
    proj[:, offsets["g"]:offsets["g"] + heads * vdim] = 30.0            # output gate open
    ones = torch.ones(heads * vdim, device="cuda")
    zeros = torch.zeros(heads, device="cuda")
    results = []
    for cuts in ([tokens], [1] * 10 + [tokens - 10], [2, 50, 3, tokens - 55]):
        S = torch.zeros((2, heads, vdim, dim), device="cuda")
        n = torch.zeros((2, heads, dim), device="cuda")
        m = torch.zeros((2, heads), device="cuda")
        rows, at = [], 0
        for count in cuts:
            part = torch.from_numpy(proj[at:at + count]).cuda()
            rows.append(mixer_ops.mlstm(part, offsets, zeros, zeros, ones, 40.0, 1.0, 1e-6, S, n, m,
                                        torch.tensor([0, count], dtype=torch.int32, device="cuda"),
                                        torch.tensor([1], dtype=torch.int32, device="cuda"), heads, dim, vdim, torch.float32))
            at += count
        results.append(torch.cat(rows).cpu().numpy())
        assert float(S[0].abs().max()) == 0.0, "another slot's state was touched"
    for other in results[1:]:
        assert np.abs(other - results[0]).max() <= 1e-5
    read = results[0][asking].reshape(heads, vdim)
    for a in range(heads):              # unit norm of the head: compare directions
        cosine = float(read[a] @ value[a] / (np.linalg.norm(read[a]) * np.linalg.norm(value[a])))
        assert cosine > 0.99, f"head {a} did not read the marked token's value back (cosine {cosine:.3f})"


def test_router_keeps_the_best_experts_with_their_softmax_scores():
    from paged_kv_serving_b200.ops import mixer_ops

    rng = np.random.default_rng(1)
    for experts, top in ((8, 2), (5, 5), (3, 1), (17, 4)):
        logits = rng.standard_normal((50, experts + 3)).astype(np.float32) * 3.0
        logits[0, :experts] = 1.0                                    # a full tie: the lowest indices win
        got = mixer_ops.route_top(torch.from_numpy(logits).cuda(), experts, top).cpu().numpy()
        z = logits[:, :experts].astype(np.float64)
        score = np.exp(z - z.max(axis=1, keepdims=True))
        score /= score.sum(axis=1, keepdims=True)
        for t in range(50):
            chosen = sorted(range(experts), key=lambda e: (-z[t, e], e))[:top]
            want = np.zeros(experts)
            want[chosen] = score[t, chosen]
            assert np.abs(got[t] - want).max() <= 1e-6, f"token {t} with {experts} experts, top {top}"


def test_one_expert_decides_when_the_router_is_sure():
    """Router weights scaled up so that each token has one clear expert: the routed output is that
    expert's alone (top 1, no shared expert), against the plain implementation."""
    config = _single(_mlstm(1, 8, 8, 9.0), _moe(4, 1, 12, 0))
    tensors = random_tensors(config, seed=41)
    tensors["l0.mlp.router"] = (tensors["l0.mlp.router"].float() * 25.0).to(torch.bfloat16)
    tokens = tokens_for(config, 30, seed=6)
    session = session_for(config, tensors, "float32", page=4)
    got = session.step([{"id": "r", "tokens": tokens, "want": list(range(30))}])
    close(got, plain_logits(config, tensors, tokens), "float32", "sure router")


@pytest.mark.parametrize("heads,rank,rot,rot_dims,page,window", [(4, 32, 16, 16, 16, 0), (3, 48, 16, 8, 8, 0), (1, 16, 0, 0, 4, 0),
                                                                  (16, 128, 32, 32, 16, 0), (5, 272, 16, 16, 16, 0), (2, 32, 16, 16, 8, 37)])
def test_latent_attention_on_tensor_cores_matches_the_general_kernel(heads, rank, rot, rot_dims, page, window):
    """A ragged batch in bfloat16 (a long portion behind a cached prefix, a short one, single
    decoded tokens at a page border and elsewhere) through both kernels, and against float64."""
    from paged_kv_serving_b200.ops import mixer_ops

    assert mixer_ops.latent_mma_supports(rank, rot)
    rng = np.random.default_rng(heads * 1000 + rank)
    dk = rank + rot
    lens, firsts = [150, 9, 1, 1, 2], [70, 0, 4 * page - 1, 4 * page, 301]
    tokens = sum(lens)
    pages_per = [-(-(f + n) // page) for f, n in zip(firsts, lens)]
    total_pages = sum(pages_per) + 2
    pool = torch.full((total_pages, 1, page, dk), float("nan"), dtype=torch.bfloat16, device="cuda")
    order = rng.permutation(total_pages)
    table = np.full((len(lens), max(pages_per)), -1, dtype=np.int32)
    caches, at = [], 0
    for s, (f, n) in enumerate(zip(firsts, lens)):
        cache = torch.from_numpy(rng.standard_normal((f + n, dk)).astype(np.float32)).to(torch.bfloat16)
        caches.append(cache.float().numpy().astype(np.float64))
        for j in range(pages_per[s]):
            table[s, j] = order[at]
            rows = cache[j * page:(j + 1) * page]
            pool[order[at], 0, :rows.shape[0]] = rows.cuda()
            at += 1
    head_stride = 8 + rot
    q = torch.from_numpy(rng.standard_normal((tokens, heads * head_stride)).astype(np.float32)).to(torch.bfloat16).cuda()
    q_lat = torch.from_numpy(rng.standard_normal((heads, tokens, rank)).astype(np.float32)).to(torch.bfloat16).float().cuda()
    gate = torch.from_numpy(rng.standard_normal((tokens, heads + 3)).astype(np.float32)).cuda()[:, :heads]
    freq = torch.tensor([10000.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(max(rot_dims // 2, 1))], device="cuda")
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    scale = dk ** -0.5

    def run(kernel, per_block):
        blocks = [-(-n * heads // per_block) for n in lens]
        work_seq = np.repeat(np.arange(len(lens)), blocks).astype(np.int32)
        work_row0 = np.concatenate([np.arange(b) * per_block for b in blocks]).astype(np.int32)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = kernel(q_lat, q, 8, head_stride, pool, torch.from_numpy(table).cuda(), torch.from_numpy(starts).cuda(),
                     torch.tensor(firsts, dtype=torch.int32, device="cuda"), torch.from_numpy(work_seq).cuda(),
                     torch.from_numpy(work_row0).cuda(), freq, gate, heads, rank, rot, rot_dims, page, window, scale, status)
        assert int(status.item()) == 0
        return out.float().cpu().numpy()

    general = run(mixer_ops.latent_attention, mixer_ops.latent_rows_per_block())
    fast = run(mixer_ops.latent_attention_mma, mixer_ops.latent_mma_rows_per_block(rank, rot))
    # float64 from the same bfloat16 inputs
    qf = q.float().cpu().numpy().astype(np.float64).reshape(tokens, heads, head_stride)[:, :, 8:]
    want = np.zeros((heads, tokens, rank))
    for s, (f, n) in enumerate(zip(firsts, lens)):
        rows = slice(int(starts[s]), int(starts[s + 1]))
        positions = torch.arange(f, f + n)
        rotated = plain.rotate_half(torch.from_numpy(qf[rows]), positions, rot_dims, 10000.0).numpy() if rot_dims else qf[rows]
        want[:, rows] = _latent_reference(q_lat[:, rows].cpu().numpy().astype(np.float64), rotated.transpose(1, 0, 2),
                                          caches[s], f, scale, rank, window)
    want *= 1.0 / (1.0 + np.exp(-gate.cpu().numpy().astype(np.float64).T[:, :, None]))
    # the key range cut into parts that are merged afterwards (what a step of few rows uses)
    for parts in (2, 5, 16):
        cut = run(lambda *a, **k: mixer_ops.latent_attention_mma(*a, num_splits=parts, **k),
                  mixer_ops.latent_mma_rows_per_block(rank, rot))
        assert np.abs(cut - fast).max() <= 0.02 * np.abs(want).max(), f"{parts} parts"
    assert np.isfinite(fast).all() and np.isfinite(general).all()
    assert np.abs(general - want).max() <= 0.02 * np.abs(want).max()
    assert np.abs(fast - want).max() <= 0.03 * np.abs(want).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_side_input_as_one_kernel_equals_the_separate_kernels(dtype):
    """The switch that sends steps of few rows through the one-kernel form of the side input."""
    from paged_kv_serving_b200.parts.token_side import TokenSideInput

    config = CONFIGS["C"]
    tensors = random_tensors(config, seed=51)
    tokens = tokens_for(config, 40, seed=8)
    want = plain_logits(config, tensors, tokens)
    before = TokenSideInput.FUSED_ROWS
    TokenSideInput.FUSED_ROWS = 16
    try:
        session = session_for(config, tensors, dtype, page=PAGE["C"])
        rows = [session.step([{"id": "r", "tokens": tokens[:20], "want": list(range(20))}]),        # separate kernels
                session.step([{"id": "r", "tokens": tokens[20:33], "want": list(range(13))}])]       # one kernel
        rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[33:]]
    finally:
        TokenSideInput.FUSED_ROWS = before
    close(np.concatenate(rows), want, dtype, "side input, one kernel")


def test_command_line_checkpoint_generation_and_trace_program(tmp_path):
    """The design through the command line as a user meets it: a random-weights folder from a
    ``config.json``, greedy generation from it, and ``bin/trace_run`` replaying a trace of it."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import load_file

    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root))
    config = CONFIGS["B"]
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    (tmp_path / "config.json").write_text(json.dumps(config))
    build = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "build-checkpoint", "--out", str(model_dir),
                            "--config", str(tmp_path / "config.json"), "--seed", "3", "--dtype", "bfloat16", "--std", "0.15"],
                           capture_output=True, text=True, env=env, check=True)
    tensors = load_file(str(model_dir / "model.safetensors"))
    assert json.loads(build.stdout)["parameters"] == sum(t.numel() for t in tensors.values())
    run = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "generate", "--model", str(model_dir),
                          "--prompt-ids", "5,17,3,20", "--max-new-tokens", "6", "--dtype", "float32", "--block-size", "4"],
                         capture_output=True, text=True, env=env, check=True)
    line = [json.loads(text) for text in run.stdout.splitlines() if text.startswith("{")][0]
    ids = line["samples"][0]
    rows = plain_logits(config, tensors, [5, 17, 3, 20] + ids[:-1])[3:]
    assert len(ids) == 6 and all(row[token] >= row.max() - 1e-4 for token, row in zip(ids, rows))

    tokens = tokens_for(config, 30, seed=9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[23:], "want": [6]}], "end": ["a"]}]
    process = subprocess.Popen([str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                                "--out", str(out_dir), "--max-tokens", "64", "--block-size", "4"],
                               stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for record in steps:
        process.stdin.write(json.dumps(record) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {record['step']}"
    process.stdin.close()
    assert process.wait(timeout=120) == 0
    want = plain_logits(config, tensors, tokens)
    read = lambda step: np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, config["vocab"])
    assert not (out_dir / "1.f32").exists()
    close(read(0), want[[0, 20]], "float32", "trace step 0")
    close(read(2), want[29:30], "float32", "trace step 2")
