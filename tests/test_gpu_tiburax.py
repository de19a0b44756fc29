"""The Tiburax design in the engine against the plain implementation of ``plain_tiburax`` (``-m gpu``).

Small configurations with random weights, none of them a model anyone serves. They differ from
each other in every size and option: head counts with and without grouped keys, key and value
sizes, rotated coordinates fewer than a head has, stretched and plain rotation, windows and kept
first tokens that do and do not fall on page borders, score caps, which layer is the first to mix
values, state sizes, taps, ranks, experts and how many a token uses, with and without a shared
expert, with and without a feed-forward. Some tests scale the scores so that a single key decides
a row, which makes a window that is one token off or a lost first token visible.
"""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

import plain_tiburax as plain

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


def _attention(heads=4, kv_heads=2, dim=24, vdim=16, window=20, keep=3, rot_dims=16, base=10000.0, scaling=True, softcap=30.0,
               v_mix=True, scale=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
                      "softcap": softcap, "v_mix": v_mix, "mask": {"size": window, "keep_first": keep}, "rot": rot}}


def _mamba(inner=48, state=12, dt_rank=5, conv=4):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def _moe(experts=6, top=2, ff=24, shared=40):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _layer(mixer, mlp):
    return {**mixer, "mlp": mlp}


def _model(layers, vocab=150, width=64, eps=1e-6, scale=3.0):
    return {"architecture": "Tiburax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


#: "A": both mixers twice, grouped keys, a window of 20 with 3 kept tokens on pages of 8, the second
#: attention layer mixes with the first.
CONFIG_A = _model([_layer(_attention(), _moe()), _layer(_mamba(), _moe(4, 4, 16, 0)), _layer(_attention(), _moe(5, 1, 20, 8)),
                   _layer(_mamba(40, 20, 3, 2), None)])
#: "B": a layer that does not mix values first, then the source, then a blender; windows and kept
#: tokens that straddle pages of 4; rotation without stretching on all coordinates of a head; no cap.
CONFIG_B = _model([_layer(_attention(3, 3, 8, 12, window=9, keep=5, rot_dims=8, scaling=False, softcap=0.0, v_mix=False), None),
                   _layer(_attention(6, 3, 12, 20, window=7, keep=0, rot_dims=4, base=500.0), _moe(3, 2, 12, 0)),
                   _layer(_mamba(72, 40, 16, 1), _moe(2, 1, 8, 16)),
                   _layer(_attention(3, 3, 16, 20, window=13, keep=6, rot_dims=10, softcap=5.0), _moe(8, 3, 8, 8))],
                  vocab=97, width=48, eps=1e-5, scale=1.0)
#: "C": sizes that are no multiples of 8, some of them odd (nothing may rest on alignment).
CONFIG_C = _model([_layer(_mamba(30, 7, 3, 3), _moe(3, 2, 10, 6)), _layer(_attention(3, 1, 10, 7, window=11, keep=2, rot_dims=6), _moe(5, 3, 9, 0)),
                   _layer(_mamba(22, 9, 11, 5), None), _layer(_attention(2, 1, 14, 7, window=5, keep=1, rot_dims=14, scaling=False), _moe(2, 2, 5, 3))],
                  vocab=77, width=52, eps=1e-5, scale=0.7)
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
PAGE = {"A": 8, "B": 4, "C": 16}


def _specs(config):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.tiburax_config import TiburaxConfig

    typed = TiburaxConfig.from_dict(config)
    return typed, registry.architecture("Tiburax").layout(typed).tensor_specs()


def random_tensors(config, seed, scale=1.0):
    """Random tensors, rounded to bfloat16 so that both number formats hold the same values.
    Matrices are drawn at ``scale / sqrt(inputs)``; norm weights lie around zero, the blending
    weight inside (0, 1), decays and step sizes in ranges where the state neither dies nor blows up."""
    _, specs = _specs(config)
    rng = np.random.default_rng(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].shape
        if name.endswith(("norm1", "norm2", "final.norm")):
            values = 0.3 * rng.standard_normal(shape)
        elif name.endswith("vmix"):
            values = np.asarray(rng.uniform(0.2, 0.8))
        elif name.endswith("dt.b"):
            values = -1.5 + 0.7 * rng.standard_normal(shape)
        elif name.endswith("A_log"):
            values = 0.6 * rng.standard_normal(shape)
        elif name.endswith(".D"):
            values = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith(".b"):
            values = 0.5 * rng.standard_normal(shape)
        elif name.endswith("mix.conv"):
            values = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
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


def close(got, want, dtype, what, routed=True):
    """Rows of logits against the plain ones: the gap with its mean taken off, as a share of the
    spread of the plain logits. float32: every row within 2e-4. bfloat16: rounding moves a row by
    about a percent; where two experts' router logits nearly tie it may pick the other expert, which
    moves that token's row by tens of percent and, through cache and state, later rows by a few. So
    the typical row stays within 5 %, at most one row in six may exceed 12 %, none 150 %; a model
    without routing stays within 12 % everywhere. The float32 runs of the same schedules are the
    sharp test."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shapes {got.shape} and {want.shape}"
    assert np.isfinite(got).all(), f"{what}: the engine's logits are not finite"
    gap = got - want
    gap = gap - gap.mean(axis=-1, keepdims=True)
    spread = max(float(want.std()), 1e-6)
    error = np.sqrt((gap ** 2).mean(axis=-1)) / spread
    worst = f"{what}: row {int(error.argmax())} is off by {error.max():.3e} of the spread"
    if dtype == "float32":
        assert float(error.max()) <= 2e-4, worst
    elif routed:
        assert float(np.median(error)) <= 0.05, f"{what}: the typical row is off by {np.median(error):.3e} of the spread"
        assert int((error > 0.12).sum()) <= max(1, error.size // 6), worst
        assert float(error.max()) <= 1.5, worst
    else:
        assert float(error.max()) <= 0.12, worst


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


def test_the_residual_stream_after_every_layer_in_float32():
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=12)
    tokens = tokens_for(config, 33, seed=5)
    _, want = plain.forward(config, tensors, tokens, return_layers=True)
    session = session_for(config, tensors, "float32")
    seen = []
    for block in session.model.layout.blocks:
        inner = block.forward

        def spy(hidden, pending, ctx, binding, next_norm=None, _inner=inner):
            out = _inner(hidden, pending, ctx, binding, next_norm=next_norm)
            seen.append(hidden.clone())
            return out

        block.forward = spy
    session.step([{"id": "r", "tokens": tokens, "want": [len(tokens) - 1]}])
    assert len(seen) == len(config["layers"])
    for index, stream in enumerate(seen):
        gap = np.abs(stream.cpu().numpy() - want[index].numpy()).max()
        assert gap <= 1e-4 * float(want[index].abs().max()), f"the stream after layer {index} is off by {gap:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token_across_windows_and_pages(name, dtype):
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=4)
    tokens = tokens_for(config, 75, seed=2)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=PAGE[name])
    bulk = 21
    rows = [session.step([{"id": "r", "tokens": tokens[:bulk], "want": [bulk - 1]}])]
    for t in tokens[bulk:]:
        rows.append(session.step([{"id": "r", "tokens": [t], "want": [0]}]))
    close(np.concatenate(rows), want[bulk - 1:], dtype, f"{name} prompt then decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_from_the_very_first_token_and_for_long(dtype):
    """Every token alone from position 0 (the convolution's zeros, the state's start, the kept first
    tokens while they are still inside the window and after they left it) for 170 steps: decode
    steps replay a captured graph, pages behind the window go back and the kept ones stay."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=5)
    tokens = tokens_for(config, 170, seed=3)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, max_tokens=192, page=4)
    rows = [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens]
    close(np.concatenate(rows), want, dtype, "decoding from the first token")
    table = session.live["r"].block_tables[0]
    assert table[0] != -1, "the page of the kept first tokens was given back"
    assert sum(1 for page in table if page == -1) >= 30, "pages behind the window were not given back"


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
    the plain implementation (the scan runs token by token whatever the cut, attention tiles are
    aligned to absolute positions)."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=8)
    tokens = tokens_for(config, 60, seed=9)
    whole = session_for(config, tensors, "float32").step([{"id": "r", "tokens": tokens, "want": list(range(60))}])
    session = session_for(config, tensors, "float32")
    parts = [session.step([{"id": "r", "tokens": tokens[i:i + 1], "want": [0]}]) for i in range(60)]
    assert np.abs(np.concatenate(parts) - whole).max() <= 2e-5 * np.abs(whole).max()
    session = session_for(config, tensors, "float32")
    parts = [session.step([{"id": "r", "tokens": tokens[i:i + 7], "want": list(range(len(tokens[i:i + 7])))}])
             for i in range(0, 60, 7)]
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
    new = 12
    got = generate(tmp_path, prompts, max_new_tokens=new, dtype=dtype, block_size=8, max_batched_tokens=24, max_running_seqs=4)
    for prompt, samples in zip(prompts, got):
        ids = samples[0]
        assert len(ids) == new
        rows = plain_logits(config, tensors, list(prompt) + ids[:-1])[len(prompt) - 1:]
        for place, (token, row) in enumerate(zip(ids, rows)):
            if dtype == "float32":
                assert token == int(row.argmax()) or row[token] >= row.max() - 1e-4, f"token {place} is not the plain choice"
            else:
                assert row[token] >= row.max() - 0.1 * row.std(), f"token {place}: far from the plain maximum"


def test_forked_samples_share_pages_and_copy_states(tmp_path):
    """Three greedy samples of one prompt: the prompt is computed once, the samples share its pages
    (keys and values of different sizes: a private copy of a page is two copies) and each gets a
    copy of the recurrent states; all three must be the plain greedy continuation."""
    from paged_kv_serving_b200.api import generate
    from paged_kv_serving_b200.weights.random_init import write_model_folder

    config = CONFIGS["A"]
    typed, _ = _specs(config)
    tensors = random_tensors(config, seed=13, scale=1.5)
    write_model_folder(tmp_path, typed, tensors)
    prompt = tokens_for(config, 29, seed=14)
    got = generate(tmp_path, [prompt], max_new_tokens=9, n=3, dtype="float32", block_size=8, max_batched_tokens=64, max_running_seqs=4)
    assert len(got[0]) == 3
    for ids in got[0]:
        rows = plain_logits(config, tensors, list(prompt) + ids[:-1])[len(prompt) - 1:]
        assert len(ids) == 9 and all(row[token] >= row.max() - 1e-4 for token, row in zip(ids, rows))


def test_a_cramped_pool_preempts_and_recomputes_states_and_pages():
    """Four requests in a pool that holds two: requests are preempted, give back pages and state
    slot, and start again from position 0 in a cleared slot; every request's tokens are still the
    plain greedy continuation."""
    from paged_kv_serving_b200.api import engine_for
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

    config = copy.deepcopy(CONFIGS["A"])
    for layer in config["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["mask"] = {"size": 500, "keep_first": 2}       # nothing leaves the window: pages pile up
    tensors = random_tensors(config, seed=15, scale=1.5)
    prompts = [tokens_for(config, n, seed=30 + n) for n in (41, 37, 44, 29)]
    new = 22
    engine = engine_for(build(config, tensors, "float32"), prompts, max_new_tokens=new, dtype="float32", block_size=8, num_blocks=20,
                        max_batched_tokens=48, max_running_seqs=4)
    for i, prompt in enumerate(prompts):
        assert engine.submit(Request(request_id=f"r{i}", prompt_token_ids=tuple(prompt), sampling=SamplingParams(max_new_tokens=new))).admitted
    outputs = {o.request_id: o for o in engine.run_until_idle()}
    assert engine.scheduler.stats.preemptions > 0, "the cramped pool must preempt"
    for i, prompt in enumerate(prompts):
        ids = list(outputs[f"r{i}"].samples[0].token_ids)
        rows = plain_logits(config, tensors, list(prompt) + ids[:-1])[len(prompt) - 1:]
        assert len(ids) == new and all(row[token] >= row.max() - 1e-4 for token, row in zip(ids, rows)), f"request {i}"


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
    config = CONFIGS["C"]
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    (tmp_path / "config.json").write_text(json.dumps(config))
    build = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "build-checkpoint", "--out", str(model_dir),
                            "--config", str(tmp_path / "config.json"), "--seed", "3", "--dtype", "bfloat16", "--std", "0.15"],
                           capture_output=True, text=True, env=env, check=True)
    tensors = load_file(str(model_dir / "model.safetensors"))
    assert json.loads(build.stdout)["parameters"] == sum(t.numel() for t in tensors.values())
    assert float(tensors["l1.norm1"].float().abs().max()) < 0.5 and float(tensors["l0.mix.A_log"].float().std()) > 0.1, \
        "the random-weights mode draws norm weights around zero and decay logarithms with a spread"
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


# --- mechanisms alone ---------------------------------------------------------------------------


def _single(mixer, mlp=None, **extra):
    return _model([_layer(mixer, mlp)], vocab=60, width=32, **extra)


SINGLE = {
    "attention_plain": _single(_attention(2, 2, 8, 8, window=200, keep=0, rot_dims=8, scaling=False, softcap=0.0, v_mix=False)),
    "attention_grouped_keys": _single(_attention(6, 2, 8, 4, window=200, keep=0, v_mix=False, rot_dims=4)),
    "attention_partly_rotated_and_stretched": _single(_attention(2, 1, 16, 8, window=200, keep=0, rot_dims=6, base=50.0, v_mix=False)),
    "attention_unrotated": _single(_attention(2, 1, 12, 8, window=200, keep=0, rot_dims=0, scaling=False, v_mix=False)),
    "attention_tight_cap": _single(_attention(2, 2, 8, 8, window=200, keep=0, rot_dims=8, softcap=0.5, scale=2.0, v_mix=False)),
    "attention_window": _single(_attention(2, 2, 8, 8, window=6, keep=0, rot_dims=4, v_mix=False)),
    "attention_window_of_one": _single(_attention(2, 2, 8, 8, window=1, keep=0, rot_dims=8, v_mix=False)),
    "attention_window_and_kept_tokens": _single(_attention(2, 2, 8, 8, window=6, keep=3, rot_dims=8, v_mix=False)),
    "attention_kept_tokens_beyond_a_page": _single(_attention(2, 1, 8, 8, window=5, keep=11, rot_dims=2, v_mix=False)),
    "attention_wide_heads": _single(_attention(1, 1, 160, 72, window=30, keep=2, rot_dims=64)),
    "mamba": _single(_mamba(32, 8, 4, 4)),
    "mamba_one_tap": _single(_mamba(24, 16, 2, 1)),
    "mamba_wide_state": _single(_mamba(16, 70, 6, 3)),
    "mamba_one_state_one_rank": _single(_mamba(40, 1, 1, 2)),
    "routed": _single(_mamba(16, 4, 2, 2), _moe(6, 2, 16, 24)),
    "routed_top_all": _single(_mamba(16, 4, 2, 2), _moe(4, 4, 16, 8)),
    "routed_top_one_no_shared": _single(_mamba(16, 4, 2, 2), _moe(5, 1, 16, 0)),
    "routed_one_expert": _single(_mamba(16, 4, 2, 2), _moe(1, 1, 16, 8)),
    "unscaled_embedding_large_eps": _single(_mamba(16, 4, 2, 2), None, eps=0.5, scale=1.0),
}


SINGLE["attention_without_mask_rotation_and_cap_keys"] = copy.deepcopy(SINGLE["attention_plain"])
for _key in ("mask", "rot", "softcap", "v_mix"):
    SINGLE["attention_without_mask_rotation_and_cap_keys"]["layers"][0]["mixer"].pop(_key)
SINGLE["attention_with_null_mask"] = copy.deepcopy(SINGLE["attention_grouped_keys"])
SINGLE["attention_with_null_mask"]["layers"][0]["mixer"]["mask"] = None


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("what", sorted(SINGLE))
def test_each_mechanism_alone(what, dtype):
    config = SINGLE[what]
    tensors = random_tensors(config, seed=21, scale=1.3)
    tokens = tokens_for(config, 45, seed=22)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=4)
    rows = [session.step([{"id": "r", "tokens": tokens[:19], "want": list(range(19))}]),
            session.step([{"id": "r", "tokens": tokens[19:23], "want": list(range(4))}])]
    rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[23:]]
    close(np.concatenate(rows), want, dtype, what, routed=config["layers"][0]["mlp"] is not None)


def test_value_mixing_takes_the_first_mixing_layers_values_of_the_same_token():
    """Three attention layers of which the second and third mix: with lambda 1 in the third its
    values are the second layer's, with lambda 0 its own; the first layer's values never enter."""
    layers = [_layer(_attention(2, 2, 8, 8, window=50, keep=0, rot_dims=8, v_mix=False), None),
              _layer(_attention(2, 2, 8, 8, window=50, keep=0, rot_dims=8), None),
              _layer(_attention(2, 2, 8, 8, window=50, keep=0, rot_dims=8), None)]
    config = _model(layers, vocab=40, width=32)
    tokens = tokens_for(config, 30, seed=1)
    for lam in (0.0, 1.0, 0.25):
        tensors = random_tensors(config, seed=2, scale=1.5)
        tensors["l2.mix.vmix"] = torch.tensor(lam, dtype=torch.bfloat16)
        tensors["l1.mix.vmix"] = torch.tensor(0.77, dtype=torch.bfloat16)       # the source's own weight is not used
        want = plain_logits(config, tensors, tokens)
        session = session_for(config, tensors, "float32")
        rows = [session.step([{"id": "r", "tokens": tokens[:12], "want": list(range(12))}])]
        rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[12:]]
        close(np.concatenate(rows), want, "float32", f"lambda {lam}")


# --- rows that a single key decides ------------------------------------------------------------------


def _peaked(window, keep, page_hint=None, heads=2, kv_heads=1, dim=16, vdim=8):
    """One attention layer whose scores are scaled so that the softmax is close to a choice of one
    key: leaving out a visible key or letting in a hidden one changes whole rows."""
    mixer = _attention(heads, kv_heads, dim, vdim, window=window, keep=keep, rot_dims=8, softcap=40.0, scale=3.0, v_mix=False)
    return _model([_layer(mixer, None)], vocab=90, width=32, scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep,page", [(16, 4, 8), (17, 5, 8), (15, 3, 8), (33, 9, 16), (6, 0, 4), (40, 1, 16), (64, 16, 16)])
def test_window_edges_and_kept_tokens_decide_rows_in_prompts_portions_and_decoding(window, keep, page, dtype):
    config = _peaked(window, keep)
    tensors = random_tensors(config, seed=31, scale=2.0)
    tokens = tokens_for(config, 150, seed=32)
    want = plain_logits(config, tensors, tokens)
    # the mask matters: the same model with a window one shorter, one longer, or one kept token fewer differs clearly
    for other in ((window - 1, keep), (window + 1, keep), (window, max(keep - 1, 0)), (window, keep + 1)):
        if other == (window, keep) or other[0] < 1:
            continue
        shifted = plain_logits(_peaked(*other), tensors, tokens)
        assert np.abs(shifted - want).max() > 0.05 * want.std(), f"the test cannot tell window, keep = {other} apart"
    session = session_for(config, tensors, dtype, max_tokens=192, page=page)
    rows = [session.step([{"id": "r", "tokens": tokens[:70], "want": list(range(70))}])]
    rows.append(session.step([{"id": "r", "tokens": tokens[70:72], "want": [0, 1]}]))
    rows.append(session.step([{"id": "r", "tokens": tokens[72:110], "want": list(range(38))}]))
    rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[110:]]
    got = np.concatenate(rows)
    if dtype == "float32":
        close(got, want, dtype, f"window {window}, keep {keep}")
    else:
        gap = got - want
        gap = gap - gap.mean(axis=-1, keepdims=True)
        error = np.sqrt((gap ** 2).mean(axis=-1)) / want.std()
        assert float(np.median(error)) <= 0.05 and float(error.max()) <= 0.5, f"rows off by up to {error.max():.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds_and_a_kept_first_token_stand_out(dtype):
    """Without a window one key far back carries all the weight of the last query; with a window it
    is out of sight unless it is one of the kept first tokens. The query and key are built by hand:
    token 1's embedding gives a large key along one direction, the last token's a large query."""
    width, dim = 32, 16
    mixer = _attention(1, 1, dim, 8, window=400, keep=0, rot_dims=0, scaling=False, softcap=0.0, scale=3.0, v_mix=False)
    base = _model([_layer(mixer, None)], vocab=50, width=width, scale=1.0)
    rng = np.random.default_rng(41)
    tensors = random_tensors(base, seed=42)
    embed = rng.standard_normal((50, width)) * 0.1
    embed[:, 0:2] = 0.0           # ordinary tokens excite neither marked coordinate
    embed[1] = 0.0
    embed[1, 0] = 4.0             # the marked key's token
    embed[2] = 0.0
    embed[2, 1] = 4.0             # the marked query's token
    q = rng.standard_normal((dim, width)) * 0.5
    k = rng.standard_normal((dim, width)) * 0.5
    q[:, 0:2] = 0.0
    k[:, 0:2] = 0.0
    q[0, :] = 0.0
    k[0, :] = 0.0
    q[0, 1] = 1.0                 # the query token puts all of its query on coordinate 0 ...
    k[0, 0] = 1.0                 # ... and the key token all of its key: their score is dim * scale, all others 0
    tensors["embed"] = torch.tensor(embed, dtype=torch.float32).to(torch.bfloat16)
    tensors["l0.mix.q"] = torch.tensor(q, dtype=torch.float32).to(torch.bfloat16)
    tensors["l0.mix.k"] = torch.tensor(k, dtype=torch.float32).to(torch.bfloat16)
    length = 300
    for place, window, keep, seen in ((5, 400, 0, True), (5, 100, 0, False), (5, 100, 6, True), (5, 100, 5, False),
                                      (length - 100, 100, 0, True), (length - 101, 100, 0, False), (127, 173, 0, True),
                                      (128, 172, 0, True), (128, 171, 0, False)):
        config = copy.deepcopy(base)
        config["layers"][0]["mixer"]["mask"] = {"size": window, "keep_first": keep}
        tokens = [int(t) for t in rng.integers(3, 50, size=length)]
        tokens[place] = 1
        tokens[-1] = 2
        want = plain_logits(config, tensors, tokens)
        without = list(tokens)
        without[place] = 7
        moved = np.abs(plain_logits(config, tensors, without)[-1] - want[-1]).max()
        assert (moved > 0.3 * want[-1].std()) == seen, f"the plain model at place {place}, window {window}, keep {keep}"
        for decode_last in (False, True):                 # the last token in the prompt, or decoded alone
            session = session_for(config, tensors, dtype, max_tokens=320, page=16)
            if decode_last:
                session.step([{"id": "r", "tokens": tokens[:-1], "want": []}])
                got = session.step([{"id": "r", "tokens": tokens[-1:], "want": [0]}])
            else:
                got = session.step([{"id": "r", "tokens": tokens, "want": [length - 1]}])
            close(got, want[-1:], dtype, f"key at {place}, window {window}, keep {keep}, decoded {decode_last}", routed=False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_decisive_router_picks_the_plain_experts(dtype):
    """Router logits far apart (a large router matrix and bias): every token's experts are clear, so
    bfloat16 must agree with the plain model row by row, and a wrong expert would show."""
    config = _single(_mamba(16, 4, 2, 2), _moe(6, 2, 16, 8))
    tensors = random_tensors(config, seed=51, scale=1.0)
    tensors["l0.mlp.router"] = (tensors["l0.mlp.router"].float() * 8.0).to(torch.bfloat16)
    tensors["l0.mlp.router.b"] = torch.tensor([3.0, -3.0, 1.0, -1.0, 2.0, -2.0], dtype=torch.bfloat16)
    tokens = tokens_for(config, 64, seed=52)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype)
    got = session.step([{"id": "r", "tokens": tokens, "want": list(range(64))}])
    if dtype == "float32":
        close(got, want, dtype, "decisive router")
    else:
        gap = got - want
        gap = gap - gap.mean(axis=-1, keepdims=True)
        error = np.sqrt((gap ** 2).mean(axis=-1)) / want.std()
        assert int((error > 0.1).sum()) <= 3, f"{int((error > 0.1).sum())} rows look like another expert"


# --- the tensor-core attention kernels (bfloat16, keys and values of one size of 64 or 128) --------------


def _sharp(dim, heads, kv_heads, window, keep, softcap, rot_dims):
    return _attention(heads, kv_heads, dim, dim, window=window, keep=keep, rot_dims=rot_dims, softcap=softcap, scale=4.0 * dim ** -0.5,
                      v_mix=False)


FAST = {
    "heads_of_64_window_past_a_tile": (_sharp(64, 4, 2, 70, 5, 30.0, 32), 8),
    "heads_of_128_kept_tokens_past_a_tile": (_sharp(128, 2, 1, 150, 66, 50.0, 128), 16),
    "window_and_kept_tokens_on_tile_borders": (_sharp(64, 2, 1, 128, 64, 20.0, 64), 16),
    "kept_tokens_meet_the_window": (_sharp(64, 2, 2, 100, 40, 0.0, 16), 32),
    "no_window_tight_cap": (_sharp(128, 4, 4, 100000, 0, 3.0, 64), 64),
    "window_of_three": (_sharp(64, 8, 2, 3, 1, 30.0, 32), 8),
}


@pytest.mark.parametrize("what", sorted(FAST))
def test_tensor_core_attention_with_window_kept_tokens_and_cap(what):
    from paged_kv_serving_b200.parts import SinkWindowAttention

    mixer, page = FAST[what]
    config = _model([_layer(mixer, None), _layer(copy.deepcopy(mixer), None)], vocab=120, width=64, scale=2.0)
    config["layers"][0]["mixer"]["v_mix"] = config["layers"][1]["mixer"]["v_mix"] = True
    tensors = random_tensors(config, seed=61, scale=1.5)
    tokens = tokens_for(config, 330, seed=62)
    want = plain_logits(config, tensors, tokens)

    def run(tensor_cores):
        before = SinkWindowAttention.USE_TENSOR_CORES
        SinkWindowAttention.USE_TENSOR_CORES = tensor_cores
        try:
            session = session_for(config, tensors, "bfloat16", max_tokens=384, page=page)
            assert session.model.layout.blocks[0].mixer._fast(type("C", (), {"dtype": torch.bfloat16})(), page) == tensor_cores
            rows = [session.step([{"id": "r", "tokens": tokens[:200], "want": list(range(200))}]),
                    session.step([{"id": "r", "tokens": tokens[200:240], "want": list(range(40))}]),
                    session.step([{"id": "r", "tokens": tokens[240:243], "want": [0, 1, 2]}])]
            rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[243:]]
            return np.concatenate(rows)
        finally:
            SinkWindowAttention.USE_TENSOR_CORES = before

    fast, general = run(True), run(False)
    for name, got in (("tensor cores", fast), ("general kernel", general)):
        gap = got - want
        gap = gap - gap.mean(axis=-1, keepdims=True)
        error = np.sqrt((gap ** 2).mean(axis=-1)) / want.std()
        assert float(np.median(error)) <= 0.03 and float(error.max()) <= 0.15, f"{what}, {name}: rows off by up to {error.max():.3e}"


def _sharp_two_sizes(dim, vdim, heads, kv_heads, window, keep, softcap, rot_dims):
    return _attention(heads, kv_heads, dim, vdim, window=window, keep=keep, rot_dims=rot_dims, softcap=softcap,
                      scale=4.0 * dim ** -0.5, v_mix=False)


MMA = {
    "keys_of_96_values_of_48": (_sharp_two_sizes(96, 48, 4, 2, 70, 5, 30.0, 32), 8),
    "keys_of_16_values_of_128": (_sharp_two_sizes(16, 128, 2, 1, 150, 66, 50.0, 16), 16),
    "keys_of_160_values_of_16_on_tile_borders": (_sharp_two_sizes(160, 16, 2, 1, 128, 64, 20.0, 64), 16),
    "keys_of_48_values_of_80_no_cap": (_sharp_two_sizes(48, 80, 3, 3, 100, 40, 0.0, 16), 4),
    "keys_of_256_no_window": (_sharp_two_sizes(256, 32, 2, 2, 100000, 0, 3.0, 64), 32),
    "window_of_three_many_heads_a_key": (_sharp_two_sizes(32, 112, 8, 1, 3, 1, 30.0, 32), 8),
}


@pytest.mark.parametrize("what", sorted(MMA))
def test_mma_attention_for_head_sizes_in_steps_of_16(what):
    from paged_kv_serving_b200.parts import SinkWindowAttention

    mixer, page = MMA[what]
    config = _model([_layer(mixer, None), _layer(copy.deepcopy(mixer), None)], vocab=120, width=64, scale=2.0)
    config["layers"][0]["mixer"]["v_mix"] = config["layers"][1]["mixer"]["v_mix"] = True
    tensors = random_tensors(config, seed=71, scale=1.5)
    tokens = tokens_for(config, 330, seed=72)
    want = plain_logits(config, tensors, tokens)

    def run(tensor_cores):
        before = SinkWindowAttention.USE_TENSOR_CORES
        SinkWindowAttention.USE_TENSOR_CORES = tensor_cores
        try:
            session = session_for(config, tensors, "bfloat16", max_tokens=384, page=page)
            probe = type("C", (), {"dtype": torch.bfloat16})()
            assert not session.model.layout.blocks[0].mixer._fast(probe, page)
            assert session.model.layout.blocks[0].mixer._mma(probe) == tensor_cores
            rows = [session.step([{"id": "r", "tokens": tokens[:200], "want": list(range(200))}]),
                    session.step([{"id": "r", "tokens": tokens[200:240], "want": list(range(40))}]),
                    session.step([{"id": "r", "tokens": tokens[240:243], "want": [0, 1, 2]}])]
            rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[243:]]
            return np.concatenate(rows)
        finally:
            SinkWindowAttention.USE_TENSOR_CORES = before

    for name, got in (("tensor cores", run(True)), ("general kernel", run(False))):
        gap = got - want
        gap = gap - gap.mean(axis=-1, keepdims=True)
        error = np.sqrt((gap ** 2).mean(axis=-1)) / want.std()
        assert float(np.median(error)) <= 0.03 and float(error.max()) <= 0.15, f"{what}, {name}: rows off by up to {error.max():.3e}"


# --- seeded random configurations ------------------------------------------------------------------


def _random_config(rng):
    """Layers, sizes and constants drawn at random: odd sizes beside round ones, heads of 64 and 128
    (the tensor-core kernels) beside others, windows and kept tokens around page and tile borders."""
    width = int(rng.choice([24, 40, 64, 96, 100, 128, 192]))
    layers, share = [], None
    for _ in range(int(rng.integers(1, 6))):
        if rng.random() < 0.55:
            kv, group = int(rng.choice([1, 2, 3, 4, 8])), int(rng.choice([1, 1, 2, 3, 4]))
            same = rng.random() < 0.4
            dim = int(rng.choice([64, 128])) if same else int(rng.choice([8, 16, 24, 32, 40, 48, 64, 96, 128, 160]))
            if share is None:
                vdim = dim if same else int(rng.choice([8, 12, 16, 32, 48, 64, 96]))
            else:
                kv, vdim = share
                if same and vdim in (64, 128):
                    dim = vdim
            rot = min(int(rng.choice([0, 2, 4, 8, dim // 4 * 2, dim // 2 * 2, dim])), dim) // 2 * 2
            mixes = bool(rng.random() < 0.6)
            if mixes and share is None:
                share = (kv, vdim)
            mixer = _attention(kv * group, kv, dim, vdim, window=int(rng.choice([1, 5, 16, 31, 32, 33, 64, 100, 150, 1000])),
                               keep=int(rng.choice([0, 0, 1, 4, 7, 16, 17, 70])), rot_dims=rot,
                               base=float(rng.choice([100.0, 10000.0, 50000.0, 1e6])), scaling=bool(rng.random() < 0.6) and rot > 0,
                               softcap=float(rng.choice([0.0, 5.0, 30.0, 80.0])), v_mix=mixes,
                               scale=float(rng.choice([dim ** -0.5, 0.2, 1.0 / dim, 3.0 * dim ** -0.5])))
            if not mixes and rng.random() < 0.5:
                mixer["mixer"].pop("v_mix")
            if rng.random() < 0.2:
                mixer["mixer"].pop("softcap")
        else:
            mixer = _mamba(int(rng.choice([16, 24, 64, 100, 256])), int(rng.choice([1, 2, 4, 8, 16, 32, 33, 64, 100])),
                           int(rng.choice([1, 2, 8, 12, 16, 20])), int(rng.choice([1, 2, 3, 4, 4, 8])))
        mlp = None
        if rng.random() < 0.8:
            experts = int(rng.choice([1, 2, 4, 8, 12]))
            mlp = _moe(experts, int(rng.integers(1, experts + 1)), int(rng.choice([8, 12, 32, 88])), int(rng.choice([0, 8, 120, 40])))
        layers.append(_layer(mixer, mlp))
    return _model(layers, vocab=int(rng.choice([50, 97, 600])), width=width, eps=float(rng.choice([1e-6, 1e-5])),
                  scale=float(rng.choice([1.0, math.sqrt(width), 0.5])))


@pytest.mark.parametrize("seed", range(1000, 1016))
def test_seeded_random_configurations_in_random_cuts(seed):
    rng = np.random.default_rng(seed)
    config = _random_config(rng)
    tensors = random_tensors(config, seed=seed, scale=1.2)
    count = int(rng.choice([40, 90, 200, 330]))
    tokens = tokens_for(config, count, seed=seed + 1)
    want = plain_logits(config, tensors, tokens)
    page = int(rng.choice([8, 16, 16, 32]))
    cuts = [int(c) for c in sorted(rng.choice(np.arange(1, count), size=min(6, count - 1), replace=False))] + [count]
    decoded = [bool(rng.random() < 0.5) for _ in cuts]
    for dtype in DTYPES:
        session = session_for(config, tensors, dtype, max_tokens=count + 64, page=page)
        rows, at = [], 0
        for cut, alone in zip(cuts, decoded):
            last = cut - 8 if alone and cut - at > 30 else cut         # the last eight tokens of some portions one by one
            part = tokens[at:last]
            rows.append(session.step([{"id": "r", "tokens": part, "want": list(range(len(part)))}]))
            rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[last:cut]]
            at = cut
        got = np.concatenate(rows)
        gap = got - want
        gap = gap - gap.mean(axis=-1, keepdims=True)
        error = np.sqrt((gap ** 2).mean(axis=-1)) / max(float(want.std()), 1e-6)
        assert np.isfinite(got).all()
        if dtype == "float32":       # (a router's near tie may move a single row a little further than rounding does)
            assert float(np.median(error)) <= 2e-5 and float(error.max()) <= 1e-3, f"seed {seed}: rows off by up to {error.max():.3e}"
        else:
            assert float(np.median(error)) <= 0.06 and float(error.max()) <= 1.5, f"seed {seed}: rows off by up to {error.max():.3e}"
