"""The Rodelix design in the engine against the plain implementation of ``plain_rodelix`` (``-m gpu``).

Small configurations with random weights, none of them a model anyone serves. They differ from
each other in every size and option: head counts with and without grouped keys, key and value
sizes, latent ranks and rotated parts, windows that do and do not fall on page borders, decays,
layer orders, a looped span of one or several layers run two or three times or no loop at all,
with and without a feed-forward, residual factors, with and without a cap on the logits. Some
tests scale the scores so that a single key decides a row, which makes a window that is one token
off, a lost state or a forgotten far key visible.
"""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

import plain_rodelix as plain

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


def _latent(heads=4, dim=24, rot_dim=8, vdim=16, kv_rank=40, base=10000.0, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}}


def _window(heads=4, kv_heads=2, dim=24, vdim=16, size=20, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size is not None:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mixer": mixer}


def _lightning(heads=3, dim=12, vdim=20, decay=(0.5, 0.9, 0.995)):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _layer(mixer, ff):
    return {**mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _model(layers, vocab=150, width=64, eps=1e-5, mult=0.6, softcap=12.0, loop=None):
    config = {"architecture": "Rodelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
              "layers": layers}
    if softcap:
        config["logit_softcap"] = softcap
    if loop:
        config["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return config


#: "A": all three mixers, grouped keys, a window of 20 on pages of 8, two layers run three times.
CONFIG_A = _model([_layer(_lightning(), 72), _layer(_latent(), 96), _layer(_window(), 80), _layer(_latent(2, 16, 4, 24, 24), None)],
                  loop=(1, 3, 3))
#: "B": sizes the tensor-core kernels take (multiples of 16), every query head with keys of its own,
#: windows that straddle pages of 4, one looped layer, no cap, factor 1.
CONFIG_B = _model([_layer(_window(4, 4, 32, 16, size=9), 64), _layer(_latent(4, 32, 16, 32, 48, base=500.0), None),
                   _layer(_lightning(2, 32, 16, (0.8, 0.97)), 48), _layer(_window(6, 2, 16, 48, size=33), 64),
                   _layer(_latent(2, 16, 32, 16, 16), 32)],
                  vocab=97, width=48, eps=1e-6, mult=1.0, softcap=0.0, loop=(2, 3, 2))
#: "C": sizes that are no multiples of 8, some of them odd; no loop; a window longer than the prompts.
CONFIG_C = _model([_layer(_latent(3, 10, 6, 7, 20), 30), _layer(_lightning(1, 9, 7, (0.93,)), None),
                   _layer(_window(3, 1, 10, 7, size=300), 22), _layer(_window(2, 1, 14, 6, size=5), 18),
                   _layer(_lightning(5, 33, 9, (0.3, 0.6, 0.9, 0.99, 1.0)), 26)],
                  vocab=77, width=52, eps=1e-4, mult=0.35, softcap=5.0)
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
PAGE = {"A": 8, "B": 4, "C": 16}


def _specs(config):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.rodelix_config import RodelixConfig

    typed = RodelixConfig.from_dict(config)
    return typed, registry.architecture("Rodelix").layout(typed).tensor_specs()


def random_tensors(config, seed, scale=1.0):
    """Random tensors, rounded to bfloat16 so that both number formats hold the same values."""
    _, specs = _specs(config)
    rng = np.random.default_rng(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].shape
        last = name.rsplit(".", 1)[-1]
        if name.endswith(".b"):
            values = 0.3 * rng.standard_normal(shape)
        elif last in ("norm1", "norm2", "norm1b", "norm2b", "norm") or name.endswith((".q.norm", ".k.norm", "dkv.norm")):
            values = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "shift":
            values = rng.uniform(0.0, 1.0, size=shape)
        elif last == "temp":
            values = rng.uniform(0.6, 1.6, size=shape)
        elif last in ("r1", "r2"):
            values = rng.uniform(0.1, 1.2, size=shape)
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


def row_errors(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"shapes {got.shape} and {want.shape}"
    assert np.isfinite(got).all(), "the engine's logits are not finite"
    gap = got - want
    gap = gap - gap.mean(axis=-1, keepdims=True)
    return np.sqrt((gap ** 2).mean(axis=-1)) / max(float(want.std()), 1e-6)


def close(got, want, dtype, what, bf16_bound=0.08):
    """Rows of logits against the plain ones: the gap with its mean taken off, as a share of the
    spread of the plain logits. float32: every row within 2e-4; bfloat16: rounding moves a row by
    about a percent, the bound leaves room for a few of those and none for a wrong key."""
    error = row_errors(got, want)
    bound = 2e-4 if dtype == "float32" else bf16_bound
    assert float(error.max()) <= bound, f"{what}: row {int(error.argmax())} is off by {error.max():.3e} of the spread"


def plain_logits(config, tensors, tokens):
    return plain.forward(tensors, config, tokens).numpy()


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


def test_the_residual_stream_after_every_layer_run_in_float32():
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=12)
    tokens = tokens_for(config, 33, seed=5)
    _, want = plain.forward(tensors, config, tokens, return_layers=True)
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
    assert len(seen) == len(plain.run_order(config)) == 8
    for index, stream in enumerate(seen):
        gap = np.abs(stream.cpu().numpy() - want[index].numpy()).max()
        assert gap <= 1e-4 * float(want[index].abs().max()), f"the stream after layer run {index} is off by {gap:.3e}"


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
    """Every token alone from position 0 (the shift's zeros, the state's start) for 170 steps:
    decode steps replay a captured graph, pages behind the window go back to the pool."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=5)
    tokens = tokens_for(config, 170, seed=3)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, max_tokens=192, page=4)
    rows = [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens]
    close(np.concatenate(rows), want, dtype, "decoding from the first token")
    given_back = max(sum(1 for page in table if page == -1) for table in session.live["r"].block_tables)
    assert given_back >= 30, "pages behind the window were not given back"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    config = CONFIGS[name]
    tensors = random_tensors(config, seed=6)
    tokens = tokens_for(config, 90, seed=4)
    want = plain_logits(config, tensors, tokens)
    session = session_for(config, tensors, dtype, page=PAGE[name])
    rows, at = [], 0
    for size in [2, 3, 1, 2, 17, 2, 1, 1, 31, 5, 2, 9, 2, 2, 10]:
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


def _plain_choice(config, tensors, prompt, ids, slack):
    rows = plain_logits(config, tensors, list(prompt) + ids[:-1])[len(prompt) - 1:]
    return all(row[token] >= row.max() - slack(row) for token, row in zip(ids, rows))


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    from paged_kv_serving_b200.api import generate
    from paged_kv_serving_b200.weights.random_init import write_model_folder

    config = CONFIGS["A"]
    typed, _ = _specs(config)
    tensors = random_tensors(config, seed=11, scale=1.5)
    write_model_folder(tmp_path, typed, tensors)
    prompts = [tokens_for(config, n, seed=20 + n) for n in (5, 33, 18)]
    got = generate(tmp_path, prompts, max_new_tokens=12, dtype=dtype, block_size=8, max_batched_tokens=24, max_running_seqs=4)
    for prompt, samples in zip(prompts, got):
        ids = samples[0]
        assert len(ids) == 12
        assert _plain_choice(config, tensors, prompt, ids, (lambda row: 1e-4) if dtype == "float32" else (lambda row: 0.1 * row.std()))


def test_forked_samples_share_pages_and_copy_states(tmp_path):
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
        assert len(ids) == 9 and _plain_choice(config, tensors, prompt, ids, lambda row: 1e-4)


def test_a_cramped_pool_preempts_and_recomputes_states_and_pages():
    from paged_kv_serving_b200.api import engine_for
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

    config = CONFIGS["A"]
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
        assert len(ids) == new and _plain_choice(config, tensors, prompt, ids, lambda row: 1e-4), f"request {i}"


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
    made = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "build-checkpoint", "--out", str(model_dir),
                           "--config", str(tmp_path / "config.json"), "--seed", "3", "--dtype", "bfloat16", "--std", "0.15"],
                          capture_output=True, text=True, env=env, check=True)
    tensors = load_file(str(model_dir / "model.safetensors"))
    assert json.loads(made.stdout)["parameters"] == sum(t.numel() for t in tensors.values())
    run = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "generate", "--model", str(model_dir),
                          "--prompt-ids", "5,17,3,20", "--max-new-tokens", "6", "--dtype", "float32", "--block-size", "4"],
                         capture_output=True, text=True, env=env, check=True)
    line = [json.loads(text) for text in run.stdout.splitlines() if text.startswith("{")][0]
    ids = line["samples"][0]
    assert len(ids) == 6 and _plain_choice(config, tensors, [5, 17, 3, 20], ids, lambda row: 1e-4)

    tokens = tokens_for(config, 30, seed=9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[23:], "want": [6]}], "end": ["a"]}]
    replay = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", "float32", "--out", str(out_dir),
                             "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, env=env, check=True)
    assert [text for text in replay.stdout.splitlines() if text.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = plain_logits(config, tensors, tokens)
    first = np.fromfile(out_dir / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out_dir / "2.f32", dtype="<f4").reshape(1, -1)
    assert not (out_dir / "1.f32").exists()
    close(np.concatenate([first, last]), want[[0, 20, 29]], "float32", "trace program")


# --- each mechanism alone ------------------------------------------------------------------------------

SINGLE = {
    "latent_attention": _model([_layer(_latent(3, 12, 6, 10, 18), None)], vocab=60, width=40),
    "latent_attention_one_head": _model([_layer(_latent(1, 16, 16, 16, 32, base=77.0), None)], vocab=60, width=32),
    "window_attention_grouped": _model([_layer(_window(6, 2, 12, 10, size=7), None)], vocab=60, width=40),
    "window_attention_own_keys": _model([_layer(_window(2, 2, 32, 32, size=11), None)], vocab=60, width=40),
    "window_of_one": _model([_layer(_window(2, 1, 8, 8, size=1), None)], vocab=60, width=40),
    "attention_without_mask": _model([_layer(_window(2, 1, 8, 12, size=None), None)], vocab=60, width=40),
    "lightning": _model([_layer(_lightning(), None)], vocab=60, width=40),
    "lightning_without_decay": _model([_layer(_lightning(2, 64, 8, (1.0, 1.0)), None)], vocab=60, width=40),
    "lightning_wide_keys": _model([_layer(_lightning(1, 130, 5, (0.9,)), None)], vocab=60, width=40),
    "dense_feed_forward": _model([_layer(_lightning(1, 4, 4, (0.5,)), 50)], vocab=60, width=40, mult=1.0, softcap=0.0),
    "one_layer_looped_thrice": _model([_layer(_window(2, 1, 8, 8, size=6), 24)], vocab=60, width=40, loop=(0, 1, 3)),
    "loop_of_one_pass": _model([_layer(_latent(2, 8, 4, 8, 12), 24), _layer(_lightning(), 24)], vocab=60, width=40, loop=(0, 2, 1)),
    "empty_loop": _model([_layer(_latent(2, 8, 4, 8, 12), 24), _layer(_lightning(), 24)], vocab=60, width=40, loop=(1, 1, 4)),
}


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
    close(np.concatenate(rows), want, dtype, what)


def test_the_plain_mechanisms_are_told_apart():
    """What the comparisons above could not see would make them worthless: the plain model without
    the shift, with halves instead of interleaved pairs, without the distance bias, without the
    temperature, without the added embeddings of a repeated pass, each differs clearly."""
    config = CONFIGS["A"]
    tensors = random_tensors(config, seed=3)
    tokens = tokens_for(config, 40, seed=1)
    want = plain_logits(config, tensors, tokens)
    for name_end, value in (("shift", 0.0), ("mix.r1", 0.0), ("mix.temp", 1.0)):
        changed = {k: (torch.full_like(v, value) if k.endswith(name_end) else v) for k, v in tensors.items()}
        assert np.abs(plain_logits(config, changed, tokens) - want).max() > 0.02 * want.std(), name_end
    no_loop = copy.deepcopy(config)
    del no_loop["loop"]
    assert np.abs(plain_logits(no_loop, tensors, tokens) - want).max() > 0.02 * want.std()


def test_norm_and_shift_kernels_against_the_plain_functions():
    from paged_kv_serving_b200.ops import mixer_ops

    rng = torch.Generator().manual_seed(5)
    n, width = 11, 52
    hidden = torch.randn((n, width), generator=rng)
    update = torch.randn((n, width), generator=rng) * 3 + 1
    addend = torch.randn((n, width), generator=rng)
    w = [torch.randn((width,), generator=rng) for _ in range(4)]
    h_dev = hidden.cuda().clone()
    out = mixer_ops.layer_norm_step(h_dev, update.cuda(), (w[0].cuda(), w[1].cuda()), 0.7, addend=addend.cuda(),
                                    pre=(w[2].cuda(), w[3].cuda()), out_dtype=torch.float32, eps=1e-5)
    x = hidden.double() + 0.7 * plain.layer_norm(update.double(), w[0], w[1], 1e-5) + addend.double()
    assert (h_dev.cpu().double() - x).abs().max() < 1e-5
    assert (out.cpu().double() - plain.layer_norm(x, w[2], w[3], 1e-5)).abs().max() < 1e-5
    rows = torch.tensor([7, 2], dtype=torch.int32).cuda()
    before = h_dev.clone()
    picked = mixer_ops.layer_norm_step(h_dev, pre=(w[2].cuda(), w[3].cuda()), out_dtype=torch.float32, rows=rows, eps=1e-5)
    assert torch.equal(h_dev, before) and (picked.cpu().double() - plain.layer_norm(x[[7, 2]], w[2], w[3], 1e-5)).abs().max() < 1e-5
    # the shift over two entries: the first continues a request whose state holds its last row
    state = torch.zeros((3, width))
    state[2] = torch.randn((width,), generator=rng)
    state_dev = state.cuda().clone()
    ints = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    shifted = mixer_ops.token_shift(hidden.cuda(), w[0].cuda(), state_dev, ints([0] * 4 + [1] * 7), ints([0, 4, 11]), ints([2, 0]),
                                    torch.float32)
    first = plain.token_shift(torch.cat([state[2:3], hidden[:4]]).double(), w[0])[1:]
    second = plain.token_shift(hidden[4:].double(), w[0])
    assert (shifted.cpu().double() - torch.cat([first, second])).abs().max() < 1e-5
    assert torch.equal(state_dev[2].cpu(), hidden[3]) and torch.equal(state_dev[0].cpu(), hidden[10])


def _plain_lightning_rows(proj, offsets, decay, weight, eps, state, heads, dim, vdim):
    """Token by token in float64 on one entry's rows; ``state [heads, dim, vdim]`` is updated in place."""
    silu = lambda z: z / (1.0 + torch.exp(-z))
    n = proj.shape[0]
    q = silu(proj[:, offsets["q"]:offsets["q"] + heads * dim]).view(n, heads, dim)
    k = silu(proj[:, offsets["k"]:offsets["k"] + heads * dim]).view(n, heads, dim)
    v = silu(proj[:, offsets["v"]:offsets["v"] + heads * vdim]).view(n, heads, vdim)
    gate = torch.sigmoid(proj[:, offsets["g"]:offsets["g"] + heads * vdim])
    rows = []
    for t in range(n):
        state.mul_(decay[:, None, None]).add_(k[t][:, :, None] * v[t][:, None, :])
        rows.append(torch.einsum("hdv,hd->hv", state, q[t]).reshape(heads * vdim))
    o = torch.stack(rows)
    return o / torch.sqrt((o * o).mean(dim=1, keepdim=True) + eps) * weight * gate


@pytest.mark.parametrize("heads,dim,vdim", [(3, 12, 20), (2, 32, 64), (1, 128, 24), (2, 130, 8), (5, 7, 3)])
def test_linear_attention_kernel_in_a_row_and_in_chunks_over_ragged_entries(heads, dim, vdim):
    """Entries of unequal lengths whose ends fall before, on and after chunk edges, an entry of one
    token and an empty one, in two steps so that the second starts from states the first left; a
    short step (every entry in a row) beside long ones (chunks side by side), all against the
    recurrence token by token."""
    from paged_kv_serving_b200.ops import mixer_ops

    rng = torch.Generator().manual_seed(heads * 1000 + dim)
    qk, vg = heads * dim, heads * vdim
    offsets = {"q": 0, "k": qk, "v": 2 * qk, "g": 2 * qk + vg}
    ld = 2 * qk + 2 * vg + 3
    decay = torch.tensor([0.999, 0.5, 0.93, 1.0, 0.8][:heads], dtype=torch.float64)
    weight = torch.randn((vg,), generator=rng).double()
    slots = [4, 0, 2, 5, 1]
    plain_states = {slot: torch.zeros((heads, dim, vdim), dtype=torch.float64) for slot in slots}
    state = torch.zeros((6, heads, vdim, dim), dtype=torch.float32).cuda()
    ints = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    for lengths, cut in (([130, 1, 64, 0, 197], True), ([63, 129, 2, 5, 128], True), ([3, 1, 2, 0, 4], False),
                         ([1000, 0, 0, 1, 0], True)):
        assert (mixer_ops.lightning_chunk(sum(lengths), len(lengths)) > 0) == cut
        tokens = sum(lengths)
        proj = (torch.randn((tokens, ld), generator=rng) * 1.5).float()
        starts = [0]
        for n in lengths:
            starts.append(starts[-1] + n)
        got = mixer_ops.lightning(proj.cuda(), offsets, decay.float().cuda(), weight.float().cuda(), 1e-5, state, ints(starts),
                                  ints(slots), heads, dim, vdim, torch.float32).cpu().double()
        for s, slot in enumerate(slots):
            if lengths[s] == 0:
                continue
            want = _plain_lightning_rows(proj[starts[s]:starts[s + 1]].double(), offsets, decay, weight, 1e-5, plain_states[slot],
                                         heads, dim, vdim)
            assert (got[starts[s]:starts[s + 1]] - want).abs().max() <= 2e-4 * want.abs().max(), (lengths, s)
        for slot in slots:
            held = state[slot].cpu().double().transpose(1, 2)
            assert (held - plain_states[slot]).abs().max() <= 1e-5 * max(1.0, plain_states[slot].abs().max().item()), (lengths, slot)
    assert state[3].abs().max().item() == 0.0               # a slot no entry named


# --- rows that a single key decides ------------------------------------------------------------------


def _peaked(size, heads=2, kv_heads=1, dim=16, vdim=8):
    """One window-attention layer whose scores are scaled so that the softmax is close to a choice
    of one key: leaving out a visible key or letting in a hidden one changes whole rows."""
    return _model([_layer(_window(heads, kv_heads, dim, vdim, size=size, scale=3.0), None)], vocab=90, width=32, mult=1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size,page,dim", [(16, 8, 16), (17, 8, 16), (15, 8, 12), (33, 16, 16), (6, 4, 16), (40, 16, 10), (64, 16, 32)])
def test_window_edges_decide_rows_in_prompts_portions_and_decoding(size, page, dim, dtype):
    config = _peaked(size, dim=dim)
    tensors = random_tensors(config, seed=31, scale=2.0)
    for name in tensors:
        if name.endswith(("r1", "r2")):
            tensors[name] = tensors[name] * 0.2          # a small bias: far keys must still matter
    tokens = tokens_for(config, 150, seed=32)
    want = plain_logits(config, tensors, tokens)
    for other in (size - 1, size + 1):
        shifted = plain_logits(_peaked(other, dim=dim), tensors, tokens)
        assert np.abs(shifted - want).max() > 0.05 * want.std(), f"the test cannot tell a window of {other} apart"
    session = session_for(config, tensors, dtype, max_tokens=192, page=page)
    rows = [session.step([{"id": "r", "tokens": tokens[:70], "want": list(range(70))}])]
    rows.append(session.step([{"id": "r", "tokens": tokens[70:72], "want": [0, 1]}]))
    rows.append(session.step([{"id": "r", "tokens": tokens[72:110], "want": list(range(38))}]))
    rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[110:]]
    got = np.concatenate(rows)
    if dtype == "float32":
        close(got, want, dtype, f"window {size}")
    else:
        error = row_errors(got, want)
        assert float(np.median(error)) <= 0.05 and float(error.max()) <= 0.5, f"rows off by up to {error.max():.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ("latent_attention", "lightning"))
def test_one_far_token_among_hundreds_decides_the_last_rows(kind, dtype):
    """A marked token early in a long sequence must reach the last positions: through the cached
    latent of a page far back (attention without a window), or through a state that hardly
    decays. The weights are built by hand on top of random ones: the marked token's embedding
    excites one coordinate that gives a large key, the last tokens' embedding another that gives a
    large query along the same direction. Taking the marked token away must change those rows."""
    width = 32
    if kind == "latent_attention":
        layer = _layer(_latent(2, 16, 16, 16, 32, scale=1.0), None)
    else:
        layer = _layer(_lightning(2, 16, 16, (0.9995, 1.0)), None)
    config = _model([layer], vocab=50, width=width, mult=1.0, softcap=0.0)
    tensors = {k: v.float() for k, v in random_tensors(config, seed=42).items()}
    embed = tensors["embed"] * 0.3
    embed[:, 0:2] = 0.0               # ordinary tokens excite neither marked coordinate
    embed[1], embed[2] = 0.0, 0.0
    embed[1, 0] = 4.0                 # the marked key's token
    embed[2, 1] = 4.0                 # the marked query's token
    tensors["embed"] = embed
    tensors["l0.shift"] = torch.zeros(width)
    tensors["l0.norm1"], tensors["l0.norm1.b"] = torch.ones(width), torch.zeros(width)
    if kind == "latent_attention":
        tensors["l0.mix.dkv"][0, 0] += 3.0         # latent coordinate 0 follows the key marker ...
        tensors["l0.mix.uk"][0, 0] += 3.0          # ... and becomes head 0's key coordinate 0
        tensors["l0.mix.q"][0, 1] += 3.0           # head 0's query coordinate 0 follows the query marker
    else:
        tensors["l0.mix.k"][0, 0] += 3.0
        tensors["l0.mix.q"][0, 1] += 3.0
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    tokens = [3 + t % 47 for t in tokens_for(config, 420, seed=43)]
    tokens[3] = 1
    tokens[401:] = [2] * 19
    other = list(tokens)
    other[3] = 7
    picked = [299] + list(range(401, 420))
    want, moved = plain_logits(config, tensors, tokens)[picked], plain_logits(config, tensors, other)[picked]
    matters = row_errors(moved[1:], want[1:])
    assert float(matters.min()) > 0.2, f"the far token does not matter enough to be missed ({matters.min():.3f})"
    session = session_for(config, tensors, dtype, max_tokens=448, page=16)
    rows = [session.step([{"id": "r", "tokens": tokens[:300], "want": [299]}]),
            session.step([{"id": "r", "tokens": tokens[300:402], "want": [101]}])]
    rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[402:]]
    error = row_errors(np.concatenate(rows), want)
    assert float(error.max()) <= (2e-4 if dtype == "float32" else 0.1), f"rows off by up to {error.max():.3e}"


# --- the tensor-core kernels against the general ones ---------------------------------------------------


def test_tensor_core_attention_kernels_serve_sizes_in_steps_of_16_and_agree_with_the_general_ones():
    from paged_kv_serving_b200.parts.latent_attention import LatentAttention
    from paged_kv_serving_b200.parts.sink_attention import SinkWindowAttention

    config = CONFIGS["B"]
    tensors = random_tensors(config, seed=51)
    tokens = tokens_for(config, 140, seed=52)
    want = plain_logits(config, tensors, tokens)
    results = {}
    for fast in (True, False):
        LatentAttention.USE_TENSOR_CORES = SinkWindowAttention.USE_TENSOR_CORES = fast
        try:
            session = session_for(config, tensors, "bfloat16", page=16)
            mixers = [block.mixer for block in session.model.layout.blocks]
            rows = [session.step([{"id": "r", "tokens": tokens[:100], "want": list(range(100))}])]
            rows += [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[100:]]
            results[fast] = np.concatenate(rows)
            if fast:
                ctx_like = type("C", (), {"dtype": torch.bfloat16})
                assert all(m._mma(ctx_like) for m in mixers if isinstance(m, SinkWindowAttention))
                assert all(m._tensor_cores(ctx_like) for m in mixers if isinstance(m, LatentAttention))
        finally:
            LatentAttention.USE_TENSOR_CORES = SinkWindowAttention.USE_TENSOR_CORES = True
    close(results[True], want, "bfloat16", "tensor-core kernels")
    close(results[False], want, "bfloat16", "general kernels")


@pytest.mark.parametrize("size,page,dim,heads,kv_heads", [(70, 16, 64, 4, 2), (33, 64, 128, 2, 1), (129, 8, 64, 3, 3), (None, 16, 64, 2, 1)])
def test_long_entries_on_tcgen05_beside_short_ones_with_temperature_and_distance_bias(size, page, dim, heads, kv_heads, monkeypatch):
    """Heads of 64 and 128 in bfloat16: a step that holds a long entry gives it to the tcgen05 kernel and its
    short entries to the ``mma.sync`` kernel. Scores are peaked so that a window off by one, a bias or a
    temperature left out (one head's is negative) would change whole rows; two requests run side by side."""
    from paged_kv_serving_b200 import ops

    config = _model([_layer(_window(heads, kv_heads, dim, dim, size=size, scale=0.6), None)], vocab=90, width=48, mult=1.0)
    tensors = random_tensors(config, seed=71, scale=2.0)
    for name in tensors:
        if name.endswith(("r1", "r2")):
            tensors[name] = tensors[name] * 0.3
        if name.endswith("temp"):
            tensors[name] = tensors[name].clone()
            tensors[name][0] = -tensors[name][0].abs()
    first, second = tokens_for(config, 330, seed=72), tokens_for(config, 200, seed=73)
    want = {"a": plain_logits(config, tensors, first), "b": plain_logits(config, tensors, second)}
    if size is not None:
        shifted = plain_logits(_model([_layer(_window(heads, kv_heads, dim, dim, size=size + 1, scale=0.6), None)], vocab=90, width=48,
                                      mult=1.0), tensors, first)
        assert np.abs(shifted - want["a"]).max() > 0.05 * want["a"].std(), "the test cannot tell a window one longer apart"
    calls = {"tcgen05": 0}
    real = ops.attention_prefill_tcgen05

    def counted(*args, **kwargs):
        calls["tcgen05"] += 1
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "attention_prefill_tcgen05", counted)
    session = session_for(config, tensors, "bfloat16", max_tokens=640, page=page)
    got = {"a": [], "b": []}
    # a: 200 tokens | 3 | 64 | 1 ... ; b: 5 | 130 | 2 | 63 (below the border: the other kernel alone)
    steps = [[("a", 0, 200), ("b", 0, 5)], [("a", 200, 203), ("b", 5, 135)], [("a", 203, 267), ("b", 135, 137)],
             [("a", 267, 268), ("b", 137, 200)], [("a", 268, 330)]]
    for step in steps:
        entries = [{"id": r, "tokens": (first if r == "a" else second)[lo:hi], "want": list(range(hi - lo))} for r, lo, hi in step]
        rows = session.step(entries)
        at = 0
        for r, lo, hi in step:
            got[r].append(rows[at:at + hi - lo])
            at += hi - lo
    assert calls["tcgen05"] == 3, "steps with an entry of 64 tokens or more did not reach the tcgen05 kernel"
    for r in ("a", "b"):
        error = row_errors(np.concatenate(got[r]), want[r])
        assert float(np.median(error)) <= 0.05 and float(error.max()) <= 0.5, f"request {r}: rows off by up to {error.max():.3e}"


# --- seeded random configurations -----------------------------------------------------------------------


def _random_config(rng):
    def mixer():
        kind = rng.choice(["latent", "window", "lightning"])
        if kind == "latent":
            rot = int(rng.choice([2, 4, 6, 8, 16]))
            return _latent(int(rng.integers(1, 5)), int(rng.choice([4, 8, 10, 16, 32])), rot, int(rng.choice([4, 7, 16, 32])),
                           int(rng.choice([8, 12, 16, 48])), base=float(rng.choice([100.0, 10000.0, 500000.0])))
        if kind == "window":
            groups = int(rng.integers(1, 4))
            return _window(groups * int(rng.integers(1, 4)), groups, int(rng.choice([6, 8, 16, 32])), int(rng.choice([5, 8, 16, 48])),
                           size=int(rng.integers(1, 40)) if rng.random() < 0.85 else None)
        heads = int(rng.integers(1, 5))
        return _lightning(heads, int(rng.choice([3, 8, 16, 40])), int(rng.choice([4, 9, 16, 32])),
                          [float(d) for d in rng.uniform(0.3, 1.0, size=heads)])

    count = int(rng.integers(1, 6))
    layers = [_layer(mixer(), int(rng.choice([0, 16, 30, 64]))) for _ in range(count)]
    loop = None
    if rng.random() < 0.7:
        start = int(rng.integers(0, count))
        stop = int(rng.integers(start, count + 1))
        loop = (start, stop, int(rng.integers(1, 4)))
    return _model(layers, vocab=int(rng.integers(20, 200)), width=int(rng.choice([24, 32, 52, 64])), eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                  mult=float(rng.uniform(0.2, 1.2)), softcap=float(rng.choice([0.0, 4.0, 30.0])), loop=loop)


@pytest.mark.parametrize("seed", range(2000, 2016))
def test_seeded_random_configurations_in_random_cuts(seed):
    rng = np.random.default_rng(seed)
    config = _random_config(rng)
    dtype = DTYPES[seed % 2]
    tensors = random_tensors(config, seed=seed)
    lengths = [int(n) for n in rng.integers(1, 90, size=3)]
    tokens = {f"r{i}": tokens_for(config, n, seed=seed + i) for i, n in enumerate(lengths)}
    want = {k: plain_logits(config, tensors, v) for k, v in tokens.items()}
    session = session_for(config, tensors, dtype, max_tokens=320, page=int(rng.choice([4, 8, 16])), max_live=3)
    got = {k: [] for k in tokens}
    at = {k: 0 for k in tokens}
    while any(at[k] < len(tokens[k]) for k in tokens):
        entries, order, end = [], [], []
        for key in tokens:
            left = len(tokens[key]) - at[key]
            if left == 0 or rng.random() < 0.25:
                continue
            count = min(left, int(rng.choice([1, 1, 2, 3, 8, 29])))
            part = tokens[key][at[key]:at[key] + count]
            entries.append({"id": key, "tokens": part, "want": list(range(count))})
            order.append((key, count))
            at[key] += count
            if at[key] == len(tokens[key]):
                end.append(key)
        if not entries:
            continue
        out = session.step(entries, end=end)
        row = 0
        for key, n in order:
            got[key].append(out[row:row + n])
            row += n
    for key in tokens:
        close(np.concatenate(got[key]), want[key], dtype, f"seed {seed} request {key}", bf16_bound=0.15)
