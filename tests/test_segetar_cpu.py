"""What of the Segetar design runs without a GPU: its configuration, its run order with the passes over a looped
span, its layout, tensor names and cache requests, the reordering of neighbouring rotation pairs into halves, the
size that only a tensor's shape gives, and the plain implementation's own consistency."""

from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_segetar as plain

CONFIG = {
    "architecture": "Segetar", "vocab": 90, "width": 40, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 24, "state": 5, "dt_rank": 3, "conv": 4}, "mlp": {"kind": "dense", "ff": 28}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "mask": {"size": 9}, "rot": {"dims": 6, "base": 100.0}},
                   "right": {"heads": 2, "dim": 6, "vdim": 10, "tau": 4.0, "rank": 3}, "left_scale": 0.7, "right_scale": 1.1},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}}},
        {"type": "parallel_2",
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "mask": {"size": 17}},
                   "right": {"heads": 2, "dim": 8, "vdim": 6, "decay": [0.9, 0.99], "rot": {"dims": 4, "base": 50.0}}},
         "mlp": None},
        {"type": "mamba1", "mixer": {"inner": 16, "state": 4, "dt_rank": 2, "conv": 2}, "mlp": None},
    ],
}


def _layout(config=CONFIG, tensor_shapes=None):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.segetar_config import SegetarConfig

    typed = SegetarConfig.from_dict(config)
    return typed, registry.architecture("Segetar").layout(typed, tensor_shapes=tensor_shapes)


def test_config_round_trip_and_refusals():
    from paged_kv_serving_b200.config.segetar_config import SegetarConfig

    typed = SegetarConfig.from_dict(CONFIG)
    assert SegetarConfig.from_dict(typed.to_dict()).to_dict() == typed.to_dict()
    assert typed.vocab_size == 90 and typed.d_model == 40 and typed.n_layers == 4 and typed.loop_times == 3
    bare = copy.deepcopy(CONFIG)
    del bare["loop"]
    assert SegetarConfig.from_dict(bare).run_order() == [(i, None) for i in range(4)] and SegetarConfig.from_dict(bare).loop_times == 0
    for change in (lambda c: c["layers"][0].update(type="something"), lambda c: c["layers"][1]["mixer"]["left"].pop("dim"),
                   lambda c: c["layers"][1]["mixer"]["left"].update(heads=3), lambda c: c["layers"][2]["mixer"]["right"].update(decay=[0.5]),
                   lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), lambda c: c["loop"].update(stop=5),
                   lambda c: c["loop"].update(times=0), lambda c: c["layers"][0]["mlp"].update(kind="other"),
                   lambda c: c["layers"][1]["mixer"].pop("left_scale"), lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0),
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                   lambda c: c["layers"][1]["mlp"]["router"].update(top=5), lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=14),
                   lambda c: c["layers"][0]["mixer"].pop("state"), lambda c: c.pop("width")):
        bad = copy.deepcopy(CONFIG)
        change(bad)
        with pytest.raises(ValueError):
            SegetarConfig.from_dict(bad)


def test_config_is_found_by_its_architecture_name(tmp_path):
    import json

    from paged_kv_serving_b200.config import load_config
    from paged_kv_serving_b200.config.segetar_config import SegetarConfig

    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    assert isinstance(load_config(tmp_path), SegetarConfig)


def test_run_order_numbers_the_passes_and_every_call_has_its_own_cache_and_states():
    typed, layout = _layout()
    assert typed.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert typed.run_order() == plain.run_order(CONFIG)
    calls = layout.resolved_order()
    assert [(c.layer, c.enter_pass) for c in calls] == typed.run_order()
    numbers = [c.cache for c in calls if c.cache is not None] + [n for c in calls for _, n in c.extra]
    assert len(numbers) == len(set(numbers))
    for loop, want in (({"start": 0, "stop": 4, "times": 2}, [0, 1, 2, 3, 0, 1, 2, 3]), ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
                       ({"start": 3, "stop": 4, "times": 1}, [0, 1, 2, 3]), ({"start": 3, "stop": 4, "times": 3}, [0, 1, 2, 3, 3, 3])):
        config = dict(copy.deepcopy(CONFIG), loop=loop)
        typed, layout = _layout(config)
        order = typed.run_order()
        assert [i for i, _ in order] == want and order == plain.run_order(config)
        passes = [number for _, number in order if number is not None]
        assert passes == (list(range(loop["times"])) if loop["stop"] > loop["start"] else [])
        # a span that never runs twice still has its pass input (the stream is mixed with the model's input once)
        assert (layout.pass_input is not None) == bool(passes)
        assert ("loop.in" in layout.tensor_specs()) == bool(passes) and ("loop.in" in layout.optional_names) != bool(passes)


def test_layout_names_roles_and_cache_requests():
    from paged_kv_serving_b200.cache.manager import plan_groups
    from paged_kv_serving_b200.parts import (
        GatedDense, GatedLinearAttention, GatedRoutedExperts, Mamba1, ParallelMixers, PreNormBlock, Retention, SinkWindowAttention,
    )

    typed, layout = _layout()
    specs = layout.tensor_specs()
    assert {"embed", "head", "final.norm", "loop.in", "loop.step", "l0.norm1", "l0.norm2", "l0.mix.A_log", "l0.mix.conv.b", "l0.mlp.gate.b",
            "l0.mlp.down.b", "l1.mix.left.q.b", "l1.mix.left.q.norm", "l1.mix.left.g", "l1.mix.right.a1", "l1.mix.right.a2.b",
            "l1.mix.right.norm", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e5.down", "l2.mix.left.out", "l2.mix.right.out",
            "l2.mix.right.g", "l3.mix.dt.b"} <= set(specs)
    assert not {"l2.norm2", "l2.mix.left.q.b", "l2.mix.left.g", "l2.mix.right.norm", "l1.mix.left.out", "l1.mlp.router.b"} & set(specs)
    assert "l2.norm2" in layout.optional_names and "l3.norm2" in layout.optional_names
    assert specs["loop.in"].shape == (40, 80) and specs["loop.step"].shape == (3, 40)
    assert specs["l1.mix.left.q.norm"].shape == (48,) and specs["l1.mix.left.k.norm"].shape == (24,) and specs["l1.mix.left.g"].shape == (4, 40)
    assert specs["l1.mix.right.a1"].shape == (3, 40) and specs["l1.mix.right.a2"].shape == (12, 3) and specs["l1.mix.right.norm"].shape == (10,)
    assert all(isinstance(block, PreNormBlock) for block in layout.blocks)
    mixers = [block.mixer for block in layout.blocks]
    assert isinstance(mixers[0], Mamba1) and isinstance(mixers[1], ParallelMixers) and isinstance(mixers[2], ParallelMixers)
    full, bare = mixers[1].left, mixers[2].left
    assert isinstance(full, SinkWindowAttention) and full.bias and full.joint_norm and full.head_gate and full.pairing == "interleaved"
    assert full.window == 9 and full.rotary.dims == 6 and full.keep_first == 0
    assert not bare.bias and bare.joint_norm and not bare.head_gate and bare.rotary is None and bare.window == 17
    assert isinstance(mixers[1].right, GatedLinearAttention) and mixers[1].right.rank == 3 and mixers[1].right.tau == 4.0
    assert isinstance(mixers[2].right, Retention) and mixers[2].right.decays == [0.9, 0.99] and mixers[2].right.rotary.dims == 4
    assert (mixers[1].combine, mixers[1].left_scale, mixers[1].right_scale) == ("scaled", 0.7, 1.1) and mixers[2].combine == "normed_mean"
    feeds = [block.feed_forward for block in layout.blocks]
    assert isinstance(feeds[0], GatedDense) and feeds[0].activation == "gelu_tanh" and feeds[0].bias
    assert isinstance(feeds[1], GatedRoutedExperts) and (feeds[1].scoring, feeds[1].groups, feeds[1].keep_groups, feeds[1].weight_scale) == ("sigmoid", 3, 2, 1.5)
    assert feeds[2] is None and feeds[3] is None
    groups, states = plan_groups(layout.cache_entries())
    # the three passes of each two-sided layer share a page group
    assert sorted(len(g.entries) for g in groups) == [3, 3] and {g.window for g in groups} == {9, 17}
    # per layer run: a scan state and a convolution tail for Mamba, a matrix state for a two-sided mixer
    assert len(states) == 2 + 3 + 3 + 2
    assert layout.parameter_count() == sum(int(np.prod(spec.shape)) for spec in specs.values())


def test_the_decay_projections_inner_size_comes_from_the_tensor():
    config = copy.deepcopy(CONFIG)
    del config["layers"][1]["mixer"]["right"]["rank"]
    with pytest.raises(ValueError):
        _layout(config)
    _, layout = _layout(config, tensor_shapes={"l1.mix.right.a1": (7, 40)})
    assert layout.tensor_specs()["l1.mix.right.a1"].shape == (7, 40) and layout.tensor_specs()["l1.mix.right.a2"].shape == (12, 7)
    # a stored tensor wins over the key of the random-weights mode
    _, layout = _layout(CONFIG, tensor_shapes={"l1.mix.right.a1": (5, 40)})
    assert layout.blocks[1].mixer.right.rank == 5


def test_neighbouring_pairs_become_halves_without_changing_a_score():
    """The rows of the query and key projections, their biases and their norm weights are reordered at load so that
    a rotation by halves equals the rotation of neighbouring pairs up to one common order of a head's coordinates."""
    from paged_kv_serving_b200.parts import ScaledRotaryFrequencies, SinkWindowAttention

    H, G, dim, rot = 4, 2, 10, 6
    part = SinkWindowAttention(16, H, G, dim, 4, 0.5, rotary=ScaledRotaryFrequencies(rot, 100.0), unit_norm=True, eps=1e-5, window=7,
                               norm_weights=True, joint_norm=True, bias=True, pairing="interleaved", head_gate=True)
    rng = torch.Generator().manual_seed(1)
    params = {name: torch.randn(spec.shape, generator=rng) for name, spec in part.param_specs().items()}
    part.load(params)
    x = torch.randn((5, 16), generator=rng, dtype=torch.float64)
    positions = torch.arange(5) * 7 + 3
    q_plain = plain.rotate_neighbours((plain.unit_rms(x @ params["q"].double().T + params["q_b"], 1e-5) * params["q_norm"]).view(5, H, dim),
                                      positions, rot, 100.0)
    k_plain = plain.rotate_neighbours((plain.unit_rms(x @ params["k"].double().T + params["k_b"], 1e-5) * params["k_norm"]).view(5, G, dim),
                                      positions, rot, 100.0)
    fused = x @ part.qkv.double().T + torch.cat([part.qkv_bias.double(), torch.zeros(part.fused_rows - part.qkv_bias.numel())])
    q_part = plain.rotate_halves((plain.unit_rms(fused[:, :H * dim], 1e-5) * part.q_norm).view(5, H, dim), positions, rot, 100.0)
    k_part = plain.rotate_halves((plain.unit_rms(fused[:, H * dim:(H + G) * dim], 1e-5) * part.k_norm).view(5, G, dim), positions, rot, 100.0)
    assert (torch.einsum("ihd,jgd->hgij", q_plain, k_plain) - torch.einsum("ihd,jgd->hgij", q_part, k_part)).abs().max() < 1e-9
    # values, gates and the unrotated coordinates stay where they were
    assert torch.equal(part.qkv[(H + G) * dim:(H + G) * dim + G * 4], params["v"]) and torch.equal(part.qkv[part.gate_at:part.gate_at + H], params["g"])
    assert torch.equal(part.qkv[:H * dim].view(H, dim, 16)[:, rot:], params["q"].view(H, dim, 16)[:, rot:])
    # without a rotation nothing moves
    still = SinkWindowAttention(16, H, G, dim, 4, 0.5, rotary=None, unit_norm=True, norm_weights=True, joint_norm=True, pairing="interleaved")
    still.load({name: params[name] for name in still.param_specs()})
    assert torch.equal(still.qkv[:H * dim], params["q"])


def test_plain_scan_equals_its_sum_form_and_plain_window_masks_by_distance():
    rng = torch.Generator().manual_seed(2)
    n, H, D, V = 9, 2, 3, 4
    q, k = (torch.randn((n, H, D), generator=rng, dtype=torch.float64) for _ in range(2))
    v = torch.randn((n, H, V), generator=rng, dtype=torch.float64)
    decay = torch.rand((n, H, D), generator=rng, dtype=torch.float64) * 0.5 + 0.5
    got = plain.matrix_state_scan(q, k, v, decay)
    # token t reads key s <= t through the product of the decays of tokens s + 1 .. t, coordinate by coordinate
    want = torch.zeros_like(got)
    for t in range(n):
        for s in range(t + 1):
            through = decay[s + 1:t + 1].prod(dim=0)                      # [H, D]
            want[t] += torch.einsum("hd,hd,hv->hv", q[t] * through, k[s], v[s])
    assert (got - want).abs().max() < 1e-12
    # window attention: a token outside the window has no influence, one just inside has
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 3}, "rot": {"dims": 2, "base": 10.0}}
    p = {name: torch.randn(shape, generator=rng, dtype=torch.float64) for name, shape in
         (("q", (8, 8)), ("k", (4, 8)), ("v", (4, 8)), ("o", (8, 8)), ("q.norm", (8,)), ("k.norm", (4,)), ("q.b", (8,)), ("k.b", (4,)),
          ("v.b", (4,)), ("g", (2, 8)))}
    h = torch.randn((n, 8), generator=rng, dtype=torch.float64)
    for full in (True, False):
        base = plain.window_attention(h, p, m, 1e-5, torch.arange(n), full)
        moved = h.clone()
        moved[2] += 1.0
        after = plain.window_attention(moved, p, m, 1e-5, torch.arange(n), full)
        assert (after[5:] - base[5:]).abs().max() < 1e-12 and (after[4] - base[4]).abs().max() > 1e-6


def test_plain_router_keeps_to_the_best_groups():
    rng = torch.Generator().manual_seed(3)
    router = {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    p = {"router": torch.eye(8, dtype=torch.float64), "correction": torch.randn((8,), generator=rng, dtype=torch.float64)}
    logits = torch.randn((40, 8), generator=rng, dtype=torch.float64)
    weights = plain.router_weights(logits, p, router)
    assert (weights != 0).sum(dim=1).eq(3).all() and torch.allclose(weights.sum(dim=1), torch.full((40,), 2.0, dtype=torch.float64))
    used_groups = (weights.view(40, 4, 2) != 0).any(dim=-1).sum(dim=1)
    assert used_groups.le(2).all()
    choice = torch.sigmoid(logits) + p["correction"]
    group_score = choice.view(40, 4, 2).sum(dim=-1)                     # groups of two: both count
    best = group_score.topk(2, dim=-1).indices
    for t in range(40):
        groups_of_chosen = {int(e) // 2 for e in (weights[t] != 0).nonzero().flatten()}
        assert groups_of_chosen <= {int(g) for g in best[t]}
