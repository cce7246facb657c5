"""What of the Rodelix design runs without a GPU: its configuration, its run order with the calls
that add the model's input again, its layout, tensor names and cache requests, the reordering of
interleaved rotation pairs into halves, and the plain implementation's own consistency."""

from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_rodelix as plain

CONFIG = {
    "architecture": "Rodelix", "vocab": 90, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "logit_softcap": 9.0,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 2, "dim": 6, "vdim": 10, "decay": [0.5, 0.99]}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "mask": {"size": 9}},
         "mlp": {"kind": "dense", "ff": 24}},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 12, "rot_dim": 6, "vdim": 10, "kv_rank": 14, "scale": 0.25, "rot": {"base": 100.0, "dims": 6}},
         "mlp": {"kind": "dense", "ff": 16}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4}, "mlp": None},
    ],
}


def _layout(config=CONFIG):
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.config.rodelix_config import RodelixConfig

    typed = RodelixConfig.from_dict(config)
    return typed, registry.architecture("Rodelix").layout(typed)


def test_config_round_trip_defaults_and_refusals():
    from paged_kv_serving_b200.config.rodelix_config import RodelixConfig

    typed = RodelixConfig.from_dict(CONFIG)
    assert RodelixConfig.from_dict(typed.to_dict()).to_dict() == typed.to_dict()
    assert typed.vocab_size == 90 and typed.d_model == 40 and typed.n_layers == 4
    assert typed.residual_mult == 0.8 and typed.logit_softcap == 9.0
    bare = copy.deepcopy(CONFIG)
    for key in ("loop", "residual_mult", "logit_softcap"):
        del bare[key]
    plainly = RodelixConfig.from_dict(bare)
    assert plainly.residual_mult == 1.0 and plainly.logit_softcap == 0.0 and plainly.run_order() == [(i, False) for i in range(4)]
    for change in (lambda c: c["layers"][0].update(type="something"), lambda c: c["layers"][1]["mixer"].pop("dim"),
                   lambda c: c["layers"][1]["mixer"].update(heads=3), lambda c: c["layers"][0]["mixer"].update(decay=[0.5]),
                   lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), lambda c: c["loop"].update(stop=5),
                   lambda c: c["loop"].update(times=0), lambda c: c["layers"][1]["mlp"].update(kind="moe"),
                   lambda c: c["layers"][2]["mixer"].pop("kv_rank"), lambda c: c.pop("width")):
        bad = copy.deepcopy(CONFIG)
        change(bad)
        with pytest.raises(ValueError):
            RodelixConfig.from_dict(bad)


def test_config_is_found_by_its_architecture_name(tmp_path):
    import json

    from paged_kv_serving_b200.config import load_config
    from paged_kv_serving_b200.config.rodelix_config import RodelixConfig

    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    assert isinstance(load_config(tmp_path), RodelixConfig)


def test_run_order_marks_the_start_of_every_repeated_pass():
    typed, layout = _layout()
    assert typed.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert typed.run_order() == plain.run_order(CONFIG)
    calls = layout.resolved_order()
    assert [(c.layer, c.add_input) for c in calls] == typed.run_order()
    # every call has a cache entry and states of its own
    numbers = [c.cache for c in calls if c.cache is not None] + [n for c in calls for _, n in c.extra]
    assert len(numbers) == len(set(numbers))
    for loop, want in (({"start": 0, "stop": 4, "times": 2}, [0, 1, 2, 3, 0, 1, 2, 3]), ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
                       ({"start": 3, "stop": 4, "times": 1}, [0, 1, 2, 3]), ({"start": 3, "stop": 4, "times": 3}, [0, 1, 2, 3, 3, 3])):
        config = dict(copy.deepcopy(CONFIG), loop=loop)
        order = _layout(config)[0].run_order()
        assert [i for i, _ in order] == want and order == plain.run_order(config)
        assert sum(again for _, again in order) == (loop["times"] - 1 if loop["stop"] > loop["start"] else 0)


def test_layout_names_roles_and_cache_requests():
    from paged_kv_serving_b200.cache.manager import plan_groups
    from paged_kv_serving_b200.parts import LatentAttention, LightningAttention, SandwichBlock, SinkWindowAttention

    typed, layout = _layout()
    names = set(layout.tensor_specs())
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm1b.b", "l0.shift", "l0.mix.g", "l0.mix.norm",
            "l1.mix.q.norm", "l1.mix.k.norm", "l1.mix.temp", "l1.mix.r1", "l1.mix.r2", "l1.norm2b", "l1.mlp.up", "l2.mix.dkv.norm",
            "l2.mix.uk", "l2.mix.q", "l3.shift"} <= names
    assert "l0.norm2" not in names and "l3.norm2b.b" not in names and {"l0.norm2", "l3.norm2b.b"} <= layout.optional_names
    assert layout.tensor_specs()["l2.mix.q"].shape == (2 * 18, 40) and layout.tensor_specs()["l2.mix.dkv"].shape == (20, 40)
    assert all(isinstance(block, SandwichBlock) and block.residual_mult == 0.8 for block in layout.blocks)
    mixers = [block.mixer for block in layout.blocks]
    assert isinstance(mixers[0], LightningAttention) and mixers[0].decays == [0.5, 0.99]
    assert isinstance(mixers[1], SinkWindowAttention) and mixers[1].window == 9 and mixers[3].window is None
    assert mixers[1].norm_weights and mixers[1].head_temperature and mixers[1].distance_bias and mixers[1].rotary is None
    assert isinstance(mixers[2], LatentAttention) and mixers[2].q_rank == 0 and not mixers[2].gate and mixers[2].pairing == "interleaved"
    assert layout.head.softcap == 9.0 and layout.blocks[0].feed_forward is None
    groups, states = plan_groups(layout.cache_entries())
    # the windowed layer's three passes share a group, the latent's three another, the last layer has its own
    assert sorted(len(g.entries) for g in groups) == [1, 3, 3]
    assert {g.window for g in groups} == {9, None} and sum(1 for g in groups if not g.values) == 1
    assert len(states) == 8 + 1                            # a shift state per layer run and the lightning layer's matrix
    assert layout.parameter_count() == sum(int(np.prod(spec.shape)) for spec in layout.tensor_specs().values())


def test_interleaved_pairs_become_halves_without_changing_a_score():
    """The rotated coordinates' rows of the query and key projections are reordered at load so
    that a rotation by halves equals the rotation of interleaved pairs up to one common order."""
    from paged_kv_serving_b200.parts import LatentAttention

    part = LatentAttention(16, 2, 4, 8, 4, 0, 6, 0.5, 100.0, 6, 1e-5, gate=False, pairing="interleaved")
    rng = torch.Generator().manual_seed(1)
    specs = part.param_specs()
    assert "dq" not in specs and "g" not in specs and specs["q"].shape == (2 * 12, 16)
    params = {name: torch.randn(spec.shape, generator=rng) for name, spec in specs.items()}
    part.load(params)
    x = torch.randn((5, 16), generator=rng, dtype=torch.float64)
    positions = torch.arange(5) * 7 + 3
    # plainly: interleaved pairs on the first 6 of the 8 coordinates
    q_plain = plain.rotate_pairs((x @ params["q"].double().T).view(5, 2, 12)[:, :, 4:], positions, 6, 100.0)
    k_plain = plain.rotate_pairs((x @ params["dkv"].double().T)[:, 6:], positions, 6, 100.0)

    def by_halves(v):
        freq = torch.tensor([100.0 ** (-2.0 * i / 6) for i in range(3)], dtype=torch.float64)
        angle = positions.double().reshape([5] + [1] * (v.dim() - 1)) * freq
        a, b = v[..., :3], v[..., 3:6]
        return torch.cat([a * torch.cos(angle) - b * torch.sin(angle), b * torch.cos(angle) + a * torch.sin(angle), v[..., 6:]], dim=-1)

    q_part = by_halves((x @ part.uq.double().T).view(5, 2, 12)[:, :, 4:])
    k_part = by_halves((x @ part.down.double().T)[:, part.kv_off + 6:part.kv_off + 14])
    want = torch.einsum("ihd,jd->hij", q_plain, k_plain)
    got = torch.einsum("ihd,jd->hij", q_part, k_part)
    assert (want - got).abs().max() < 1e-9
    # the unrotated parts and the latent's rows stay where they were
    assert torch.equal(part.uq.view(2, 12, 16)[:, :4], params["q"].view(2, 12, 16)[:, :4])
    assert torch.equal(part.down[part.kv_off:part.kv_off + 6], params["dkv"][:6])


def test_plain_lightning_equals_its_sum_form_and_plain_window_masks_by_distance():
    rng = torch.Generator().manual_seed(2)
    m = {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.7, 1.0]}
    p = {name: torch.randn(shape, generator=rng, dtype=torch.float64) for name, shape in
         (("q", (6, 8)), ("k", (6, 8)), ("v", (8, 8)), ("g", (8, 8)), ("o", (8, 8)), ("norm", (8,)))}
    h = torch.randn((9, 8), generator=rng, dtype=torch.float64)
    got = plain.lightning(h, p, m, 1e-5)
    q, k, v = (plain.silu(h @ p[n].T).view(9, 2, -1) for n in ("q", "k", "v"))
    t = torch.arange(9)
    power = (t[:, None] - t[None, :]).clamp(min=0).double()
    weights = torch.tensor(m["decay"], dtype=torch.float64)[:, None, None] ** power * (t[None, :] <= t[:, None])
    o = torch.einsum("hts,thd,shd,shv->thv", weights, q, k, v).reshape(9, 8)
    want = (plain.rms_weighted(o, p["norm"], 1e-5) * torch.sigmoid(h @ p["g"].T)) @ p["o"].T
    assert (got - want).abs().max() < 1e-10
    # window attention: a token outside the window has no influence, one just inside has
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 3}}
    p = {name: torch.randn(shape, generator=rng, dtype=torch.float64) for name, shape in
         (("q", (8, 8)), ("k", (4, 8)), ("v", (4, 8)), ("o", (8, 8)), ("q.norm", (4,)), ("k.norm", (4,)), ("temp", (2,)))}
    p["r1"], p["r2"] = torch.tensor([0.3, 0.6], dtype=torch.float64), torch.tensor([0.5, 2.0], dtype=torch.float64)
    base = plain.window_attention(h, p, m, 1e-5)
    moved = h.clone()
    moved[2] += 1.0
    after = plain.window_attention(moved, p, m, 1e-5)
    assert (after[5:] - base[5:]).abs().max() < 1e-12 and (after[4] - base[4]).abs().max() > 1e-6
