"""Typed configuration of the Rodelix design, read from the ``config.json`` of a model folder.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (the factor on every
residual update), ``logit_softcap``, ``layers`` (each with ``type``: "latent_attention", "attention"
or "lightning", the mixer's sizes and constants under ``mixer``, and ``mlp``: a dense feed-forward
or null for none) and the optional section ``loop`` (``start``, ``stop``, ``times``: layers ``start
.. stop - 1`` run ``times`` times in a row with the same weights). The class keeps the file's
content as it is (``to_dict`` returns it) and checks the keys the design needs.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

__all__ = ["RodelixConfig"]

_REQUIRED = {
    "latent_attention": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"},
    "attention": {"heads", "kv_heads", "dim", "vdim", "scale"},
    "lightning": {"heads", "dim", "vdim", "decay"},
}
#: Positions an engine may be asked for when the file sets no bound of its own: angles are
#: computed from the position, no table limits them.
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be an integer >= 1, found {value!r}")
    return value


@dataclass(frozen=True)
class RodelixConfig:
    data: dict = field(repr=False)
    architecture: str = "Rodelix"

    def __post_init__(self) -> None:
        d = self.data
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
            if kind not in _REQUIRED:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(sorted(_REQUIRED))}")
            mixer = layer.get("mixer") or {}
            lacking = sorted(_REQUIRED[kind] - set(mixer))
            if lacking:
                raise ValueError(f"layer {i} ({kind}): missing keys {lacking}")
            for key in ("heads", "dim", "vdim"):
                _positive_int(mixer[key], f"layer {i}: mixer.{key}")
            if kind == "attention":
                if mixer["heads"] % _positive_int(mixer["kv_heads"], f"layer {i}: mixer.kv_heads"):
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
                if (mixer.get("mask") or {}).get("size") is not None:
                    _positive_int(mixer["mask"]["size"], f"layer {i}: mixer.mask.size")
            if kind == "lightning" and len(mixer["decay"]) != mixer["heads"]:
                raise ValueError(f"layer {i}: one decay per head")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
        loop = d.get("loop")
        if loop:
            start, stop = loop["start"], loop["stop"]
            _positive_int(loop["times"], "loop.times")
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

    @property
    def residual_mult(self) -> float:
        value = self.data.get("residual_mult")
        return 1.0 if value is None else float(value)

    @property
    def logit_softcap(self) -> float:
        return float(self.data.get("logit_softcap") or 0.0)

    def run_order(self) -> list[tuple[int, bool]]:
        """``(layer, the model's input is added in front of it)`` in the order the layers run: a
        repeated pass over the looped span starts by adding the input once more."""
        count = len(self.data["layers"])
        loop = self.data.get("loop")
        if not loop or loop["stop"] <= loop["start"]:
            return [(i, False) for i in range(count)]
        start, stop, times = loop["start"], loop["stop"], loop["times"]
        order = [(i, False) for i in range(start)]
        for pass_number in range(times):
            order += [(i, pass_number > 0 and i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, count)]

    def to_dict(self) -> dict[str, Any]:
        out = copy.deepcopy(self.data)
        out["architecture"] = self.architecture
        return out

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "RodelixConfig":
        data = copy.deepcopy(dict(data))
        name = data.get("architecture", "Rodelix")
        return cls(data, architecture=name)
