"""Typed configuration of the Segetar design, read from the ``config.json`` of a model folder.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``layers`` and the optional section ``loop``
(``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row with the same
weights). Each layer has ``type`` ("parallel", "parallel_2" or "mamba1"), its mixer's sizes and
constants under ``mixer`` (the two-sided mixers hold a ``left`` and a ``right`` section), and ``mlp``:
``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {...}}`` or null for
none. The class keeps the file's content as it is (``to_dict`` returns it) and checks the keys the
design needs.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

__all__ = ["SegetarConfig"]

_ATTENTION = {"heads", "kv_heads", "dim", "vdim", "scale"}
_REQUIRED = {
    "parallel": {"left", "right", "left_scale", "right_scale"},
    "parallel_2": {"left", "right"},
    "mamba1": {"inner", "state", "dt_rank", "conv"},
}
_RIGHT = {"parallel": {"heads", "dim", "vdim", "tau"}, "parallel_2": {"heads", "dim", "vdim", "decay"}}
#: Positions an engine may be asked for when the file sets no bound of its own: angles are
#: computed from the position, no table limits them.
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be an integer >= 1, found {value!r}")
    return value


def _lacking(section: Any, keys: set, what: str) -> None:
    if not isinstance(section, dict):
        raise ValueError(f"{what}: a section with the keys {sorted(keys)} is missing")
    lacking = sorted(keys - set(section))
    if lacking:
        raise ValueError(f"{what}: missing keys {lacking}")


def _check_rotation(section: dict, what: str) -> None:
    rot = section.get("rot")
    if rot:
        dims = rot.get("dims", 0)
        if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > section["dim"]:
            raise ValueError(f"{what}: rot.dims must be even and at most the head size")
        if dims and not float(rot.get("base", 0.0)) > 1.0:
            raise ValueError(f"{what}: rot.base must be > 1")


@dataclass(frozen=True)
class SegetarConfig:
    data: dict = field(repr=False)
    architecture: str = "Segetar"

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
            mixer = layer.get("mixer")
            _lacking(mixer, _REQUIRED[kind], f"layer {i} ({kind})")
            if kind == "mamba1":
                for key in _REQUIRED[kind]:
                    _positive_int(mixer[key], f"layer {i}: mixer.{key}")
            else:
                left, right = mixer["left"], mixer["right"]
                _lacking(left, _ATTENTION, f"layer {i} ({kind}) left")
                _lacking(right, _RIGHT[kind], f"layer {i} ({kind}) right")
                for side, keys in ((left, ("heads", "kv_heads", "dim", "vdim")), (right, ("heads", "dim", "vdim"))):
                    for key in keys:
                        _positive_int(side[key], f"layer {i}: mixer.{key}")
                if left["heads"] % left["kv_heads"]:
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
                if (left.get("mask") or {}).get("size") is not None:
                    _positive_int(left["mask"]["size"], f"layer {i}: mixer.left.mask.size")
                _check_rotation(left, f"layer {i} left")
                _check_rotation(right, f"layer {i} right")
                if kind == "parallel" and not float(right["tau"]) > 0.0:
                    raise ValueError(f"layer {i}: tau must be > 0")
                if kind == "parallel_2" and len(right["decay"]) != right["heads"]:
                    raise ValueError(f"layer {i}: one decay per head")
            self._check_mlp(i, layer.get("mlp"))
        loop = d.get("loop")
        if loop:
            start, stop = loop.get("start"), loop.get("stop")
            _positive_int(loop.get("times"), "loop.times")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start <= stop <= len(d["layers"])):
                raise ValueError("loop.start and loop.stop must bound a range of layers")
        if "max_positions" in d:
            _positive_int(d["max_positions"], "max_positions")

    @staticmethod
    def _check_mlp(i: int, mlp: Any) -> None:
        if mlp is None:
            return
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
        elif kind == "moe":
            _positive_int((mlp.get("expert") or {}).get("ff"), f"layer {i}: mlp.expert.ff")
            router = mlp.get("router") or {}
            experts = _positive_int(router.get("experts"), f"layer {i}: mlp.router.experts")
            top = _positive_int(router.get("top"), f"layer {i}: mlp.router.top")
            groups = router.get("groups")
            allowed = experts
            if groups:
                count = _positive_int(groups.get("count"), f"layer {i}: mlp.router.groups.count")
                keep = _positive_int(groups.get("keep"), f"layer {i}: mlp.router.groups.keep")
                if experts % count or keep > count:
                    raise ValueError(f"layer {i}: the experts form equal groups, of which at most all are kept")
                allowed = experts // count * keep
            if top > allowed:
                raise ValueError(f"layer {i}: more experts to choose than may be chosen")
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

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
    def loop_times(self) -> int:
        """How often the looped span runs (0: the model has no such span)."""
        loop = self.data.get("loop")
        if not loop or loop["stop"] <= loop["start"]:
            return 0
        return int(loop["times"])

    def run_order(self) -> list[tuple[int, int | None]]:
        """``(layer, pass)`` in the order the layers run; ``pass`` is the number of the pass over the
        looped span that starts right in front of this run of the layer, ``None`` elsewhere."""
        count = len(self.data["layers"])
        if not self.loop_times:
            return [(i, None) for i in range(count)]
        loop = self.data["loop"]
        start, stop = loop["start"], loop["stop"]
        order: list[tuple[int, int | None]] = [(i, None) for i in range(start)]
        for number in range(self.loop_times):
            order += [(i, number if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, count)]

    def to_dict(self) -> dict[str, Any]:
        out = copy.deepcopy(self.data)
        out["architecture"] = self.architecture
        return out

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "SegetarConfig":
        data = copy.deepcopy(dict(data))
        name = data.get("architecture", "Segetar")
        return cls(data, architecture=name)
