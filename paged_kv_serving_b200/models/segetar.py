"""The Segetar design: a decoder whose layers, in an order the configuration lists, mix tokens by a Mamba selective
scan or by two mixers side by side that read the same input: grouped-query attention over a sliding window beside a
linear attention with a matrix state. In a "parallel" layer the attention has biases, a norm over its whole query and
key projections, a rotation of interleaved pairs and a sigmoid gate per head, the other side is gated linear attention
(a decay per token and key coordinate), and the two outputs are added with one factor each. In a "parallel_2" layer
the attention has neither biases nor rotation nor gate, the other side is retention (a fixed decay per head, rotated
queries and keys), and the update is half the sum of the two outputs after an RMS norm of each. Layers are pre-norm
(``x += mixer(norm1(x)); x += ff(norm2(x))``) with a dense gated feed-forward (tanh GELU, biases), a mixture of gated
experts chosen by sigmoid scores within the best groups of experts, or none. A span of layers may run several times with
the same weights, each pass with its own cache and states; in front of every pass the stream becomes ``W [x; x0] +
step[pass]`` with ``x0`` the embedding output.

This module is all that is specific to the design: which parts a layer has, with which numbers of the configuration,
the run order, and the tensor names of a model folder (``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step`` and per
layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``).
"""

from __future__ import annotations

from paged_kv_serving_b200.config.registry import register_architecture
from paged_kv_serving_b200.config.segetar_config import SegetarConfig
from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
from paged_kv_serving_b200.parts import (
    GatedDense, GatedLinearAttention, GatedRoutedExperts, Mamba1, ParallelMixers, PassInput, PreNormBlock, Retention, RMSNorm,
    ScaledRotaryFrequencies, SinkWindowAttention,
)
from paged_kv_serving_b200.parts.base import Part

__all__ = ["Segetar"]


def _rotary(sizes: dict):
    rot = sizes.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    return ScaledRotaryFrequencies(dims, float(rot["base"])) if dims else None


def _window_attention(sizes: dict, width: int, eps: float, full: bool):
    """The attention side; ``full``: with biases, rotation of interleaved pairs and a gate per head."""
    mask = sizes.get("mask") or {}
    part = SinkWindowAttention(width, sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"], float(sizes["scale"]),
                               rotary=_rotary(sizes) if full else None, unit_norm=True, eps=eps, window=mask.get("size"),
                               norm_weights=True, joint_norm=True, bias=full, pairing="interleaved" if full else "halves",
                               head_gate=full)
    names = {"q": "q", "k": "k", "v": "v", "o": "o", "q.norm": "q_norm", "k.norm": "k_norm"}
    if full:
        names.update({"q.b": "q_b", "k.b": "k_b", "v.b": "v_b", "g": "g"})
    return part, names


def _mamba(sizes: dict, width: int):
    part = Mamba1(width, sizes["inner"], sizes["state"], sizes["dt_rank"], sizes["conv"])
    names = {"in": "in_proj", "conv": "conv", "conv.b": "conv_b", "x": "x_proj", "dt": "dt_proj", "dt.b": "dt_b",
             "A_log": "A_log", "D": "D", "o": "o"}
    return part, names


def _mixer(kind: str, sizes: dict, width: int, eps: float, tensor_shape) -> tuple[Part, dict[str, tuple[Part, str]]]:
    """The mixer of a layer and the map from its tensors' names in the file (behind ``l<i>.mix.``) to (part, local
    name). ``tensor_shape(name)`` gives the shape of a stored tensor where a size is not in the configuration."""
    if kind == "mamba1":
        part, names = _mamba(sizes, width)
        return part, {stored: (part, local) for stored, local in names.items()}
    left, left_names = _window_attention(sizes["left"], width, eps, full=kind == "parallel")
    r = sizes["right"]
    if kind == "parallel":
        rank = tensor_shape("right.a1")[0]          # the decay's projection goes through as many numbers as a1 has rows
        right = GatedLinearAttention(width, r["heads"], r["dim"], r["vdim"], rank, float(r["tau"]), eps)
        right_names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2.b": "a2_b"}
        part = ParallelMixers(left, right, width, "scaled", float(sizes["left_scale"]), float(sizes["right_scale"]), eps)
        own = {}
    else:
        right = Retention(width, r["heads"], r["dim"], r["vdim"], r["decay"], eps, rotary=_rotary(r))
        right_names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
        part = ParallelMixers(left, right, width, "normed_mean", eps=eps)
        own = {"left.out": (part, "left_out"), "right.out": (part, "right_out")}
    names = dict(own)
    names.update({f"left.{stored}": (left, local) for stored, local in left_names.items()})
    names.update({f"right.{stored}": (right, local) for stored, local in right_names.items()})
    return part, names


def _feed_forward(mlp: dict, width: int):
    if mlp.get("kind", "dense") == "dense":
        part = GatedDense(width, mlp["ff"], "gelu_tanh", bias=True)
        return part, {"gate": "gate", "gate.b": "gate_b", "up": "up", "up.b": "up_b", "down": "down", "down.b": "down_b"}
    router = mlp["router"]
    groups = router.get("groups") or {}
    experts = router["experts"]
    part = GatedRoutedExperts(width, experts, router["top"], mlp["expert"]["ff"], 0, "silu", scoring="sigmoid",
                              groups=int(groups.get("count") or 1), keep_groups=int(groups.get("keep") or groups.get("count") or 1),
                              weight_scale=float(router.get("scale", 1.0)))
    names = {"router": "router", "correction": "correction"}
    for e in range(experts):
        for kind in ("gate", "up", "down"):
            names[f"e{e}.{kind}"] = f"e{e}_{kind}"
    return part, names


@register_architecture("Segetar")
class Segetar:
    config_class = SegetarConfig
    #: ``layout`` takes the shapes of a model folder's tensors: the number of values the decay's projection of a gated
    #: linear attention passes through is the row count of its first matrix (without tensors, in the random-weights
    #: mode, the key ``rank`` beside that mixer's sizes gives it)
    sizes_from_tensors = True

    @staticmethod
    def layout(config: SegetarConfig, tensor_shapes: dict | None = None) -> ModelLayout:
        d = config.data
        width, vocab, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        names: dict = {}
        optional: set = set()
        blocks = []
        for index, layer in enumerate(d["layers"]):
            prefix = f"l{index}."

            def tensor_shape(name: str, prefix=prefix, layer=layer):
                if tensor_shapes is not None and f"{prefix}mix.{name}" in tensor_shapes:
                    return tuple(tensor_shapes[f"{prefix}mix.{name}"])
                rank = (layer["mixer"].get("right") or {}).get("rank")
                if name == "right.a1" and rank:
                    return (int(rank), width)
                raise ValueError(f"the size of {prefix}mix.{name} is neither in the configuration nor known from a tensor")

            mixer, mixer_names = _mixer(layer["type"], layer["mixer"], width, eps, tensor_shape)
            for stored, target in mixer_names.items():
                names[f"{prefix}mix.{stored}"] = target
            norm1 = RMSNorm(width, eps)
            names[prefix + "norm1"] = (norm1, "weight")
            norm2 = feed_forward = None
            if layer.get("mlp"):
                norm2 = RMSNorm(width, eps)
                names[prefix + "norm2"] = (norm2, "weight")
                feed_forward, ff_names = _feed_forward(layer["mlp"], width)
                for stored, local in ff_names.items():
                    names[f"{prefix}mlp.{stored}"] = (feed_forward, local)
            else:
                optional.add(prefix + "norm2")
            blocks.append(PreNormBlock(norm1, mixer, norm2, feed_forward))
        final_norm = RMSNorm(width, eps)
        names["final.norm"] = (final_norm, "weight")
        pass_input = None
        if config.loop_times:
            pass_input = PassInput(width, config.loop_times)
            names["loop.in"], names["loop.step"] = (pass_input, "mix"), (pass_input, "step")
        else:
            optional.update(("loop.in", "loop.step"))
        return ModelLayout(
            width=width, vocab_size=vocab, max_positions=config.max_seq_len, blocks=blocks,
            # every call gets a cache and states of its own
            order=[LayerCall(index, enter_pass=number) for index, number in config.run_order()],
            final_norm=final_norm, names=names, embedding_name="embed", head_name="head", optional_names=optional,
            pass_input=pass_input,
        )
