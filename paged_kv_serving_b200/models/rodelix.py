"""The Rodelix design: a decoder whose layers, in an order the configuration lists, mix tokens by
attention over a cached latent (interleaved rotation of a key part all heads share), by
grouped-query attention over a sliding window (weighted unit-norm queries and keys, a temperature
per head, a bias growing with the logarithm of the distance, no rotation) or by linear attention
with a fixed decay per head; every mixer reads its input blended with that of the token before
(token shift); feed-forwards are dense with a squared relu; layer norms with weight and bias sit in
front of and behind every sublayer and every update is multiplied by one factor; a span of layers
may run several times with the same weights, each pass with its own cache and states and each
repeated pass starting from the stream plus the embeddings; the logits are softly capped.

This module is all that is specific to the design: which parts a layer has, with which numbers
of the configuration, the run order, and the tensor names of a model folder (``embed``, ``head``,
``final.norm``, ``final.norm.b``, and per layer ``l<i>.norm1`` ``.norm1b`` ``.norm2`` ``.norm2b`` (each
with ``.b``), ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``).
"""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_architecture
from paged_kv_serving_b200.config.rodelix_config import RodelixConfig
from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
from paged_kv_serving_b200.parts import (
    Dense, LatentAttention, LayerNorm, LightningAttention, LinearHead, SandwichBlock, SinkWindowAttention, TokenShift,
)

__all__ = ["Rodelix"]


def _mixer(kind: str, sizes: dict, width: int, eps: float):
    """The mixer of a layer and the map from its tensors' names in the file to the part's."""
    if kind == "latent_attention":
        rot = sizes.get("rot") or {}
        rot_dims = int(rot.get("dims") or 0)
        part = LatentAttention(width, sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], 0, sizes["kv_rank"],
                               float(sizes["scale"]), float(rot.get("base") or 10000.0), rot_dims, eps, gate=False,
                               pairing="interleaved")
        names = {"q": "q", "dkv": "dkv", "dkv.norm": "dkv_norm", "uk": "uk", "uv": "uv", "o": "o"}
    elif kind == "attention":
        mask = sizes.get("mask") or {}
        part = SinkWindowAttention(width, sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"], float(sizes["scale"]),
                                   rotary=None, unit_norm=True, eps=eps, window=mask.get("size"), norm_weights=True,
                                   head_temperature=True, distance_bias=True)
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q.norm": "q_norm", "k.norm": "k_norm", "temp": "temp", "r1": "r1",
                 "r2": "r2"}
    elif kind == "lightning":
        part = LightningAttention(width, sizes["heads"], sizes["dim"], sizes["vdim"], sizes["decay"], eps)
        names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
    else:
        raise ValueError(f"unknown mixer type {kind!r}")
    return part, names


@register_architecture("Rodelix")
class Rodelix:
    config_class = RodelixConfig

    @staticmethod
    def layout(config: RodelixConfig) -> ModelLayout:
        d = config.data
        width, vocab, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        names: dict = {}
        optional: set = set()

        def norm(name: str, rows_dtype=None) -> LayerNorm:
            part = LayerNorm(width, eps, rows_dtype=rows_dtype)
            names[name], names[name + ".b"] = (part, "weight"), (part, "bias")
            return part

        blocks = []
        for index, layer in enumerate(d["layers"]):
            prefix = f"l{index}."
            norm1 = norm(prefix + "norm1", torch.float32)        # the shift reads float32 rows
            shift = TokenShift(width)
            names[prefix + "shift"] = (shift, "mix")
            mixer, mixer_names = _mixer(layer["type"], layer["mixer"], width, eps)
            for stored, local in mixer_names.items():
                names[f"{prefix}mix.{stored}"] = (mixer, local)
            norm1b = norm(prefix + "norm1b")
            norm2 = feed_forward = norm2b = None
            if layer.get("mlp"):
                norm2, norm2b = norm(prefix + "norm2"), norm(prefix + "norm2b")
                feed_forward = Dense(width, layer["mlp"]["ff"], "relu_squared")
                names[prefix + "mlp.up"], names[prefix + "mlp.down"] = (feed_forward, "up"), (feed_forward, "down")
            else:
                optional.update(prefix + n for n in ("norm2", "norm2.b", "norm2b", "norm2b.b"))
            blocks.append(SandwichBlock(norm1, mixer, norm1b, norm2, feed_forward, norm2b, residual_mult=config.residual_mult,
                                        input_shift=shift))
        final_norm = norm("final.norm")
        head = LinearHead(vocab, width, softcap=config.logit_softcap)
        names["head"] = (head, "weight")
        return ModelLayout(
            width=width, vocab_size=vocab, max_positions=config.max_seq_len, blocks=blocks,
            # every call gets a cache and states of its own
            order=[LayerCall(index, add_input=again) for index, again in config.run_order()],
            final_norm=final_norm, names=names, embedding_name="embed", head=head, optional_names=optional,
        )
