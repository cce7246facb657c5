"""The two ends of a model: token ids to the residual stream, and normalised rows to logits."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import ParamSpec, Part, StepContext

__all__ = ["LinearHead", "PassInput", "TokenEmbedding"]


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``hidden = table[ids] * scale`` widened to float32, ``scale`` 1 unless given
    (reference: src/paged_kv_serving/engine/model.py:266-267). ``forward(ctx)`` reads the step's
    token ids from ``ctx`` (and, for a token that was sampled on the device by the step before,
    from ``ctx.fed_back_ids``). An architecture whose embeddings are summed with others or
    looked up otherwise gives its layout another part with the same ``forward``."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, scale: float = 1.0) -> None:
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.scale = float(scale)
        self.table: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"table": ParamSpec((self.vocab_size, self.width))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.table = params["table"].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        fed_back_at = ctx.ints(ctx.TOKEN_FEEDBACK) if ctx.fed_back_ids is not None else None
        return ops.embedding_gather(self.table, ctx.ints(ctx.TOKEN_IDS), ctx.status, ctx.fed_back_ids, fed_back_at, self.scale)


@register_part("head", "linear")
class LinearHead(Part):
    """``logits = normed @ weight^T`` in float32, ``weight [vocab, width]``; with ``tied`` the
    weight is that embedding part's table (reference: src/paged_kv_serving/engine/model.py:261-264,
    where the head is always tied). ``forward(normed, ctx)`` gets the rows the final norm left
    (only the wanted ones). With ``softcap`` ``c > 0`` the logits become ``c * tanh(logits / c)``. A head
    with a scale or several outputs is another part with the same ``forward``."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, tied: TokenEmbedding | None = None, softcap: float = 0.0) -> None:
        if softcap < 0:
            raise ValueError("softcap must be >= 0")
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.tied = tied
        self.softcap = float(softcap)
        self._weight: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {} if self.tied is not None else {"weight": ParamSpec((self.vocab_size, self.width))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        if "weight" in params:
            self._weight = params["weight"].contiguous()

    @property
    def weight(self) -> torch.Tensor:
        return self.tied.table if self.tied is not None else self._weight

    def forward(self, normed: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = gemm.linear(normed, self.weight, out_dtype=torch.float32, chain=True)
        if self.softcap > 0.0:
            from paged_kv_serving_b200.ops import mixer_ops

            mixer_ops.softcap(logits, self.softcap)
        return logits


@register_part("embedding", "pass_input")
class PassInput(Part):
    """What stands in front of each pass over a span of layers that runs several times: the stream ``x`` is replaced by
    ``W [x; x0] + step[t]``, with ``x0`` the model's input (the embedding part's output for the step's tokens), ``W
    [width, 2 width]`` (tensor ``mix``, the columns of ``x`` first) and ``step [passes, width]``, ``t`` the number of the
    pass. ``forward(hidden, pending, model_input, t)`` adds a pending update to the stream first, then gives the stream
    its new value in place. The product takes operands in the compute type and keeps its float32 result, to which the
    step vector is added in float32."""

    graph_safe = True

    def __init__(self, width: int, passes: int) -> None:
        if width < 1 or passes < 1:
            raise ValueError("width and passes must be >= 1")
        self.width, self.passes = int(width), int(passes)
        self.mix: torch.Tensor | None = None
        self.step: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"mix": ParamSpec((self.width, 2 * self.width)),
                "step": ParamSpec((self.passes, self.width), "vector", init=(0.0, 0.1))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.mix = params["mix"].contiguous()
        self.step = params["step"].contiguous()

    def forward(self, hidden: torch.Tensor, pending: torch.Tensor | None, model_input: torch.Tensor, number: int) -> None:
        from paged_kv_serving_b200.ops import mixer_ops

        if not 0 <= number < self.passes:
            raise ValueError(f"pass {number} of {self.passes}")
        both = mixer_ops.pair_rows(hidden, pending, model_input, self.mix.dtype)
        mixed = gemm.linear(both, self.mix, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        mixer_ops.assign_bias(hidden, mixed, self.step[number])
