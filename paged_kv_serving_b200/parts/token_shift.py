"""A blend of every token's mixer input with that of the token before it."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext

__all__ = ["TokenShift"]


@register_part("mixer", "token_shift")
class TokenShift(Part):
    """``h_t <- h_t + (h_{t-1} - h_t) * mix``, element by element, with ``h_{t-1}`` the row of the
    token before as it was before this step (zeros in front of a sequence's first token). The
    last row a request has brought so far is a float32 state of the layer call
    (``state_requests``), so a sequence may arrive in portions. Takes float32 rows and hands out
    the compute type."""

    graph_safe = True
    STATE = "shift_previous"

    def __init__(self, width: int) -> None:
        self.width = int(width)
        self.mix: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"mix": ParamSpec((self.width,), "vector", init=(0.5, 0.2))}

    def state_requests(self) -> dict[str, StateRequest]:
        return {self.STATE: StateRequest((self.width,))}

    def forward(self, h: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        return mixer_ops.token_shift(h, self.mix, ctx.states[binding.extra[self.STATE]], ctx.ints(ctx.TOKEN_SEQ),
                                     ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS), ctx.dtype)
