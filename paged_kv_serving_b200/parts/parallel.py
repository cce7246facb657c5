"""Two mixers side by side that read the same input."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import arena, gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StepContext

__all__ = ["ParallelMixers"]


@register_part("mixer", "parallel_pair")
class ParallelMixers(Part):
    """``left`` and ``right`` are mixers that both read the mixer's input ``h``; their tensors are named with the
    prefixes ``left.`` and ``right.``. Their outputs (float32, the width of the stream) become one update:

    * ``combine="scaled"``: ``left_scale * left(h) + right_scale * right(h)``;
    * ``combine="normed_mean"``: ``(norm(left(h)) * left_out + norm(right(h)) * right_out) / 2``, each output divided by
      its root mean square over the width (``eps`` inside the root) and multiplied by its weight vector (tensors
      ``left_out``, ``right_out``).

    At most one of the two may ask for paged keys and values (``cache_request``); fixed-size states of both are states
    of the layer call under their own names.

    Where both mixers end in a product and can stop in front of it (``inner(h, ctx, binding, out, factor)`` and
    ``last_weight``), the scaled form is one product: each writes its last activations, times its scale, into its
    columns of one matrix, which meets the two weights side by side. Otherwise, and for the normed mean, one kernel
    forms the update from the two float32 outputs.
    """

    def __init__(self, left: Part, right: Part, width: int, combine: str = "scaled", left_scale: float = 1.0,
                 right_scale: float = 1.0, eps: float = 1e-6) -> None:
        if combine not in ("scaled", "normed_mean"):
            raise ValueError("combine is 'scaled' or 'normed_mean'")
        if left.cache_request() is not None and right.cache_request() is not None:
            raise ValueError("only one of two parallel mixers may use paged keys and values")
        self.left, self.right, self.width, self.combine = left, right, int(width), combine
        self.left_scale, self.right_scale, self.eps = float(left_scale), float(right_scale), float(eps)
        self.left_out = self.right_out = None
        self._joined: torch.Tensor | None = None

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def sub_parts(self) -> dict[str, Part]:
        return {"left": self.left, "right": self.right}

    def param_specs(self) -> dict[str, ParamSpec]:
        if self.combine != "normed_mean":
            return {}
        return {"left_out": ParamSpec((self.width,), "vector"), "right_out": ParamSpec((self.width,), "vector")}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        for name, tensor in params.items():
            setattr(self, name, tensor.contiguous())

    def cache_request(self):
        return self.left.cache_request() or self.right.cache_request()

    def state_requests(self):
        requests = {}
        for child in (self.left, self.right):
            for name, request in child.state_requests().items():
                if name in requests:
                    raise ValueError(f"two parallel mixers ask for a state named {name!r}")
                requests[name] = request
        return requests

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        for child in (self.left, self.right):
            if type(child).plan_step is not Part.plan_step:
                child.plan_step(ctx, binding)

    def _joins(self) -> bool:
        return self.combine == "scaled" and all(hasattr(m, "inner") and hasattr(m, "last_weight") for m in (self.left, self.right))

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        if self._joins():
            if self._joined is None:
                # (the parts have their tensors by the first step)
                self._joined = torch.cat([self.left.last_weight, self.right.last_weight], dim=1).contiguous()
            n_left = self.left.last_weight.shape[1]
            both = arena.empty((x.shape[0], self._joined.shape[1]), ctx.dtype, x.device)
            self.left.inner(x, ctx, binding, out=both[:, :n_left], factor=self.left_scale)
            self.right.inner(x, ctx, binding, out=both[:, n_left:], factor=self.right_scale)
            # the float32 result of the last product goes to a norm
            return gemm.linear(both, self._joined, out_dtype=torch.float32, few_rows_f32=True)
        a = self.left.forward(x, ctx, binding)
        b = self.right.forward(x, ctx, binding)
        if self.combine == "scaled":
            return mixer_ops.combine_pair(a, b, self.left_scale, self.right_scale)
        return mixer_ops.combine_pair(a, b, 0.5, 0.5, norm_weights=(self.left_out, self.right_out), eps=self.eps)
