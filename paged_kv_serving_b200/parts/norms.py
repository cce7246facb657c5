"""Normalisation parts."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.parts.base import ParamSpec, Part

__all__ = ["IdentityNorm", "LayerNorm", "OffsetRMSNorm", "RMSNorm", "ScalarRMSNorm"]


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """``y = (x / sqrt(mean(x^2) + eps)) * weight`` in float32
    (reference: src/paged_kv_serving/engine/model.py:43-46), fused with the residual add in
    front of it: the stream ``hidden`` (float32) first takes the pending ``delta``."""

    graph_safe = True


    def __init__(self, width: int, eps: float) -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "vector")}

    def add_norm(self, hidden: torch.Tensor, delta: torch.Tensor | None, out_dtype: torch.dtype,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        """``hidden += delta`` in place, then the normalised rows (all, or only ``rows``; with
        ``rows`` the stream itself is not updated)."""
        return ops.add_rmsnorm(hidden, delta, self.weight, self.eps, out_dtype, rows)

    def add_norm_of_linear(self, hidden: torch.Tensor, x: torch.Tensor, w_nk: torch.Tensor,
                           out_dtype: torch.dtype, chain: bool = False) -> torch.Tensor:
        """``add_norm(hidden, x @ w_nk^T)`` for a producer whose last step is that product: the
        product's kernel carries the residual add, and the norm is left to the product that reads
        the result, where the kernels can do that. ``chain`` as in ``ops.gemm.linear``."""
        return gemm.linear_add_norm(x, w_nk, hidden, self.weight, self.eps, out_dtype, chain=chain)

    def norm_add(self, hidden: torch.Tensor, update: torch.Tensor, out_dtype: torch.dtype | None = None
                 ) -> torch.Tensor | None:
        """The norm on a sublayer's output: ``hidden += norm(update)`` in place, and, with
        ``out_dtype``, the updated stream in that type (for a sublayer that reads the stream itself)."""
        from paged_kv_serving_b200.ops import mixer_ops

        return mixer_ops.norm_residual(hidden, update, self.weight, self.eps, out_dtype)


@register_part("norm", "scalar_rmsnorm")
class ScalarRMSNorm(RMSNorm):
    """RMS norm whose weight is a single number for all coordinates:
    ``y = x / sqrt(mean(x^2) + eps) * g``. The stored tensor has no axes; at load it is spread
    over the width, so that the kernels of ``RMSNorm`` (and its fusions) serve it unchanged."""

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((), "vector")}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"].reshape(1).expand(self.width).contiguous()


@register_part("norm", "offset_rmsnorm")
class OffsetRMSNorm(RMSNorm):
    """RMS norm whose stored weight is centred on zero: ``y = x / sqrt(mean(x^2) + eps) * (offset +
    w)`` with ``offset`` 1 unless given. The sum is formed once at load (in float32), after which
    the kernels of ``RMSNorm`` serve it unchanged."""

    def __init__(self, width: int, eps: float, offset: float = 1.0) -> None:
        super().__init__(width, eps)
        self.offset = float(offset)

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "vector", init=(1.0 - self.offset, 0.0))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.weight = (params["weight"].to(torch.float32) + self.offset).contiguous()


@register_part("norm", "identity")
class IdentityNorm(Part):
    """No norm at all, in the shape of one: ``add_norm`` adds the pending update to the stream and
    hands out the stream itself in the asked type. It is the ``first_norm`` of a block whose
    sublayers read the stream as it is, so that the block before can leave that copy behind."""

    graph_safe = True

    def add_norm(self, hidden: torch.Tensor, delta: torch.Tensor | None, out_dtype: torch.dtype,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        if rows is not None:
            raise ValueError("the identity norm hands out whole streams only")
        if delta is None and out_dtype == torch.float32:
            return hidden
        out = mixer_ops.residual_add(hidden, delta, None, None if out_dtype == torch.float32 else out_dtype)
        return hidden if out is None else out


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """``y = (x - mean) / sqrt(variance + eps) * weight + bias`` in float32, the variance being the
    mean of the squared deviations from the mean. ``add_norm`` is the interface every norm has
    (the pending update is added to the stream first); a block that wraps its sublayers in such
    norms calls ``ops.mixer_ops.layer_norm_step`` with the weights of two of them at once.
    ``rows_dtype`` is the type of the rows the norm hands out when a block applies it for its
    owner (``None``: the compute type; float32 for a norm whose rows an element-wise step reads)."""

    graph_safe = True

    def __init__(self, width: int, eps: float, rows_dtype: torch.dtype | None = None) -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.rows_dtype = rows_dtype
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "vector"), "bias": ParamSpec((self.width,), "vector", init=(0.0, 0.02))}

    @property
    def pair(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.weight, self.bias

    def add_norm(self, hidden: torch.Tensor, delta: torch.Tensor | None, out_dtype: torch.dtype,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        if delta is not None:
            mixer_ops.residual_add(hidden, delta)
        return mixer_ops.layer_norm_step(hidden, pre=self.pair, out_dtype=out_dtype, rows=rows, eps=self.eps)
