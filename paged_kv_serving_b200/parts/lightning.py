"""Linear attention with a fixed decay per head."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext

__all__ = ["LightningAttention"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part("mixer", "lightning_attention")
class LightningAttention(Part):
    """Lightning attention: per head a matrix state ``S [dim, vdim]`` (float32, starting at zero)
    that decays by a fixed factor per token and takes the outer product of key and value:

    ``q = silu(W_q h)``, ``k = silu(W_k h)`` (``heads x dim``), ``v = silu(W_v h)`` (``heads x vdim``);
    ``S_t = decay[a] S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` for head ``a``, no other scale. The
    heads' outputs together are divided by their root mean square (``eps`` inside the root),
    multiplied by ``norm`` and by ``sigmoid(W_g h)``, and go through ``W_o``.

    ``decays`` are the factors, one per head, constants of the model. The state is a further state
    of the layer call (``state_requests``); the recurrence runs token by token in the kernel
    whether the tokens arrive as a prompt, in portions or one at a time, so the result does not
    depend on the cut. The four input projections are one product whose float32 result the
    kernel reads; the activation, the recurrence, the norm and the gate are float32 arithmetic.
    """

    graph_safe = True
    STATE = "lightning_S"

    def __init__(self, width: int, heads: int, dim: int, vdim: int, decays, eps: float) -> None:
        decays = [float(d) for d in decays]
        if len(decays) != heads:
            raise ValueError("one decay per head")
        if dim > 256:
            raise ValueError("the lightning attention kernel takes a key size of up to 256")
        self.width, self.heads, self.dim, self.vdim, self.eps = int(width), int(heads), int(dim), int(vdim), float(eps)
        self.decays = decays
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        self.offsets = {"q": 0, "k": qk, "v": 2 * qk, "g": 2 * qk + vg}
        self.fused_rows = _round_up(2 * qk + 2 * vg, 8)
        self.decay: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        return {"q": ParamSpec((qk, self.width)), "k": ParamSpec((qk, self.width)), "v": ParamSpec((vg, self.width)),
                "g": ParamSpec((vg, self.width)), "o": ParamSpec((self.width, vg)), "norm": ParamSpec((vg,), "vector")}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        q = params["q"]
        fused = torch.zeros((self.fused_rows, self.width), dtype=q.dtype, device=q.device)
        for name in ("q", "k", "v", "g"):
            fused[self.offsets[name]:self.offsets[name] + params[name].shape[0]] = params[name]
        self.fused = fused
        self.o = params["o"].contiguous()
        self.norm = params["norm"].contiguous()
        self.decay = torch.tensor(self.decays, dtype=torch.float64).to(torch.float32).to(q.device)

    def state_requests(self) -> dict[str, StateRequest]:
        return {self.STATE: StateRequest((self.heads, self.vdim, self.dim))}

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        proj = gemm.linear(x, self.fused, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        out = mixer_ops.lightning(proj, self.offsets, self.decay, self.norm, self.eps, ctx.states[binding.extra[self.STATE]],
                                  ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS), self.heads, self.dim, self.vdim, ctx.dtype)
        # the float32 result of the last product goes to a norm
        return gemm.linear(out, self.o, out_dtype=torch.float32, few_rows_f32=True, chain=True)
