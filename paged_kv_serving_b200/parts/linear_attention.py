"""Linear attention with a matrix state per head: a decay computed per token and key coordinate (gated linear
attention) or a fixed one per head (retention)."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import arena, gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, ParamSpec, Part, StateRequest, StepContext
from paged_kv_serving_b200.parts.position import ScaledRotaryFrequencies

__all__ = ["GatedLinearAttention", "Retention"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class _MatrixStateAttention(Part):
    """What the two mixers share: per head a state ``S [dim, vdim]`` (float32, zero at the start of a sequence) with
    ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t``; each head's ``o`` is divided by its root mean square
    over ``vdim`` (``eps`` inside the root), the heads are concatenated, multiplied by ``silu(W_g h)`` and projected by
    ``W_o``. The input projections are one product whose float32 result the kernel reads; decays, rotation, state,
    outputs, norm and gate are float32 arithmetic. The state is a further state of the layer call
    (``state_requests``); the recurrence is the same sequence of operations per token whether the tokens arrive as a
    prompt, in portions or one at a time.

    ``forward`` returns the float32 result of ``W_o``; ``inner`` stops in front of ``W_o`` (times ``factor``) and may
    write into a column range of a wider matrix, for a caller that joins several last products into one."""

    graph_safe = True
    STATE = "linear_attention_S"

    def __init__(self, width: int, heads: int, dim: int, vdim: int, eps: float) -> None:
        if min(width, heads, dim, vdim) < 1:
            raise ValueError("every size of the mixer must be >= 1")
        if dim > 256:
            raise ValueError("the linear attention kernel takes a key size of up to 256")
        self.width, self.heads, self.dim, self.vdim, self.eps = int(width), int(heads), int(dim), int(vdim), float(eps)
        self.out_cols = self.heads * self.vdim

    def _fuse(self, params: dict[str, torch.Tensor], names: tuple[str, ...]) -> torch.Tensor:
        """The named projections as one matrix; ``self.offsets`` says where each one's rows begin."""
        first = params[names[0]]
        self.offsets, at = {}, 0
        for name in names:
            self.offsets[name], at = at, at + _round_up(params[name].shape[0], 8)
        fused = torch.zeros((at, self.width), dtype=first.dtype, device=first.device)
        for name in names:
            fused[self.offsets[name]:self.offsets[name] + params[name].shape[0]] = params[name]
        return fused

    def state_requests(self) -> dict[str, StateRequest]:
        return {self.STATE: StateRequest((self.heads, self.vdim, self.dim))}

    def inner(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, out: torch.Tensor | None = None,
              factor: float = 1.0) -> torch.Tensor:
        raise NotImplementedError

    @property
    def last_weight(self) -> torch.Tensor:
        return self.o

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        # the float32 result of the last product goes to a norm
        return gemm.linear(self.inner(x, ctx, binding), self.o, out_dtype=torch.float32, few_rows_f32=True, chain=True)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(_MatrixStateAttention):
    """Gated linear attention (Yang, Wang, Shen, Panda and Kim, "Gated Linear Attention Transformers with
    Hardware-Efficient Training"): ``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (``heads x dim``), ``v = W_v h`` (``heads x
    vdim``) and a decay per token and key coordinate, ``a = sigmoid(W_a2 (W_a1 h) + b_a2) ^ (1 / tau)`` (a projection
    through ``rank`` numbers). The heads' normalised outputs are multiplied by ``norm [vdim]``, the same for every
    head."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, rank: int, tau: float, eps: float) -> None:
        super().__init__(width, heads, dim, vdim, eps)
        if rank < 1 or not tau > 0.0:
            raise ValueError("the decay's projection needs a rank >= 1 and tau > 0")
        self.rank, self.tau = int(rank), float(tau)
        self.rank_padded = _round_up(self.rank, 8)

    def param_specs(self) -> dict[str, ParamSpec]:
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        return {"q": ParamSpec((qk, self.width)), "k": ParamSpec((qk, self.width)), "v": ParamSpec((vg, self.width)),
                "g": ParamSpec((vg, self.width)), "o": ParamSpec((self.width, vg)), "norm": ParamSpec((self.vdim,), "vector"),
                "a1": ParamSpec((self.rank, self.width)), "a2": ParamSpec((qk, self.rank)),
                "a2_b": ParamSpec((qk,), "vector", init=(3.0, 1.0))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.fused = self._fuse(params, ("q", "k", "v", "g", "a1"))
        a2 = torch.zeros((self.heads * self.dim, self.rank_padded), dtype=params["a2"].dtype, device=params["a2"].device)
        a2[:, :self.rank] = params["a2"]
        self.a2 = a2
        self.a2_b = params["a2_b"].contiguous()
        self.norm = params["norm"].contiguous()
        self.o = params["o"].contiguous()

    def inner(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, out: torch.Tensor | None = None,
              factor: float = 1.0) -> torch.Tensor:
        proj = gemm.linear(x, self.fused, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        low = proj[:, self.offsets["a1"]:self.offsets["a1"] + self.rank_padded]
        if ctx.dtype == torch.float32:
            decay_pre = gemm.matmul(low, self.a2.t())
        else:
            low_c = arena.empty((proj.shape[0], self.rank_padded), ctx.dtype, proj.device)
            low_c.copy_(low)
            decay_pre = gemm.linear(low_c, self.a2, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        return mixer_ops.linear_attention(
            proj, self.offsets, ctx.states[binding.extra[self.STATE]], ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS),
            self.heads, self.dim, self.vdim, ctx.dtype, decay_pre=decay_pre, decay_bias=self.a2_b, inv_tau=1.0 / self.tau,
            q_scale=self.dim ** -0.5, norm_weight=self.norm, eps=self.eps, out_factor=factor, out=out)


@register_part("mixer", "retention")
class Retention(_MatrixStateAttention):
    """Retention (Sun, Dong, Huang, Ma, Xia, Xue, Wang and Wei, "Retentive Network: A Successor to Transformer for
    Large Language Models"): linear attention with a fixed decay per head and neither softmax nor denominator. ``q =
    W_q h``, ``k = W_k h`` (``heads x dim``), ``v = W_v h`` (``heads x vdim``) without biases; ``rotary`` turns the first
    coordinates of every query and key head by the token's position (coordinate ``i`` with ``i + rot / 2``); the keys
    are then multiplied by ``dim^(-1/2)``; ``S_t = decay[a] S_(t-1) + k_t v_t^T`` for head ``a``. The heads' normalised
    outputs carry no weight."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, decays, eps: float,
                 rotary: ScaledRotaryFrequencies | None = None) -> None:
        super().__init__(width, heads, dim, vdim, eps)
        decays = [float(d) for d in decays]
        if len(decays) != heads:
            raise ValueError("one decay per head")
        if rotary is not None and rotary.dims > dim:
            raise ValueError("more rotated coordinates than a head has")
        if rotary is not None and rotary.amplitude != 1.0:
            raise ValueError("the retention kernel rotates without a factor on cos and sin")
        self.decays, self.rotary = decays, rotary
        self.decay: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        return {"q": ParamSpec((qk, self.width)), "k": ParamSpec((qk, self.width)), "v": ParamSpec((vg, self.width)),
                "g": ParamSpec((vg, self.width)), "o": ParamSpec((self.width, vg))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.fused = self._fuse(params, ("q", "k", "v", "g"))
        self.o = params["o"].contiguous()
        self.decay = torch.tensor(self.decays, dtype=torch.float64).to(torch.float32).to(self.o.device)

    def inner(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, out: torch.Tensor | None = None,
              factor: float = 1.0) -> torch.Tensor:
        proj = gemm.linear(x, self.fused, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        rotary = self.rotary if self.rotary is not None and self.rotary.dims else None
        return mixer_ops.linear_attention(
            proj, self.offsets, ctx.states[binding.extra[self.STATE]], ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.STATE_SLOTS),
            self.heads, self.dim, self.vdim, ctx.dtype, head_decay=self.decay, k_scale=self.dim ** -0.5,
            rot_dims=rotary.dims if rotary else 0, freq=rotary.device_frequencies(ctx.device) if rotary else None,
            positions=ctx.ints(ctx.POSITIONS) if rotary else None, eps=self.eps, out_factor=factor, out=out)
