"""Feed-forward parts."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import ParamSpec, Part, StepContext

__all__ = ["BiasedDense", "Dense", "GatedDense", "GatedRoutedExperts", "RoutedExperts", "SwiGLU"]


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """Dense gated feed-forward: ``(silu(x @ gate) * (x @ up)) @ down`` without biases, the
    argument of the sigmoid's exponential clipped to ``[-clip, clip]``
    (reference: src/paged_kv_serving/engine/model.py:49-51, 256-259).

    Weights are re-laid at load as ``[out, in]``. Gate and up become one matrix so that a single
    product feeds the ``silu * up`` step: in bfloat16 their rows are interleaved in blocks of
    128 (padded with zero rows to a multiple of 128), which lets the tensor-core kernel apply the
    step in its epilogue; in float32 they are simply stacked.
    """

    graph_safe = True
    BLOCK = 128

    def __init__(self, width: int, inner: int, clip: float = 60.0) -> None:
        self.width = int(width)
        self.inner = int(inner)
        self.clip = float(clip)
        self.gate_up: torch.Tensor | None = None    # [2 * inner (padded), width]
        self.down_proj: torch.Tensor | None = None  # [width, inner]
        self.interleave = 0

    def param_specs(self) -> dict[str, ParamSpec]:
        return {
            "gate_proj": ParamSpec((self.width, self.inner)),
            "up_proj": ParamSpec((self.width, self.inner)),
            "down_proj": ParamSpec((self.inner, self.width)),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        gate, up = params["gate_proj"].t(), params["up_proj"].t()          # [inner, width]
        if gate.dtype == torch.bfloat16:
            block = self.BLOCK
            blocks = -(-self.inner // block)
            fused = torch.zeros((blocks, 2, block, self.width), dtype=gate.dtype, device=gate.device)
            flat = fused.view(blocks, 2, block * self.width)
            padded = torch.zeros((2, blocks * block, self.width), dtype=gate.dtype, device=gate.device)
            padded[0, :self.inner] = gate
            padded[1, :self.inner] = up
            flat[:, 0] = padded[0].view(blocks, block * self.width)
            flat[:, 1] = padded[1].view(blocks, block * self.width)
            self.gate_up = fused.view(2 * blocks * block, self.width)
            self.interleave = block
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
            self.interleave = 0
        self.down_proj = params["down_proj"].t().contiguous()

    fuses_last_linear = True
    accepts_pending_norm = True

    def forward(self, x: torch.Tensor, ctx: StepContext, finish=None) -> torch.Tensor:
        gated = gemm.linear_silu_mul(x, self.gate_up, self.inner, self.interleave, self.clip, chain=True)
        if finish is not None:
            return finish(gated, self.down_proj)
        return gemm.linear(gated, self.down_proj, chain=True)


@register_part("feed_forward", "biased_dense")
class BiasedDense(Part):
    """``W_down act(W_up x + b_up) + b_down`` with the exact (erf) GELU by default; weights
    ``[out, in]``. The bias of the last product is not added here: ``forward`` returns the
    product and ``last_bias`` names the vector, so that whoever adds the update to the stream adds
    the bias in the same pass (``forward(..., add_bias=True)`` adds it at once)."""

    graph_safe = True
    accepts_pending_norm = True

    def __init__(self, width: int, inner: int, activation: str = "gelu_erf") -> None:
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"up": ParamSpec((self.inner, self.width)), "up_b": ParamSpec((self.inner,), "vector"),
                "down": ParamSpec((self.width, self.inner)), "down_b": ParamSpec((self.width,), "vector")}

    @property
    def last_bias(self) -> torch.Tensor:
        return self.down_b

    def forward(self, x: torch.Tensor, ctx: StepContext, add_bias: bool = True) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        inner = mixer_ops.bias_act(gemm.linear(x, self.up), self.up_b, self.activation)
        out = gemm.linear(inner, self.down)
        return mixer_ops.bias_act(out, self.down_b, "none") if add_bias else out


@register_part("feed_forward", "dense")
class Dense(Part):
    """``W_down act(W_up x)`` without biases and without a gate (``act`` the square of relu unless
    given); weights ``[out, in]``. The result is float32: what a norm on the sublayer's output reads."""

    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "relu_squared") -> None:
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"up": ParamSpec((self.inner, self.width)), "down": ParamSpec((self.width, self.inner))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.up, self.down = params["up"].contiguous(), params["down"].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        inner = mixer_ops.bias_act(gemm.linear(x, self.up, chain=True), None, self.activation)
        return gemm.linear(inner, self.down, out_dtype=torch.float32, few_rows_f32=True, chain=True)


@register_part("feed_forward", "gated_dense")
class GatedDense(Part):
    """``W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down`` (``act`` the tanh form of GELU unless given;
    ``bias=False``: no biases); weights ``[out, in]``. Gate and up are one product; the result is float32: what a norm
    or the residual sum reads."""

    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "gelu_tanh", bias: bool = True) -> None:
        self.width, self.inner, self.activation, self.bias = int(width), int(inner), activation, bool(bias)
        self.up_at = -(-self.inner // 8) * 8           # the up columns start on a 16-byte boundary
        self.gate_b = self.up_b = self.down_b = None

    def param_specs(self) -> dict[str, ParamSpec]:
        specs = {"gate": ParamSpec((self.inner, self.width)), "up": ParamSpec((self.inner, self.width)),
                 "down": ParamSpec((self.width, self.inner))}
        if self.bias:
            specs.update({"gate_b": ParamSpec((self.inner,), "vector", init=(0.0, 0.1)),
                          "up_b": ParamSpec((self.inner,), "vector", init=(0.0, 0.1)),
                          "down_b": ParamSpec((self.width,), "vector", init=(0.0, 0.1))})
        return specs

    def load(self, params: dict[str, torch.Tensor]) -> None:
        gate = params["gate"]
        gate_up = torch.zeros((2 * self.up_at, self.width), dtype=gate.dtype, device=gate.device)
        gate_up[:self.inner] = gate
        gate_up[self.up_at:self.up_at + self.inner] = params["up"]
        self.gate_up = gate_up                                              # [gate (padded) | up (padded), width]
        self.down = params["down"].contiguous()
        for name in ("gate_b", "up_b", "down_b"):
            setattr(self, name, params[name].contiguous() if name in params else None)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        gate_up = gemm.linear(x, self.gate_up, chain=True)
        inner = mixer_ops.gated_bias_act(gate_up, self.up_at, self.inner, self.gate_b, self.up_b, self.activation)
        out = gemm.linear(inner, self.down, out_dtype=torch.float32, few_rows_f32=True, chain=True)
        return mixer_ops.bias_act(out, self.down_b, "none") if self.down_b is not None else out


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of small feed-forward experts ``W_down act(W_up x)`` without biases (``act`` the
    square of relu by default). Router logits ``W_router x`` and their softmax over all experts
    are float32; a token uses its ``top`` best experts, weighted by their softmax scores as they
    are (not renormalised). An optional shared expert of the same form runs for every token and
    is added times ``sigmoid(W_sg x)``, one number per token.

    Kernels: one product over the stacked up-projections of all experts (and the shared one), the
    activation scaled by the router's weight of each column's expert (zero for an expert the
    token does not use), one product over the stacked down-projections. Every expert's weights
    are read once per step whatever the routing, and nothing of the step depends on values read
    back to the host, so decode steps can be captured.
    """

    graph_safe = True

    def __init__(self, width: int, experts: int, top: int, inner: int, shared_inner: int = 0,
                 activation: str = "relu_squared") -> None:
        if not 1 <= top <= experts:
            raise ValueError("top must be between 1 and the number of experts")
        self.width, self.experts, self.top, self.inner = int(width), int(experts), int(top), int(inner)
        self.shared_inner, self.activation = int(shared_inner), activation
        self.columns = self.experts * self.inner + self.shared_inner

    def param_specs(self) -> dict[str, ParamSpec]:
        specs = {"router": ParamSpec((self.experts, self.width))}
        for e in range(self.experts):
            specs[f"e{e}_up"] = ParamSpec((self.inner, self.width))
            specs[f"e{e}_down"] = ParamSpec((self.width, self.inner))
        if self.shared_inner:
            specs["shared_up"] = ParamSpec((self.shared_inner, self.width))
            specs["shared_down"] = ParamSpec((self.width, self.shared_inner))
            specs["shared_sg"] = ParamSpec((1, self.width))
        return specs

    def load(self, params: dict[str, torch.Tensor]) -> None:
        ups = [params[f"e{e}_up"] for e in range(self.experts)]
        downs = [params[f"e{e}_down"] for e in range(self.experts)]
        route = [params["router"]]
        if self.shared_inner:
            ups.append(params["shared_up"])
            downs.append(params["shared_down"])
            route.append(params["shared_sg"])
        padded = -(-self.columns // 8) * 8             # rows of a product's result start on 16-byte boundaries
        up = torch.zeros((padded, self.width), dtype=ups[0].dtype, device=ups[0].device)
        up[:self.columns] = torch.cat(ups, dim=0)
        self.up = up                                                       # [columns (padded), width]
        self.down = torch.cat(downs, dim=1).contiguous()                   # [width, columns]
        rows = -(-(self.experts + 1) // 8) * 8
        router = torch.zeros((rows, self.width), dtype=ups[0].dtype, device=ups[0].device)
        router[:self.experts + len(route) - 1] = torch.cat(route, dim=0)
        self.router = router                                               # router rows, then the shared gate's row

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        logits = gemm.linear(x, self.router, out_dtype=torch.float32)      # [tokens, experts + 1 (padded)]
        weights = mixer_ops.route_top(logits, self.experts, self.top)
        up = gemm.linear(x, self.up)
        gate = logits[:, self.experts] if self.shared_inner else None
        inner = mixer_ops.expert_act(up, weights, gate, self.experts, self.inner, self.shared_inner, self.activation)
        return gemm.linear(inner, self.down)


@register_part("feed_forward", "gated_routed_experts")
class GatedRoutedExperts(Part):
    """A mixture of small gated experts ``W_down (act(W_gate x) * (W_up x))`` without biases
    (``act`` SiLU by default). Router logits ``W_router x + b_router`` are float32; a token uses
    the ``top`` experts with the largest logits, weighted by the softmax over those logits only
    (``renormalise``; otherwise by their softmax scores over all experts). An optional shared
    expert of the same form runs for every token and is added with weight 1.

    Kernels, as in ``RoutedExperts``: one product over the stacked gate and up projections of all
    experts (and the shared one), the gated activation scaled by the router's weight of each
    column's expert (exact zeros for an expert the token does not use), one product over the
    stacked down-projections, whose result stays float32. Nothing depends on values read back to
    the host, so decode steps can be captured.

    ``scoring="sigmoid"`` is another router: an expert's score is ``sigmoid(logit)`` (no bias on the logits); experts
    are chosen by score plus the tensor ``correction [experts]`` and weighted by the score alone; the experts form
    ``groups`` equal groups of neighbours, a group's score is the sum of its two largest choice scores, and only experts
    of the ``keep_groups`` best groups can be chosen; the chosen scores are divided by their sum (plus ``1e-20``) and
    multiplied by ``weight_scale``.
    """

    graph_safe = True

    def __init__(self, width: int, experts: int, top: int, inner: int, shared_inner: int = 0, activation: str = "silu",
                 router_bias: bool = True, renormalise: bool = True, scoring: str = "softmax", groups: int = 1,
                 keep_groups: int = 1, weight_scale: float = 1.0) -> None:
        if not 1 <= top <= experts:
            raise ValueError("top must be between 1 and the number of experts")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError("scoring is 'softmax' or 'sigmoid'")
        if scoring == "sigmoid":
            if groups < 1 or groups > 64 or experts % groups or not 1 <= keep_groups <= groups:
                raise ValueError("the experts form up to 64 equal groups, of which at least one and at most all are kept")
            if top > experts // groups * keep_groups:
                raise ValueError("more experts to choose than the kept groups hold")
            router_bias = False
        self.scoring, self.groups, self.keep_groups, self.weight_scale = scoring, int(groups), int(keep_groups), float(weight_scale)
        self.width, self.experts, self.top, self.inner = int(width), int(experts), int(top), int(inner)
        self.shared_inner, self.activation = int(shared_inner), activation
        self.router_bias, self.renormalise = bool(router_bias), bool(renormalise)
        self.columns = self.experts * self.inner + self.shared_inner
        self.up_at = -(-self.columns // 8) * 8           # the up columns start on a 16-byte boundary

    def param_specs(self) -> dict[str, ParamSpec]:
        specs = {"router": ParamSpec((self.experts, self.width))}
        if self.router_bias:
            specs["router_b"] = ParamSpec((self.experts,), "vector", init=(0.0, 0.1))
        if self.scoring == "sigmoid":
            specs["correction"] = ParamSpec((self.experts,), "vector", init=(0.0, 0.1))
        names = [f"e{e}" for e in range(self.experts)]
        for name in names:
            specs[f"{name}_gate"] = ParamSpec((self.inner, self.width))
            specs[f"{name}_up"] = ParamSpec((self.inner, self.width))
            specs[f"{name}_down"] = ParamSpec((self.width, self.inner))
        if self.shared_inner:
            specs["shared_gate"] = ParamSpec((self.shared_inner, self.width))
            specs["shared_up"] = ParamSpec((self.shared_inner, self.width))
            specs["shared_down"] = ParamSpec((self.width, self.shared_inner))
        return specs

    def load(self, params: dict[str, torch.Tensor]) -> None:
        names = [f"e{e}" for e in range(self.experts)] + (["shared"] if self.shared_inner else [])
        first = params["router"]
        gate_up = torch.zeros((2 * self.up_at, self.width), dtype=first.dtype, device=first.device)
        gate_up[:self.columns] = torch.cat([params[f"{n}_gate"] for n in names], dim=0)
        gate_up[self.up_at:self.up_at + self.columns] = torch.cat([params[f"{n}_up"] for n in names], dim=0)
        self.gate_up = gate_up                                              # [gates (padded) | ups (padded), width]
        self.down = torch.cat([params[f"{n}_down"] for n in names], dim=1).contiguous()     # [width, columns]
        rows = -(-self.experts // 8) * 8
        router = torch.zeros((rows, self.width), dtype=first.dtype, device=first.device)
        router[:self.experts] = first
        self.router = router
        self.router_b = params["router_b"].contiguous() if self.router_bias else None
        self.correction = params["correction"].contiguous() if self.scoring == "sigmoid" else None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from paged_kv_serving_b200.ops import mixer_ops

        logits = gemm.linear(x, self.router, out_dtype=torch.float32, few_rows_f32=True, chain=True)       # [tokens, experts (padded)]
        if self.scoring == "sigmoid":
            weights = mixer_ops.route_scored(logits, self.experts, self.top, self.correction, self.groups, self.keep_groups,
                                             self.weight_scale)
        else:
            weights = mixer_ops.route_top(logits, self.experts, self.top, bias=self.router_b, renormalise=self.renormalise)
        gate_up = gemm.linear(x, self.gate_up, chain=True)
        inner = mixer_ops.expert_gated_act(gate_up, self.up_at, weights, self.experts, self.inner, self.shared_inner,
                                           self.activation)
        # the float32 result of the last product goes to a norm
        return gemm.linear(inner, self.down, out_dtype=torch.float32, few_rows_f32=True, chain=True)
