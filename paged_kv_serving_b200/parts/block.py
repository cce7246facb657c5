"""Arrangement of the parts of one layer."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import Block, CacheBinding, Normed, Part, StepContext

__all__ = ["ConvSideBlock", "PostNormBlock", "PreNormBlock", "SandwichBlock"]


@register_part("block", "prenorm_residual")
class PreNormBlock(Block):
    """Pre-norm residual arrangement: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
    (reference: src/paged_kv_serving/engine/model.py:283-287, src/paged_kv_serving/engine/runner.py:213-214);
    a layer may have no feed-forward (and then no second norm).

    The hand-over between blocks (pending updates, ``Normed``) is the one ``parts.base.Block``
    describes: a block receives the previous block's output as a pending update and returns its
    own feed-forward output as the next one, or the stream already normalised for the next block.
    """

    @property
    def graph_safe(self) -> bool:
        return all(child.graph_safe for child in self.sub_parts().values())


    def __init__(self, mixer_norm: Part, mixer: Part, ff_norm: Part | None = None, feed_forward: Part | None = None) -> None:
        if (ff_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its norm go together")
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ff_norm = ff_norm
        self.feed_forward = feed_forward

    def sub_parts(self) -> dict[str, Part]:
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ff_norm": self.ff_norm, "feed_forward": self.feed_forward}
        return {name: part for name, part in parts.items() if part is not None}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_requests(self):
        return self.mixer.state_requests()

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        # only the children that plan anything (this runs for every layer of every step)
        planners = self.__dict__.get("_planners")
        if planners is None:
            planners = self._planners = [child for child in self.sub_parts().values()
                                         if type(child).plan_step is not Part.plan_step]
        for child in planners:
            child.plan_step(ctx, binding)

    @property
    def first_norm(self) -> Part:
        """The norm this block applies to the stream it is given (with the pending update)."""
        return self.mixer_norm

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: StepContext,
                binding: CacheBinding | None, next_norm: Part | None = None) -> "torch.Tensor | Normed":
        """One layer call. ``pending`` is what the block before handed on: its residual update not
        yet added (a tensor, or None at the start), or a ``Normed`` when it already added it and
        applied this block's first norm. ``next_norm`` is the first norm of the block that runs
        next; where the feed-forward can carry the residual add and that norm in the tail of its
        last product, this block hands on a ``Normed``, else its own pending update.
        """
        if isinstance(pending, Normed) and pending.norm is self.mixer_norm:
            normed = pending.values if self.mixer.accepts_pending_norm else gemm.as_tensor(pending.values)
        else:
            if isinstance(pending, Normed):
                raise ValueError("the stream was normalised for another block than the one that runs next")
            normed = self.mixer_norm.add_norm(hidden, pending, ctx.dtype)
        if self.feed_forward is None:
            # a layer without a feed-forward: the mixer's update is what is pending behind the block
            return self.mixer.forward(gemm.as_tensor(normed), ctx, binding)
        follow = getattr(self.ff_norm, "add_norm_of_linear", None)
        if self.mixer.fuses_last_linear and follow is not None:
            chain = self.mixer.chains_last_linear
            normed = self.mixer.forward(normed, ctx, binding,
                                        finish=lambda x, w: follow(hidden, x, w, ctx.dtype, chain=chain))
        else:
            normed = self.ff_norm.add_norm(hidden, self.mixer.forward(normed, ctx, binding), ctx.dtype)
        if not self.feed_forward.accepts_pending_norm:
            normed = gemm.as_tensor(normed)
        follow = getattr(next_norm, "add_norm_of_linear", None)
        if self.feed_forward.fuses_last_linear and follow is not None:
            chain = self.feed_forward.chains_last_linear
            values = self.feed_forward.forward(
                normed, ctx, finish=lambda x, w: follow(hidden, x, w, ctx.dtype, chain=chain))
            return Normed(values, next_norm)
        return self.feed_forward.forward(normed, ctx)


@register_part("block", "prenorm_conv_side")
class ConvSideBlock(Block):
    """Pre-norm residual arrangement with two optional additions:

    ``h = norm1(x)``; with ``input_conv``, ``h <- h + conv(h)`` (a short causal convolution whose
    tail is state of the layer call); ``x += mixer(h)``; with a feed-forward, ``x += ff(norm2(x))``;
    with ``side``, ``x += side(x, tokens)`` (a per-token input computed from the stream itself).

    The mixer is called as ``forward(h, ctx, binding)``, the feed-forward as ``forward(h, ctx)``.
    Updates travel as pending tensors as ``Block`` describes; this block applies no norm for its
    successor and accepts none from its predecessor (``first_norm`` is ``None``).
    """

    def __init__(self, mixer_norm: Part, mixer: Part, ff_norm: Part | None = None, feed_forward: Part | None = None,
                 input_conv: Part | None = None, side: Part | None = None) -> None:
        if (ff_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its norm go together")
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward
        self.input_conv, self.side = input_conv, side

    @property
    def graph_safe(self) -> bool:
        return all(child.graph_safe for child in self.sub_parts().values())

    def sub_parts(self) -> dict[str, Part]:
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ff_norm": self.ff_norm,
                 "feed_forward": self.feed_forward, "input_conv": self.input_conv, "side": self.side}
        return {name: part for name, part in parts.items() if part is not None}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_requests(self):
        requests = {}
        for child in self.sub_parts().values():
            for name, request in child.state_requests().items():
                if name in requests:
                    raise ValueError(f"two parts of one block ask for a state named {name!r}")
                requests[name] = request
        return requests

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        for child in self.sub_parts().values():
            if type(child).plan_step is not Part.plan_step:
                child.plan_step(ctx, binding)

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: StepContext,
                binding: CacheBinding | None, next_norm: Part | None = None) -> torch.Tensor:
        if isinstance(pending, Normed):
            raise ValueError("this block normalises the stream itself")
        h = self.mixer_norm.add_norm(hidden, pending, ctx.dtype)
        if self.input_conv is not None:
            h = self.input_conv.forward(h, ctx, binding)
        bias = None
        follow = getattr(self.ff_norm, "add_norm_of_linear", None) if self.feed_forward is not None else None
        if follow is not None and self.mixer.fuses_last_linear:
            # the mixer's last product carries the residual add, and for the few rows of a decode step
            # leaves the norm to the product that reads it
            chain = self.mixer.chains_last_linear
            h = self.mixer.forward(h, ctx, binding, finish=lambda x, w: follow(hidden, x, w, ctx.dtype, chain=chain))
            if not self.feed_forward.accepts_pending_norm:
                h = gemm.as_tensor(h)
            update = None
        else:
            update = self.mixer.forward(h, ctx, binding)
            if self.feed_forward is not None:
                h = self.ff_norm.add_norm(hidden, update, ctx.dtype)
        if self.feed_forward is not None:
            if self.side is not None and hasattr(self.feed_forward, "last_bias"):
                # the side input adds the update to the stream anyway: the last bias rides along
                update, bias = self.feed_forward.forward(h, ctx, add_bias=False), self.feed_forward.last_bias
            else:
                update = self.feed_forward.forward(h, ctx)
        if self.side is not None:
            update = self.side.forward(hidden, update, ctx, bias)
        return update


@register_part("block", "postnorm_residual")
class PostNormBlock(Block):
    """Residual arrangement with the norm on each sublayer's output: ``x += norm1(mixer(x))``, then
    (with a feed-forward) ``x += norm2(feed_forward(x))``. The sublayers read the stream itself, in
    the compute type.

    The hand-over between blocks uses ``Block``'s interface with an ``IdentityNorm`` as this
    block's first norm: what a block before may leave behind is the stream in the compute type.
    This block adds its updates itself (the kernel that normalises an update also adds it and
    writes the copy of the stream the next sublayer reads), so it hands on a ``Normed`` for a
    block of its own kind that follows and ``None`` (nothing pending) otherwise.
    """

    def __init__(self, mixer_norm: Part, mixer: Part, ff_norm: Part | None = None, feed_forward: Part | None = None) -> None:
        from paged_kv_serving_b200.parts.norms import IdentityNorm

        if (ff_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its norm go together")
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward
        self.reads = IdentityNorm()

    @property
    def graph_safe(self) -> bool:
        return all(child.graph_safe for child in self.sub_parts().values())

    def sub_parts(self) -> dict[str, Part]:
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ff_norm": self.ff_norm, "feed_forward": self.feed_forward}
        return {name: part for name, part in parts.items() if part is not None}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_requests(self):
        return self.mixer.state_requests()

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        for child in self.sub_parts().values():
            if type(child).plan_step is not Part.plan_step:
                child.plan_step(ctx, binding)

    @property
    def first_norm(self) -> Part:
        return self.reads

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: StepContext,
                binding: CacheBinding | None, next_norm: Part | None = None) -> "Normed | None":
        from paged_kv_serving_b200.parts.norms import IdentityNorm

        if isinstance(pending, Normed):
            if pending.norm is not self.reads:
                raise ValueError("the stream was normalised for another block than the one that runs next")
            x = gemm.as_tensor(pending.values)
        else:
            x = self.reads.add_norm(hidden, pending, ctx.dtype)
        copy_type = None if ctx.dtype == torch.float32 else ctx.dtype      # in float32 the stream is its own copy
        wants_copy = isinstance(next_norm, IdentityNorm)
        update = self.mixer.forward(x, ctx, binding)
        last = self.feed_forward is None
        x = self.mixer_norm.norm_add(hidden, update, copy_type if (not last or wants_copy) else None)
        if not last:
            update = self.feed_forward.forward(hidden if x is None else x, ctx)
            x = self.ff_norm.norm_add(hidden, update, copy_type if wants_copy else None)
        if wants_copy:
            return Normed(hidden if x is None else x, next_norm)
        return None


@register_part("block", "sandwich_layernorm")
class SandwichBlock(Block):
    """Residual arrangement with a layer norm in front of and behind each sublayer and a factor on
    every update: ``x += m * norm1b(mixer(shift(norm1(x))))``, then (with a feed-forward) ``x += m *
    norm2b(feed_forward(norm2(x)))``. ``input_shift`` (a ``TokenShift``, optional) blends the
    mixer's input with that of the token before it.

    The norms are ``LayerNorm`` parts; the norm behind a sublayer, the residual add and the norm
    in front of the next sublayer are one kernel (``ops.mixer_ops.layer_norm_step``), also across
    the border to a following block of this kind: its ``first_norm`` is applied in the tail of
    this block's last step and handed on as a ``Normed`` (in that norm's ``rows_dtype``: float32
    when the block shifts its input, since the shift reads float32 rows). The block adds its updates itself, so nothing is ever pending
    behind it.
    """

    def __init__(self, mixer_norm: Part, mixer: Part, mixer_out_norm: Part, ff_norm: Part | None = None,
                 feed_forward: Part | None = None, ff_out_norm: Part | None = None, residual_mult: float = 1.0,
                 input_shift: Part | None = None) -> None:
        if (ff_norm is None) != (feed_forward is None) or (ff_out_norm is None) != (feed_forward is None):
            raise ValueError("a feed-forward and its two norms go together")
        self.mixer_norm, self.mixer, self.mixer_out_norm = mixer_norm, mixer, mixer_out_norm
        self.ff_norm, self.feed_forward, self.ff_out_norm = ff_norm, feed_forward, ff_out_norm
        self.residual_mult, self.input_shift = float(residual_mult), input_shift
        if input_shift is not None and mixer_norm.rows_dtype != torch.float32:
            raise ValueError("the norm in front of a shifted mixer input hands out float32 rows")

    @property
    def graph_safe(self) -> bool:
        return all(child.graph_safe for child in self.sub_parts().values())

    def sub_parts(self) -> dict[str, Part]:
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_out_norm": self.mixer_out_norm,
                 "ff_norm": self.ff_norm, "feed_forward": self.feed_forward, "ff_out_norm": self.ff_out_norm,
                 "input_shift": self.input_shift}
        return {name: part for name, part in parts.items() if part is not None}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_requests(self):
        requests = {}
        for child in self.sub_parts().values():
            for name, request in child.state_requests().items():
                if name in requests:
                    raise ValueError(f"two parts of one block ask for a state named {name!r}")
                requests[name] = request
        return requests

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        for child in self.sub_parts().values():
            if type(child).plan_step is not Part.plan_step:
                child.plan_step(ctx, binding)

    @property
    def first_norm(self) -> Part:
        return self.mixer_norm

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: StepContext,
                binding: CacheBinding | None, next_norm: Part | None = None) -> "Normed | None":
        from paged_kv_serving_b200.ops import mixer_ops
        from paged_kv_serving_b200.parts.norms import LayerNorm

        eps, mult = self.mixer_norm.eps, self.residual_mult
        first_type = self.mixer_norm.rows_dtype or ctx.dtype
        if isinstance(pending, Normed):
            if pending.norm is not self.mixer_norm or pending.values.dtype != first_type:
                raise ValueError("the stream was normalised for another block than the one that runs next")
            h = pending.values
        else:
            if pending is not None:
                mixer_ops.residual_add(hidden, pending)
            h = mixer_ops.layer_norm_step(hidden, pre=self.mixer_norm.pair, out_dtype=first_type, eps=eps)
        if self.input_shift is not None:
            h = self.input_shift.forward(h, ctx, binding)
        update = self.mixer.forward(h, ctx, binding)
        carried = next_norm if isinstance(next_norm, LayerNorm) else None
        carried_type = (carried.rows_dtype or ctx.dtype) if carried is not None else None
        if self.feed_forward is not None:
            h = mixer_ops.layer_norm_step(hidden, update, self.mixer_out_norm.pair, mult, pre=self.ff_norm.pair,
                                          out_dtype=ctx.dtype, eps=eps)
            update = self.feed_forward.forward(h, ctx)
            last = self.ff_out_norm
        else:
            last = self.mixer_out_norm
        values = mixer_ops.layer_norm_step(hidden, update, last.pair, mult, pre=carried.pair if carried is not None else None,
                                           out_dtype=carried_type, eps=eps)
        return Normed(values, carried) if carried is not None else None
