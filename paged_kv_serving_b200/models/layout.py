"""What an architecture module hands to the framework: parts, layer order, tensor names."""

from __future__ import annotations

from dataclasses import dataclass, field, replace

from paged_kv_serving_b200.parts.base import ParamSpec, Part

__all__ = ["LayerCall", "ModelLayout", "collect_param_specs", "layout_for"]


@dataclass(frozen=True, slots=True)
class LayerCall:
    """One entry of the run order. ``layer`` indexes ``ModelLayout.blocks``; the same layer may
    be named by several calls. ``cache`` is the number of the cache entry the call's mixer uses:
    by default a fresh one per call; a call that names an earlier call's entry with
    ``write=False`` reads that layer's keys and values without writing its own."""

    layer: int
    cache: int | None = None
    write: bool = True
    #: ``(name, cache entry number)`` of the call's further states (``Part.state_requests``);
    #: ``resolved_order`` fills it in, a fresh entry per call and name.
    extra: tuple = ()
    #: The model's input (the embedding part's output for the step's tokens) is added to the
    #: stream once more right before this call: the start of a repeated pass over a span of layers.
    add_input: bool = False
    #: The number of the pass over a repeated span of layers that starts right before this call: the
    #: layout's ``pass_input`` part gives the stream its new value from the stream and the model's input
    #: (``None``: no pass starts here).
    enter_pass: int | None = None


@dataclass(slots=True)
class ModelLayout:
    """A model as data.

    ``names`` maps each tensor name of the model folder to ``(part, local name)``; the embedding
    table and an untied head are named separately because the framework itself applies them.
    """

    width: int
    vocab_size: int
    max_positions: int
    blocks: list[Part]
    order: list[LayerCall]
    final_norm: Part
    names: dict[str, tuple[Part, str]]
    embedding_name: str = "token_embedding"
    head_name: str | None = None          # None: the head is the embedding table (tied)
    notes: dict[str, str] = field(default_factory=dict)
    #: The part that turns the step's token ids into the residual stream (``forward(ctx)``) and
    #: the part that turns the final norm's rows into float32 logits (``forward(normed, ctx)``).
    #: Left ``None`` they are a plain table lookup named ``embedding_name`` and a linear head
    #: named ``head_name`` (tied to the table when that is ``None``). An architecture with
    #: another kind of embedding or head passes its own parts and names their tensors in ``names``.
    embedding: Part | None = None
    head: Part | None = None
    #: Tensors a model folder may hold although the layout has no use for them (they are not loaded).
    optional_names: set = field(default_factory=set)
    #: The part that runs in front of every layer call with ``enter_pass`` (``forward(hidden, pending,
    #: model_input, pass number)`` gives the stream its new value in place); its tensors are named in ``names``.
    pass_input: Part | None = None

    def __post_init__(self) -> None:
        from paged_kv_serving_b200.parts.io import LinearHead, TokenEmbedding

        if self.embedding is None:
            self.embedding = TokenEmbedding(self.vocab_size, self.width)
            self.names[self.embedding_name] = (self.embedding, "table")
        if self.head is None:
            tied = self.embedding if self.head_name is None and isinstance(self.embedding, TokenEmbedding) else None
            if self.head_name is None and tied is None:
                raise ValueError("a head tied to the embedding needs the plain embedding part, or a head of its own")
            self.head = LinearHead(self.vocab_size, self.width, tied=tied)
            if self.head_name is not None:
                self.names[self.head_name] = (self.head, "weight")

        if self.pass_input is None and any(call.enter_pass is not None for call in self.order):
            raise ValueError("a layer call starts a pass but the layout has no part for it")

    def tensor_specs(self) -> dict[str, ParamSpec]:
        return {name: part.param_specs()[local] for name, (part, local) in self.names.items()}

    def parameter_count(self) -> int:
        """Number of parameters in the tensors of a model folder (a tied head counts once)."""
        total = 0
        for spec in self.tensor_specs().values():
            count = 1
            for size in spec.shape:
                count *= int(size)
            total += count
        return total

    def cache_entries(self) -> list[tuple[int, object]]:
        """``(entry number, request)`` of every distinct cache entry of the run order."""
        seen: dict[int, object] = {}
        next_free = 0
        for call in self.resolved_order():
            request = self.blocks[call.layer].cache_request()
            if request is None or call.cache is None:
                continue
            if call.cache in seen:
                if seen[call.cache] != request:
                    raise ValueError(f"layer calls sharing cache entry {call.cache} ask for different storage")
            else:
                seen[call.cache] = request
            next_free = max(next_free, call.cache + 1)
        for call in self.resolved_order():
            requests = self.blocks[call.layer].state_requests()
            for name, number in call.extra:
                seen[number] = requests[name]
        return sorted(seen.items())

    def resolved_order(self) -> list[LayerCall]:
        """The run order with a cache entry number on every call whose mixer wants a cache."""
        explicit = [c.cache for c in self.order if c.cache is not None]
        next_free = max(explicit) + 1 if explicit else 0
        out = []
        for call in self.order:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"layer call names layer {call.layer}, the model has {len(self.blocks)}")
            if call.cache is None and self.blocks[call.layer].cache_request() is not None:
                call = replace(call, cache=next_free)
                next_free += 1
            out.append(call)
        # the further states of every call come after all primary entries, one entry per call and name
        for i, call in enumerate(out):
            names = sorted(self.blocks[call.layer].state_requests())
            if names and not call.extra:
                out[i] = replace(call, extra=tuple((name, next_free + k) for k, name in enumerate(names)))
                next_free += len(names)
        return out


def collect_param_specs(prefix: str, part: Part, into: dict[str, tuple[Part, str]]) -> None:
    """Register ``prefix + local`` for every tensor of ``part`` and of its children
    (children's names are prefixed with ``child.``)."""
    for local in part.param_specs():
        into[prefix + local] = (part, local)
    for child_name, child in part.sub_parts().items():
        collect_param_specs(f"{prefix}{child_name}.", child, into)


def layout_for(config, tensors: dict | None = None) -> ModelLayout:
    """The layout of the architecture ``config`` names. An architecture some of whose sizes only a tensor's shape gives
    (its class says ``sizes_from_tensors``) also gets the shapes of ``tensors`` (name -> tensor) where there are any."""
    from paged_kv_serving_b200.config import registry

    builder = registry.architecture(config.architecture)
    if tensors is not None and getattr(builder, "sizes_from_tensors", False):
        return builder.layout(config, tensor_shapes={name: tuple(t.shape) for name, t in tensors.items()})
    return builder.layout(config)
