"""Attention over a sliding window that also keeps the first tokens, with capped scores."""

from __future__ import annotations

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import arena, gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, PagedKVRequest, ParamSpec, Part, StepContext
from paged_kv_serving_b200.parts.position import ScaledRotaryFrequencies

__all__ = ["SinkWindowAttention"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part("mixer", "sink_window_attention")
class SinkWindowAttention(Part):
    """Causal grouped-query softmax attention with these ingredients, each a parameter:

    * ``H`` query heads and ``G`` key/value heads (query head ``h`` reads key/value head ``h // (H
      // G)``), keys and queries of size ``dim``, values of size ``vdim``; ``q = W_q x``, ``k = W_k
      x``, ``v = W_v x`` without biases, ``W_o`` on the concatenated heads;
    * ``rotary``: a ``ScaledRotaryFrequencies`` that turns the first coordinates of every query and
      key head by the token's position (``None``: no rotation);
    * ``unit_norm``: after the rotation every query and key head is divided by its root mean square
      (``eps`` inside the root); with ``norm_weights`` the result is multiplied by the tensor
      ``q_norm`` (queries) or ``k_norm`` (keys), ``[dim]`` each and the same for every head;
    * ``score = q . k * scale``, with ``head_temperature`` times the head's entry of the tensor ``temp``
      ``[H]``, then, with ``softcap`` ``c > 0``, ``c * tanh(score / c)``; with ``distance_bias`` the score of
      query position ``i`` and key position ``j`` then loses ``r1[h] * ln(1 + r2[h] * (i - j))`` (tensors
      ``r1``, ``r2`` ``[H]``);
    * ``window`` and ``keep_first``: position ``i`` sees ``j <= i`` when ``i - j < window`` or ``j <
      keep_first`` (``window=None``: all earlier positions); kept tokens keep their own positions;
    * ``bias``: the three projections have biases (tensors ``q_b``, ``k_b``, ``v_b``), added before anything else;
    * ``joint_norm`` (with ``unit_norm``): in place of the norm per head, all query columns of a token are divided by
      their joint root mean square and multiplied by ``q_norm [H dim]``, the key columns by theirs and ``k_norm [G
      dim]``, before the rotation;
    * ``pairing``: the rotation pairs coordinate ``i`` with ``i + rot / 2`` ("halves") or ``2i`` with ``2i + 1``
      ("interleaved"; the rows of ``W_q`` and ``W_k``, their biases and norm weights are reordered at load, evens in
      front of odds, which turns one into the other without changing any score);
    * ``head_gate``: head ``h``'s output is multiplied by ``sigmoid(W_g x)_h`` (tensor ``g [H, width]``) before ``W_o``;
    * ``value_share``: ``"source"`` leaves this layer's values of the step's tokens in the step's
      scratch under ``share_key``; ``"blend"`` replaces ``v`` by ``(1 - lambda) v + lambda v_source``
      with ``lambda`` the tensor ``vmix`` and ``v_source`` what the source layer left for the same
      tokens; the blended values are what is cached. ``None``: plain values.

    Keys are cached rotated and normalised, in pages of ``[G, page_size, dim]`` and ``[G,
    page_size, vdim]``. Angles, norms, scores, softmax and the blend are float32 arithmetic.

    Kernels: one for rotation, unit norm, blend and cache write (``ops.mixer_ops.qkv_prepare``);
    for the attention itself, in bfloat16 with keys and values of one size of 64 or 128, pages
    of a multiple of 8 keys and neither temperature nor distance bias, the tensor-core kernels of ``PagedAttention`` (tcgen05 for runs of
    queries, the TMA-fed split-key kernel for entries of a few rows), which take the kept first
    tokens as further tiles in front of the window's and cap the scores in their softmax; in
    bfloat16 with other head sizes that are multiples of 16 (keys and values may differ) the
    ``mma.sync`` kernel ``ops.mixer_ops.attention_sink_mma``; for every other size and for float32
    the general kernel ``ops.mixer_ops.attention_sink``. With a temperature or a distance bias (and
    no cap) and heads of 64 or 128, a step that holds a long entry gives its long entries to the tcgen05
    kernel, which applies both in its softmax, and the short ones to the ``mma.sync`` kernel.
    """

    graph_safe = True
    #: Set to False to keep every step on the general kernel (tests compare the two).
    USE_TENSOR_CORES = True
    #: With a temperature or a distance bias: entries of at least this many tokens go to the tcgen05 kernel
    #: (blocks of 128 queries of one head), shorter ones to the ``mma.sync`` kernel (64 rows of a head group).
    SHAPED_TCGEN05_MIN_TOKENS = 64

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 rotary: ScaledRotaryFrequencies | None = None, unit_norm: bool = True, eps: float = 1e-6,
                 softcap: float = 0.0, window: int | None = None, keep_first: int = 0, value_share: str | None = None,
                 share_key: str = "sink_attention/shared_values", norm_weights: bool = False,
                 head_temperature: bool = False, distance_bias: bool = False, bias: bool = False, joint_norm: bool = False,
                 pairing: str = "halves", head_gate: bool = False) -> None:
        if n_heads < 1 or n_kv_heads < 1 or n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if window is not None and window < 1:
            raise ValueError("window must be >= 1 or None")
        if keep_first < 0 or softcap < 0:
            raise ValueError("keep_first and softcap must be >= 0")
        if value_share not in (None, "source", "blend"):
            raise ValueError("value_share is None, 'source' or 'blend'")
        if rotary is not None and rotary.dims > dim:
            raise ValueError("more rotated coordinates than a head has")
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.dim, self.vdim = int(dim), int(vdim)
        self.scale, self.softcap, self.eps = float(scale), float(softcap), float(eps)
        self.rotary, self.unit_norm = rotary, bool(unit_norm)
        self.window, self.keep_first = window, int(keep_first)
        self.value_share, self.share_key = value_share, share_key
        if norm_weights and not unit_norm:
            raise ValueError("norm weights belong to the unit norm of queries and keys")
        self.norm_weights, self.head_temperature, self.distance_bias = bool(norm_weights), bool(head_temperature), bool(distance_bias)
        if joint_norm and not (unit_norm and norm_weights):
            raise ValueError("the joint norm of queries and keys is a unit norm with weights")
        if pairing not in ("halves", "interleaved"):
            raise ValueError("pairing is 'halves' or 'interleaved'")
        self.bias, self.joint_norm, self.pairing, self.head_gate = bool(bias), bool(joint_norm), pairing, bool(head_gate)
        self.q_norm = self.k_norm = self.temp = self.r1 = self.r2 = self.qkv_bias = None
        self.q_cols = self.n_heads * self.dim
        self.kv_cols = self.n_kv_heads * (self.dim + self.vdim)
        self.gate_at = self.q_cols + self.kv_cols          # the gates' columns in the fused projection
        self.fused_rows = _round_up(self.gate_at + (self.n_heads if self.head_gate else 0), 8)
        self._fast_ok: dict = {}

    @property
    def group_size(self) -> int:
        return self.n_heads // self.n_kv_heads

    def param_specs(self) -> dict[str, ParamSpec]:
        specs = {
            "q": ParamSpec((self.q_cols, self.width)), "k": ParamSpec((self.n_kv_heads * self.dim, self.width)),
            "v": ParamSpec((self.n_kv_heads * self.vdim, self.width)), "o": ParamSpec((self.width, self.n_heads * self.vdim)),
        }
        if self.value_share is not None:
            specs["vmix"] = ParamSpec((), "vector", init=(0.5, 0.0))
        if self.norm_weights:
            specs["q_norm"] = ParamSpec((self.q_cols if self.joint_norm else self.dim,), "vector")
            specs["k_norm"] = ParamSpec((self.n_kv_heads * self.dim if self.joint_norm else self.dim,), "vector")
        if self.bias:
            specs["q_b"] = ParamSpec((self.q_cols,), "vector", init=(0.0, 0.1))
            specs["k_b"] = ParamSpec((self.n_kv_heads * self.dim,), "vector", init=(0.0, 0.1))
            specs["v_b"] = ParamSpec((self.n_kv_heads * self.vdim,), "vector", init=(0.0, 0.1))
        if self.head_gate:
            specs["g"] = ParamSpec((self.n_heads, self.width))
        if self.head_temperature:
            specs["temp"] = ParamSpec((self.n_heads,), "vector", init=(1.0, 0.2))
        if self.distance_bias:
            specs["r1"] = ParamSpec((self.n_heads,), "vector", init=(0.5, 0.2))
            specs["r2"] = ParamSpec((self.n_heads,), "vector", init=(0.5, 0.2))
        return specs

    def _halves_order(self, heads: int) -> torch.Tensor | None:
        """For an interleaved rotation: the order of the ``heads * dim`` rows (or elements) that puts, inside every
        head, the even rotated coordinates in front of the odd ones; ``None`` when nothing moves."""
        rot = self.rotary.dims if self.rotary is not None else 0
        if self.pairing != "interleaved" or not rot:
            return None
        inside = list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, self.dim))
        return torch.tensor([h * self.dim + d for h in range(heads) for d in inside], dtype=torch.long)

    def load(self, params: dict[str, torch.Tensor]) -> None:
        q = params["q"]
        params = dict(params)
        for heads, names in ((self.n_heads, ("q", "q_b", "q_norm")), (self.n_kv_heads, ("k", "k_b", "k_norm"))):
            order = self._halves_order(heads)
            if order is None:
                continue
            for name in names:
                if name not in params:
                    continue
                t = params[name]
                if name.endswith("_norm") and not self.joint_norm:
                    t = t[order[:self.dim].to(t.device)]            # one weight per coordinate of a head
                else:
                    t = t[order.to(t.device)]
                params[name] = t
        fused = torch.zeros((self.fused_rows, self.width), dtype=q.dtype, device=q.device)
        at = 0
        for name in ("q", "k", "v") + (("g",) if self.head_gate else ()):
            rows = params[name].shape[0]
            fused[at:at + rows] = params[name]
            at += rows
        self.qkv = fused                                   # [H dim + G dim + G vdim (+ H gates) (padded), width]
        self.o = params["o"].contiguous()
        self.blend = params["vmix"].reshape(1).contiguous() if "vmix" in params else None
        for name in ("q_norm", "k_norm", "temp", "r1", "r2"):
            setattr(self, name, params[name].contiguous() if name in params else None)
        if self.bias:
            self.qkv_bias = torch.cat([params["q_b"], params["k_b"], params["v_b"]]).to(torch.float32).contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.n_kv_heads, self.dim, self.window, value_dim=self.vdim,
                              keep_first=self.keep_first if self.window is not None else 0)

    # --- per step ------------------------------------------------------------------------

    def _work_names(self) -> tuple[str, str]:
        return (f"sink_attention/work_seq/g{self.group_size}", f"sink_attention/work_row0/g{self.group_size}")

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        if self._fast(ctx, ctx.groups[binding.group].page_size):
            self._plan_fast(ctx, ctx.groups[binding.group].page_size)
            return
        if self._shaped_split(ctx, ctx.groups[binding.group].page_size):
            self._plan_shaped(ctx, ctx.groups[binding.group].page_size)
            return
        if self._mma(ctx):
            self._plan_mma(ctx)
            return
        seq_name, row_name = self._work_names()
        if seq_name in ctx.arena:
            return
        rows_per_block = mixer_ops.attention_sink_rows_per_block()
        rows = np.asarray(ctx.seq_lens, dtype=np.int64) * self.group_size
        blocks = (rows + rows_per_block - 1) // rows_per_block
        work_seq = np.repeat(np.arange(len(rows), dtype=np.int64), blocks)
        starts = np.cumsum(blocks) - blocks
        work_row0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * rows_per_block
        ctx.arena.add(seq_name, work_seq)
        ctx.arena.add(row_name, work_row0)

    def _fast(self, ctx: StepContext, page_size: int) -> bool:
        """Whether the tensor-core kernels serve this mixer in this step."""
        if not self.USE_TENSOR_CORES or ctx.dtype != torch.bfloat16 or self.dim != self.vdim:
            return False
        if self.head_temperature or self.distance_bias:      # those kernels know neither
            return False
        key = page_size
        if key not in self._fast_ok:
            self._fast_ok[key] = (ops.attention_tcgen05_supports(self.dim, page_size, self.fused_rows)
                                  and ops.attention_decode_tma_supports(self.dim, page_size, self.fused_rows))
        return self._fast_ok[key]

    def _shaped_split(self, ctx: StepContext, page_size: int) -> bool:
        """Whether this step goes to two kernels: the tcgen05 kernel (which knows the head temperature and
        the distance bias, not the cap) for entries of at least ``SHAPED_TCGEN05_MIN_TOKENS`` tokens and the
        ``mma.sync`` kernel for the others. Only for mixers with a temperature or a bias, and only in steps
        that hold such an entry; decode steps stay with the ``mma.sync`` kernel and its shares."""
        if not (self.head_temperature or self.distance_bias) or self.softcap or self.dim != self.vdim or not self._mma(ctx):
            return False
        if max(ctx.seq_lens) < self.SHAPED_TCGEN05_MIN_TOKENS:
            return False
        key = ("shaped", page_size)
        if key not in self._fast_ok:
            self._fast_ok[key] = ops.attention_tcgen05_supports(self.dim, page_size, self.fused_rows)
        return self._fast_ok[key]

    def _shaped_key(self, page_size: int) -> str:
        return (f"sink_attention/shaped/h{self.n_heads}k{self.n_kv_heads}d{self.dim}w{self.window or 0}s{self.keep_first}"
                f"p{page_size}")

    def _plan_shaped(self, ctx: StepContext, page_size: int) -> None:
        """Work lists of a step that two kernels share: blocks of 128 queries of the long entries, heaviest
        first, and blocks of (token, head in group) rows of the short ones."""
        key = self._shaped_key(page_size)
        if key in ctx.scratch:
            return
        lens = np.asarray(ctx.seq_lens, dtype=np.int64)
        first = np.asarray(ctx.first_positions, dtype=np.int64)
        long_entries = np.nonzero(lens >= self.SHAPED_TCGEN05_MIN_TOKENS)[0]
        short_entries = np.nonzero(lens < self.SHAPED_TCGEN05_MIN_TOKENS)[0]

        def blocks_of(entries, rows_of_entry, block_rows):
            blocks = (rows_of_entry + block_rows - 1) // block_rows
            seq = np.repeat(entries, blocks)
            starts = np.cumsum(blocks) - blocks
            return seq, (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * block_rows

        long_seq, long_q0 = blocks_of(long_entries, lens[long_entries], ops.attention_tcgen05_rows())
        cost = first[long_seq] + long_q0
        if self.window:
            cost = np.minimum(cost, self.window + self.keep_first)
        order = np.argsort(-cost, kind="stable")
        short_seq, short_q0 = blocks_of(short_entries, lens[short_entries] * self.group_size, mixer_ops.attention_sink_mma_rows())
        names = {k: f"{key}/{k}" for k in ("long_seq", "long_q0", "short_seq", "short_q0")}
        ctx.arena.add(names["long_seq"], long_seq[order])
        ctx.arena.add(names["long_q0"], long_q0[order])
        ctx.arena.add(names["short_seq"], short_seq if len(short_seq) else [0])
        ctx.arena.add(names["short_q0"], short_q0 if len(short_q0) else [0])
        ctx.scratch[key] = {"names": names, "n_short": int(len(short_seq))}

    def _attend_shaped(self, qkv: torch.Tensor, ctx: StepContext, group, k_pool, v_pool, bias) -> torch.Tensor:
        plan = ctx.scratch[self._shaped_key(group.page_size)]
        names = plan["names"]
        out = arena.empty((qkv.shape[0], self.n_heads * self.vdim), qkv.dtype, qkv.device)
        table, starts, first = ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS)
        ops.attention_prefill_tcgen05(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["long_seq"]),
                                      ctx.ints(names["long_q0"]), self.n_heads, self.n_kv_heads, self.dim, group.page_size,
                                      self.window or 0, self.scale, ctx.status, keep_first=self.keep_first,
                                      head_scale=self.temp, distance_bias=bias)
        if plan["n_short"]:
            mixer_ops.attention_sink_mma(
                qkv, k_pool, v_pool, table, starts, first, ctx.ints(names["short_seq"]), ctx.ints(names["short_q0"]),
                self.n_heads, self.n_kv_heads, self.dim, self.vdim, group.page_size, self.window or 0, self.keep_first,
                self.scale, self.softcap, ctx.status, head_scale=self.temp, distance_bias=bias, out=out)
        return out

    def _mma(self, ctx: StepContext) -> bool:
        """Whether the ``mma.sync`` kernel serves this mixer in this step (when ``_fast`` does not)."""
        return (self.USE_TENSOR_CORES and ctx.dtype == torch.bfloat16
                and mixer_ops.attention_sink_mma_supports(self.dim, self.vdim, self.fused_rows))

    def _mma_names(self) -> tuple[str, str]:
        return (f"sink_attention/mma/work_seq/g{self.group_size}", f"sink_attention/mma/work_row0/g{self.group_size}")

    def _mma_splits(self, ctx: StepContext) -> int:
        """Shares of the key range per block of the ``mma.sync`` kernel: one, unless the step holds
        only entries of a few tokens over long contexts (decode steps), whose few blocks would
        each walk their tiles in a row; then as many as still run in one round of blocks, at most 8
        and at most one per tile (a captured graph plans from its fixed context length)."""
        key = f"sink_attention/mma/splits/k{self.n_kv_heads}w{self.window or 0}s{self.keep_first}"
        if key not in ctx.scratch:
            from paged_kv_serving_b200.parts.attention import _sm_count

            splits = 1
            if max(ctx.seq_lens) <= 4:
                longest = max(f + n for f, n in zip(ctx.first_positions, ctx.seq_lens))
                if ctx.planning_context_len is not None:
                    longest = ctx.planning_context_len
                if self.window:
                    longest = min(longest, self.window + self.keep_first + 64)
                tiles = max(1, -(-longest // 64))
                blocks = len(ctx.seq_lens) * self.n_kv_heads
                splits = int(max(1, min(8, tiles, (4 * _sm_count(ctx.device)) // max(blocks, 1))))      # about four blocks fit an SM
            ctx.scratch[key] = splits
        return ctx.scratch[key]

    def _plan_mma(self, ctx: StepContext) -> None:
        seq_name, q0_name = self._mma_names()
        self._mma_splits(ctx)
        if seq_name in ctx.arena:
            return
        rows = mixer_ops.attention_sink_mma_rows()
        lens = np.asarray(ctx.seq_lens, dtype=np.int64) * self.group_size     # rows of an (entry, key/value head)
        first = np.asarray(ctx.first_positions, dtype=np.int64)
        blocks = (lens + rows - 1) // rows
        work_seq = np.repeat(np.arange(len(lens), dtype=np.int64), blocks)
        starts = np.cumsum(blocks) - blocks
        work_q0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * rows
        order = np.argsort(-(first[work_seq] + work_q0 // self.group_size), kind="stable")      # the longest key ranges first
        ctx.arena.add(seq_name, work_seq[order])
        ctx.arena.add(q0_name, work_q0[order])

    def _fast_key(self, page_size: int) -> str:
        return (f"sink_attention/fast/h{self.n_heads}k{self.n_kv_heads}d{self.dim}w{self.window or 0}s{self.keep_first}"
                f"p{page_size}")

    def _plan_fast(self, ctx: StepContext, page_size: int) -> None:
        """Work lists of the tensor-core kernels: entries of at most 16 rows per key/value head go to
        the split-key decode kernel, longer ones are cut into blocks of 128 queries, heaviest first."""
        key = self._fast_key(page_size)
        if key in ctx.scratch:
            return
        from paged_kv_serving_b200.parts.attention import _sm_count

        block_rows = ops.attention_tcgen05_rows()
        lens = np.asarray(ctx.seq_lens, dtype=np.int64)
        first = np.asarray(ctx.first_positions, dtype=np.int64)
        small = lens * self.group_size <= 16
        decode_entries = np.nonzero(small)[0]
        large = np.nonzero(~small)[0]
        blocks = (lens[large] + block_rows - 1) // block_rows
        work_seq = np.repeat(large, blocks)
        starts = np.cumsum(blocks) - blocks
        work_q0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * block_rows
        cost = first[work_seq] + work_q0
        if self.window:
            cost = np.minimum(cost, self.window + self.keep_first)
        order = np.argsort(-cost, kind="stable")
        num_splits = 1
        if len(decode_entries):
            longest = int((first[decode_entries] + lens[decode_entries]).max())
            if ctx.planning_context_len is not None:
                longest = ctx.planning_context_len
            if self.window:
                longest = min(longest, self.window + self.keep_first + 64)
            tiles = max(1, -(-longest // 64))
            resident = 2 * _sm_count(ctx.device)
            num_splits = int(max(1, min(tiles, 8, resident // (len(decode_entries) * self.n_kv_heads))))
            if num_splits > 4:
                rows = int(lens[decode_entries].max()) * self.group_size
                pushed = ops.attention_decode_tma_pushed_splits(self.dim, rows)
                if 4 <= pushed < num_splits:
                    num_splits = pushed
        names = {k: f"{key}/{k}" for k in ("prefill_seq", "prefill_q0", "decode_seq")}
        ctx.arena.add(names["prefill_seq"], work_seq[order] if len(order) else [0])
        ctx.arena.add(names["prefill_q0"], work_q0[order] if len(order) else [0])
        ctx.arena.add(names["decode_seq"], decode_entries if len(decode_entries) else [0])
        ctx.scratch[key] = {"names": names, "n_prefill": int(len(order)), "n_decode": int(len(decode_entries)),
                            "max_small_tokens": int(lens[decode_entries].max()) if len(decode_entries) else 0,
                            "num_splits": num_splits}

    def _attend_fast(self, qkv: torch.Tensor, ctx: StepContext, group, k_pool, v_pool) -> torch.Tensor:
        plan = ctx.scratch[self._fast_key(group.page_size)]
        names = plan["names"]
        out = arena.empty((qkv.shape[0], self.n_heads * self.vdim), qkv.dtype, qkv.device)
        table, starts, first = ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS)
        if plan["n_prefill"]:
            ops.attention_prefill_tcgen05(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["prefill_seq"]),
                                          ctx.ints(names["prefill_q0"]), self.n_heads, self.n_kv_heads, self.dim,
                                          group.page_size, self.window or 0, self.scale, ctx.status,
                                          keep_first=self.keep_first, softcap=self.softcap)
        if plan["n_decode"]:
            ops.attention_decode_tma(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["decode_seq"]),
                                     plan["max_small_tokens"], self.n_heads, self.n_kv_heads, self.dim, group.page_size,
                                     self.window or 0, self.scale, plan["num_splits"], ctx.status, False,
                                     keep_first=self.keep_first, softcap=self.softcap)
        return out

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        attended, chain = self._inner(x, ctx, binding, None, 1.0)
        # the float32 result of the last product goes to a norm
        return gemm.linear(attended, self.o, out_dtype=torch.float32, few_rows_f32=True, chain=chain)

    @property
    def last_weight(self) -> torch.Tensor:
        return self.o

    def inner(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, out: torch.Tensor | None = None,
              factor: float = 1.0) -> torch.Tensor:
        """Everything in front of ``W_o``: the heads' (gated) outputs times ``factor``, ``[tokens, H vdim]`` in the compute
        type, written to ``out`` where one is given (a view whose rows may have a stride)."""
        return self._inner(x, ctx, binding, out, factor)[0]

    def _inner(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, out: torch.Tensor | None,
               factor: float) -> tuple[torch.Tensor, bool]:
        group = ctx.groups[binding.group]
        k_pool, v_pool = group.k_pool[binding.index], group.v_pool[binding.index]
        slots = ctx.ints(group.slots_name) if binding.write else None
        qkv = gemm.linear(x, self.qkv, chain=True)
        other = None
        if self.value_share == "blend":
            other = ctx.scratch.get(self.share_key)
            if other is None:
                raise RuntimeError("a layer blends its values with those of a layer that has not run in this step")
        shared = None
        if self.value_share == "source":
            # the values of the step's tokens as this layer caches them, for the layers that blend with
            # them: a copy that lives as long as the step
            shared = arena.empty_for_step((qkv.shape[0], self.n_kv_heads * self.vdim), qkv.dtype, qkv.device)
            ctx.scratch[self.share_key] = shared
        rotary = self.rotary if self.rotary is not None and self.rotary.dims else None
        mixer_ops.qkv_prepare(
            qkv, ctx.ints(ctx.POSITIONS), rotary.device_frequencies(ctx.device) if rotary else None,
            rotary.dims if rotary else 0, rotary.amplitude if rotary else 1.0, self.eps, self.unit_norm, k_pool, v_pool,
            slots, self.n_heads, self.n_kv_heads, self.dim, self.vdim, group.page_size, ctx.status,
            v_other=other, blend=self.blend if other is not None else None, keep_values=shared,
            q_weight=self.q_norm, k_weight=self.k_norm, bias=self.qkv_bias, joint_norm=self.joint_norm)
        attended, chain = self.attend(qkv, ctx, group, k_pool, v_pool)
        if self.head_gate or out is not None or factor != 1.0:
            gate = qkv[:, self.gate_at:self.gate_at + self.n_heads] if self.head_gate else None
            attended = mixer_ops.head_gate(attended, gate, self.n_heads, self.vdim, factor, out=out)
        return attended, chain

    def attend(self, qkv: torch.Tensor, ctx: StepContext, group, k_pool, v_pool) -> tuple[torch.Tensor, bool]:
        """The attention itself over prepared queries and the cache: ``[tokens, H vdim]`` in the compute type, and
        whether a product behind it may be chained to the kernel that made it."""
        bias = (self.r1, self.r2) if self.distance_bias else None
        if self._fast(ctx, group.page_size):
            return self._attend_fast(qkv, ctx, group, k_pool, v_pool), False
        if self._shaped_split(ctx, group.page_size):
            return self._attend_shaped(qkv, ctx, group, k_pool, v_pool, bias), False
        if self._mma(ctx):
            attended = mixer_ops.attention_sink_mma(
                qkv, k_pool, v_pool, ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS),
                ctx.ints(self._mma_names()[0]), ctx.ints(self._mma_names()[1]), self.n_heads, self.n_kv_heads,
                self.dim, self.vdim, group.page_size, self.window or 0, self.keep_first, self.scale, self.softcap, ctx.status,
                num_splits=self._mma_splits(ctx), head_scale=self.temp, distance_bias=bias)
            return attended, True
        seq_name, row_name = self._work_names()
        attended = mixer_ops.attention_sink(
            qkv, k_pool, v_pool, ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS),
            ctx.ints(seq_name), ctx.ints(row_name), self.n_heads, self.n_kv_heads, self.dim, self.vdim, group.page_size,
            self.window or 0, self.keep_first, self.scale, self.softcap, ctx.status, head_scale=self.temp, distance_bias=bias)
        return attended, True
