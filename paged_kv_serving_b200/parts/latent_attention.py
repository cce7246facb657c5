"""Attention whose keys and values are read out of one cached latent vector per position."""

from __future__ import annotations

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm, mixer_ops
from paged_kv_serving_b200.parts.base import CacheBinding, PagedKVRequest, ParamSpec, Part, StepContext

__all__ = ["LatentAttention"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """Causal softmax attention with low-rank keys and values, optionally low-rank queries and an
    output gate.

    With ``h`` the input: ``c_q = rmsnorm(W_dq h) * dq_norm`` and ``q = W_uq c_q`` (with ``q_rank``
    0: ``q = W_q h``, one matrix named ``q``), laid out head
    by head as ``[dim unrotated | rot_dim rotated]``. ``W_dkv h`` gives ``kv_rank`` numbers whose
    RMS norm (times ``dkv_norm``) is the latent ``c``, and ``rot_dim`` more that form one rotated
    key part shared by all heads. Head ``a`` has keys ``W_uk[a] c`` and values ``W_uv[a] c``; the
    score is ``(q_unrotated . k_unrotated + q_rotated . k_rotated) * scale``; the head's result is
    multiplied by ``sigmoid(W_g h)[a]`` (with ``gate``) and the heads go through ``W_o``. Rotation acts on the
    first ``rot_dims`` coordinates of the rotated parts with angle ``position * base^(-2i /
    rot_dims)`` for pair ``i``: coordinate ``i`` pairs with ``i + rot_dims / 2`` (``pairing="halves"``) or
    coordinate ``2i`` with ``2i + 1`` (``pairing="interleaved"``). The kernels rotate halves; for the
    interleaved pairing the rows of the query and key projections that produce the rotated
    coordinates are reordered at load (even ones first, then odd ones), which changes no score
    because queries and keys are reordered alike and only their dot product is used.

    Only ``[c | rotated key part]`` is cached, ``kv_rank + rot_dim`` numbers a position for all
    heads (a page group without values). The kernels use the absorbed form: the unrotated query of
    a head is multiplied by ``W_uk[a]`` first (``q_lat = W_uk[a]^T q_unrotated``, one batched
    product), so that the score is a dot product with the cached row, the softmax-weighted sum
    runs over the latents themselves, and ``W_uv[a]`` is applied to that sum (a second batched
    product). Norms, angles, scores and softmax are float32 in both compute types.
    """

    graph_safe = True
    #: The output projection may carry the caller's residual add and norm (``finish``, see ``Part``);
    #: it is not chained to the kernels before it, which are library products and a copy.
    fuses_last_linear = True
    chains_last_linear = False
    #: Set to False to keep bfloat16 steps on the general (float32-arithmetic) kernel; tests compare the two.
    USE_TENSOR_CORES = True

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float,
                 rot_base: float, rot_dims: int, eps: float, window: int | None = None, gate: bool = True,
                 pairing: str = "halves") -> None:
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ValueError("the rotated coordinates must be an even number within the rotated part")
        if pairing not in ("halves", "interleaved"):
            raise ValueError("pairing is 'halves' or 'interleaved'")
        self.gate, self.pairing = bool(gate), pairing
        if kv_rank > 512:
            raise ValueError("the latent attention kernel takes a latent of up to 512 numbers")
        self.width, self.heads, self.dim, self.rot_dim, self.vdim = int(width), int(heads), int(dim), int(rot_dim), int(vdim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.rot_base, self.rot_dims, self.window = float(rot_base), int(rot_dims), window
        # columns of the fused down-projection: [query latent | key/value latent, key part | gate], padded
        self.q_off, self.kv_off = 0, self.q_rank
        self.g_off = self.q_rank + self.kv_rank + self.rot_dim
        self.fused_rows = _round_up(self.g_off + (self.heads if self.gate else 0), 8)
        half = self.rot_dims // 2
        self._freq_host = np.asarray([self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(half)] or [0.0],
                                     dtype=np.float64).astype(np.float32)
        self.freq: torch.Tensor | None = None
        self._mma_ok: bool | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        head = self.dim + self.rot_dim
        specs = {
            "dkv": ParamSpec((self.kv_rank + self.rot_dim, self.width)), "dkv_norm": ParamSpec((self.kv_rank,), "vector"),
            "uk": ParamSpec((self.heads * self.dim, self.kv_rank)), "uv": ParamSpec((self.heads * self.vdim, self.kv_rank)),
            "o": ParamSpec((self.width, self.heads * self.vdim)),
        }
        if self.q_rank:
            specs.update({"dq": ParamSpec((self.q_rank, self.width)), "dq_norm": ParamSpec((self.q_rank,), "vector"),
                          "uq": ParamSpec((self.heads * head, self.q_rank))})
        else:
            specs["q"] = ParamSpec((self.heads * head, self.width))
        if self.gate:
            specs["g"] = ParamSpec((self.heads, self.width))
        return specs

    def _halves_order(self, rows: torch.Tensor, start: int) -> torch.Tensor:
        """``rows`` with the ``rot_dims`` rows from ``start`` on reordered from interleaved pairs to halves."""
        if self.pairing != "interleaved" or not self.rot_dims:
            return rows
        order = torch.arange(rows.shape[0], device=rows.device)
        turned = torch.cat([torch.arange(0, self.rot_dims, 2), torch.arange(1, self.rot_dims, 2)]).to(rows.device)
        order[start:start + self.rot_dims] = start + turned
        return rows[order]

    def load(self, params: dict[str, torch.Tensor]) -> None:
        head = self.dim + self.rot_dim
        dkv = self._halves_order(params["dkv"], self.kv_rank)
        fused = torch.zeros((self.fused_rows, self.width), dtype=dkv.dtype, device=dkv.device)
        if self.q_rank:
            fused[:self.q_rank] = params["dq"]
        fused[self.kv_off:self.g_off] = dkv
        if self.gate:
            fused[self.g_off:self.g_off + self.heads] = params["g"]
        self.down = fused                                                     # [fused_rows, width]
        up = params["uq"] if self.q_rank else params["q"]
        up = up.view(self.heads, head, up.shape[1])
        self.uq = torch.stack([self._halves_order(up[a], self.dim) for a in range(self.heads)]).view(self.heads * head, -1).contiguous()
        self.uk = params["uk"].view(self.heads, self.dim, self.kv_rank).contiguous()        # q_lat = q_unrot @ uk[a]
        self.uv_t = params["uv"].view(self.heads, self.vdim, self.kv_rank).transpose(1, 2).contiguous()   # [a, rank, vdim]
        self.o = params["o"].contiguous()
        self.dq_norm, self.dkv_norm = params.get("dq_norm"), params["dkv_norm"]
        self.freq = torch.from_numpy(self._freq_host).to(dkv.device)

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(1, self.kv_rank + self.rot_dim, self.window, values=False)

    def _tensor_cores(self, ctx: StepContext) -> bool:
        if ctx.dtype != torch.bfloat16 or not self.USE_TENSOR_CORES:
            return False
        if self._mma_ok is None:
            self._mma_ok = mixer_ops.latent_mma_supports(self.kv_rank, self.rot_dim)
        return self._mma_ok

    def _work_names(self, ctx: StepContext) -> tuple[str, str]:
        # (everything the work list depends on is part of its name: layers share a list only when it is the same)
        kind = f"mma{self.kv_rank}+{self.rot_dim}" if self._tensor_cores(ctx) else "general"
        return (f"latent_attention/{kind}/work_seq/h{self.heads}", f"latent_attention/{kind}/work_row0/h{self.heads}")

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        seq_name, row_name = self._work_names(ctx)
        if seq_name in ctx.arena:
            return
        per_block = mixer_ops.latent_mma_rows_per_block(self.kv_rank, self.rot_dim) if self._tensor_cores(ctx) \
            else mixer_ops.latent_rows_per_block()
        rows = np.asarray(ctx.seq_lens, dtype=np.int64) * self.heads
        blocks = (rows + per_block - 1) // per_block
        work_seq = np.repeat(np.arange(len(rows), dtype=np.int64), blocks)
        starts = np.cumsum(blocks) - blocks
        work_row0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * per_block
        # the blocks with the most keys to walk first, so that the last round of blocks is short
        cost = np.asarray(ctx.first_positions, dtype=np.int64)[work_seq] + work_row0 // self.heads
        order = np.argsort(-cost, kind="stable")
        ctx.arena.add(seq_name, work_seq[order])
        ctx.arena.add(row_name, work_row0[order])
        # A step of few rows over long contexts (decoding) would leave most SMs idle with one block
        # an entry: the key range is then cut into parts that run side by side and are merged.
        splits = 1
        if self._tensor_cores(ctx) and len(work_seq):
            longest = ctx.planning_context_len or int((np.asarray(ctx.first_positions) + np.asarray(ctx.seq_lens)).max())
            columns = -(-self.kv_rank // 256)
            places = 2 * torch.cuda.get_device_properties(ctx.device).multi_processor_count
            splits = int(max(1, min(16, places // (len(work_seq) * columns), longest // 128)))
        ctx.scratch[seq_name] = splits

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, finish=None) -> torch.Tensor:
        group = ctx.groups[binding.group]
        pool = group.k_pool[binding.index]
        tokens = x.shape[0]
        head = self.dim + self.rot_dim
        # every down-projection of the input in one product, kept in float32 for the norms
        fused = gemm.linear(x, self.down, out_dtype=torch.float32)
        slots = ctx.ints(group.slots_name) if binding.write else None
        c_q = mixer_ops.latent_prepare(fused, self.q_off, self.q_rank, self.kv_off, self.kv_rank, self.rot_dim, self.rot_dims,
                                       self.dq_norm, self.dkv_norm, self.freq, self.eps, ctx.ints(ctx.POSITIONS), slots, pool,
                                       ctx.status)
        q = gemm.linear(c_q if self.q_rank else x, self.uq)                    # [tokens, heads * (dim + rot_dim)]
        q_unrotated = q.view(tokens, self.heads, head)[:, :, :self.dim].transpose(0, 1)     # [heads, tokens, dim], a view
        q_lat = torch.bmm(q_unrotated, self.uk, out_dtype=torch.float32) if q.dtype != torch.float32 \
            else torch.bmm(q_unrotated, self.uk)
        seq_name, row_name = self._work_names(ctx)
        gate = fused[:, self.g_off:self.g_off + self.heads] if self.gate else None
        kernel = mixer_ops.latent_attention_mma if self._tensor_cores(ctx) else mixer_ops.latent_attention
        extra = {"num_splits": ctx.scratch.get(seq_name, 1)} if self._tensor_cores(ctx) else {}
        attended = kernel(
            q_lat, q, self.dim, head, pool, ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS),
            ctx.ints(seq_name), ctx.ints(row_name), self.freq, gate, self.heads, self.kv_rank, self.rot_dim, self.rot_dims,
            group.page_size, self.window or 0, self.scale, ctx.status, **extra)
        values = torch.bmm(attended, self.uv_t)                                # [heads, tokens, vdim]
        merged = values.transpose(0, 1).reshape(tokens, self.heads * self.vdim)
        return finish(merged, self.o) if finish is not None else gemm.linear(merged, self.o)
