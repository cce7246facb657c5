"""Bindings of the kernels in ``csrc/pointwise.cu``, ``csrc/conv_state.cu``, ``csrc/mlstm.cu``,
``csrc/selective_scan.cu``, ``csrc/latent_attention.cu``, ``csrc/attention_sink.cu``, ``csrc/layernorm.cu``,
``csrc/lightning.cu`` and ``csrc/linear_attention.cu``: what mixers
with a state of their own, a cached latent, a window that keeps the first tokens, routed experts
and per-token side inputs need beside the kernels bound in ``ops/__init__.py``.
The same conventions hold: CUDA tensors only, launches on torch's current stream, a refused
argument raises ``ValueError``, nothing falls back to a library or to the CPU.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.ops import _check, _fn, _need, _ptr, _stream, dtype_code
from paged_kv_serving_b200.ops.arena import empty as _empty

__all__ = ["ACTIVATIONS", "act_times_table", "bias_act", "conv_residual", "expert_act", "expert_gated_act", "norm_residual", "latent_attention",
           "latent_attention_mma", "latent_mma_rows_per_block", "latent_mma_supports", "latent_prepare",
           "latent_rows_per_block", "mlstm", "residual_add", "route_top", "token_side", "attention_sink",
           "attention_sink_mma", "attention_sink_mma_rows", "attention_sink_mma_supports", "attention_sink_rows_per_block", "qkv_prepare", "selective_scan",
           "layer_norm_step", "lightning", "lightning_chunk", "softcap", "token_shift", "route_scored", "gated_bias_act",
           "pair_rows", "assign_bias", "combine_pair", "head_gate", "linear_attention", "linear_attention_chunk"]

#: activation names of ``bias_act`` / ``act_times_table`` / ``expert_act``
ACTIVATIONS = {"none": 0, "gelu_erf": 1, "gelu_tanh": 2, "relu_squared": 3, "sigmoid": 4, "silu": 5}


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, act: str, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``act(x + bias)`` for ``x [rows, cols]`` and a float32 ``bias [cols]`` (or none)."""
    _need(x, None, "x")
    rows, cols = x.shape
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != cols:
            raise ValueError(f"bias has {bias.numel()} elements for {cols} columns")
    out = _empty((rows, cols), out_dtype or x.dtype, x.device)
    fn = _fn("pointwise", "pkv_bias_act", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), _ptr(bias), _ptr(out), dtype_code(out.dtype), rows, cols, ACTIVATIONS[act],
              _stream()), "bias_act")
    return out


def residual_add(hidden: torch.Tensor, delta: torch.Tensor | None, bias: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """``hidden += delta + bias`` in place (float32 stream) and, with ``out_dtype``, the stream in
    that type (what a product that reads the stream itself, not a norm of it, takes)."""
    _need(hidden, torch.float32, "hidden")
    rows, cols = hidden.shape
    if delta is not None:
        _need(delta, None, "delta")
        if delta.shape != hidden.shape:
            raise ValueError("delta and hidden differ in shape")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != cols:
            raise ValueError("bias does not fit the stream's width")
    out = _empty((rows, cols), out_dtype, hidden.device) if out_dtype is not None else None
    fn = _fn("pointwise", "pkv_residual_add", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(fn(_ptr(hidden), _ptr(delta), dtype_code(delta.dtype) if delta is not None else 0, _ptr(bias), _ptr(out),
              dtype_code(out_dtype) if out_dtype is not None else 0, rows, cols, _stream()), "residual_add")
    return out


def act_times_table(z: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int, act: str, status: torch.Tensor,
                    fed_back: torch.Tensor | None = None, fed_back_at: torch.Tensor | None = None) -> torch.Tensor:
    """``act(z[t, j]) * table[ids[t], col0 + j]`` for ``z [tokens, n]``; ids as in ``embedding_gather``."""
    _need(z, None, "z"); _need(table, z.dtype, "table"); _need(ids, torch.int32, "ids")
    tokens, n = z.shape
    out = _empty((tokens, n), z.dtype, z.device)
    fn = _fn("pointwise", "pkv_act_times_table",
             [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p])
    _check(fn(_ptr(z), _ptr(table), dtype_code(z.dtype), table.shape[1], table.shape[0], _ptr(ids), int(col0), _ptr(out),
              tokens, n, ACTIVATIONS[act], _ptr(fed_back), _ptr(fed_back_at), _ptr(status), _stream()), "act_times_table")
    return out


def route_top(logits: torch.Tensor, experts: int, top: int, bias: torch.Tensor | None = None,
              renormalise: bool = False) -> torch.Tensor:
    """Router weights ``[tokens, experts]`` (float32) of each token's ``top`` experts with the
    largest logits, zero elsewhere: their softmax scores over all experts as they are, or, with
    ``renormalise``, the softmax over the chosen logits only. ``logits [tokens, >= experts]``
    float32 (further columns are ignored); ``bias [experts]`` float32 is added to them first."""
    _need(logits, torch.float32, "logits")
    tokens, ld = logits.shape
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != experts:
            raise ValueError("the router's bias needs one element per expert")
    out = _empty((tokens, experts), torch.float32, logits.device)
    fn = _fn("pointwise", "pkv_route_top", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(logits), ld, _ptr(bias), _ptr(out), tokens, experts, top, int(bool(renormalise)), _stream()), "route_top")
    return out


def expert_gated_act(gate_up: torch.Tensor, up_at: int, weights: torch.Tensor, experts: int, ff: int, shared_ff: int,
                     act: str) -> torch.Tensor:
    """``weights[t, e] * act(gate[t, e * ff + j]) * up[t, e * ff + j]`` for the routed experts'
    columns and ``act(gate) * up`` for the ``shared_ff`` columns behind them. A row of ``gate_up``
    holds all gate columns and, ``up_at`` columns further on, all up columns in the same order."""
    _need(gate_up, None, "gate_up"); _need(weights, torch.float32, "weights")
    tokens, ld = gate_up.shape
    cols = experts * ff + shared_ff
    if up_at < cols or ld < up_at + cols or weights.shape != (tokens, experts):
        raise ValueError("expert_gated_act: sizes do not fit")
    out = _empty((tokens, cols), gate_up.dtype, gate_up.device)
    fn = _fn("pointwise", "pkv_expert_gated_act",
             [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), dtype_code(gate_up.dtype), ld, int(up_at), _ptr(weights), _ptr(out), tokens, experts, ff,
              shared_ff, ACTIVATIONS[act], _stream()), "expert_gated_act")
    return out


def norm_residual(hidden: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """``hidden += delta / sqrt(mean(delta^2) + eps) * weight`` in place (float32 stream) and, with
    ``out_dtype``, the updated stream in that type: the residual step of a block that normalises
    a sublayer's output, whose next sublayer reads the stream itself."""
    _need(hidden, torch.float32, "hidden"); _need(delta, None, "delta"); _need(weight, torch.float32, "weight")
    rows, d = hidden.shape
    if delta.shape != hidden.shape or weight.numel() != d:
        raise ValueError("norm_residual: sizes do not fit")
    out = _empty((rows, d), out_dtype, hidden.device) if out_dtype is not None else None
    fn = _fn("pointwise", "pkv_norm_residual",
             [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(hidden), _ptr(delta), dtype_code(delta.dtype), _ptr(weight), float(eps), _ptr(out),
              dtype_code(out_dtype) if out_dtype is not None else 0, rows, d, _stream()), "norm_residual")
    return out


def expert_act(up: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor | None, experts: int, ff: int, shared_ff: int,
               act: str) -> torch.Tensor:
    """``weights[t, e] * act(up[t, e * ff + j])`` for the routed experts' columns and
    ``sigmoid(gate[t]) * act(up)`` for the ``shared_ff`` columns behind them; ``gate`` is a float32
    column view ``[tokens]`` (any stride) or none. ``up`` may have further (padding) columns."""
    _need(up, None, "up"); _need(weights, torch.float32, "weights")
    tokens, ld = up.shape
    cols = experts * ff + shared_ff
    if ld < cols or weights.shape != (tokens, experts):
        raise ValueError("expert_act: sizes do not fit")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 1 or gate.shape[0] != tokens:
            raise ValueError("gate must be float32 [tokens]")
        gate_ld = gate.stride(0)
    out = _empty((tokens, cols), up.dtype, up.device)
    fn = _fn("pointwise", "pkv_expert_act",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(up), dtype_code(up.dtype), ld, _ptr(weights), _ptr(gate), gate_ld, _ptr(out), tokens, experts, ff,
              shared_ff, ACTIVATIONS[act], _stream()), "expert_act")
    return out


def conv_residual(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, token_seq: torch.Tensor,
                  seq_starts: torch.Tensor, state_slots: torch.Tensor, weight_t: torch.Tensor | None = None,
                  bias: torch.Tensor | None = None, residual: bool = True, act: str = "none") -> torch.Tensor:
    """A causal convolution per channel for a ragged batch, ``weight [width, taps]`` float32 with
    tap ``taps - 1`` on the token itself: ``x + conv(x)`` (``residual``, the default) or
    ``act(conv(x) + bias)`` with ``act`` "none" or "silu". ``x [tokens, width]`` may be a column
    range of a wider matrix (its rows keep their stride). ``state [slots, taps - 1, width]`` (type
    of ``x``) holds every request's last inputs and is brought up to date. ``weight_t`` (the
    weights as ``[taps, width]``) lets bfloat16 rows of a width that is a multiple of 8 take the
    16-byte kernel."""
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a CUDA matrix whose rows are contiguous")
    _need(weight, torch.float32, "weight")
    if weight_t is not None:
        _need(weight_t, torch.float32, "weight_t")
        if weight_t.shape != (weight.shape[1], weight.shape[0]):
            raise ValueError("weight_t must be the transpose of weight")
    tokens, width = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != width:
        raise ValueError("conv weight does not fit the width")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != width:
            raise ValueError("conv bias does not fit the width")
    if taps > 1:
        _need(state, x.dtype, "state")
        if state.shape[1:] != (taps - 1, width):
            raise ValueError("conv state must be [slots, taps - 1, width]")
    seqs = seq_starts.numel() - 1
    out = _empty((tokens, width), x.dtype, x.device)
    fn = _fn("conv_state", "pkv_conv_residual",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), x.stride(0) if tokens > 1 else max(x.stride(0), width), _ptr(weight), _ptr(weight_t),
              _ptr(bias), _ptr(state), _ptr(token_seq), _ptr(seq_starts), _ptr(state_slots), _ptr(out), tokens, seqs, width,
              taps, int(bool(residual)), {"none": 0, "silu": 1}[act], _stream()), "conv_residual")
    ops.LAUNCHES["count"] += 1 if taps > 1 else 0
    return out


def mlstm(proj: torch.Tensor, offsets: dict[str, int], i_bias: torch.Tensor, f_bias: torch.Tensor, norm_weight: torch.Tensor,
          cap: float, q_scale: float, eps: float, s_state: torch.Tensor, n_state: torch.Tensor, m_state: torch.Tensor,
          seq_starts: torch.Tensor, state_slots: torch.Tensor, heads: int, dim: int, vdim: int,
          out_dtype: torch.dtype) -> torch.Tensor:
    """The mLSTM recurrence over a ragged batch. ``proj`` float32 ``[tokens, ld]`` holds the
    projections q, k ``[heads, dim]``, v, g ``[heads, vdim]`` and the two gates' pre-activations
    ``[heads]`` at ``offsets`` ("q", "k", "v", "g", "i", "f"). States (float32): ``s_state [slots,
    heads, vdim, dim]`` (column by column), ``n_state [slots, heads, dim]``, ``m_state [slots, heads]``. Returns the
    heads' outputs after their unit norm, the norm's weight and the output gate, ``[tokens, heads * vdim]``."""
    _need(proj, torch.float32, "proj")
    for name, t in (("s_state", s_state), ("n_state", n_state), ("m_state", m_state), ("i_bias", i_bias), ("f_bias", f_bias),
                    ("norm_weight", norm_weight)):
        _need(t, torch.float32, name)
    tokens, ld = proj.shape
    if s_state.shape[1:] != (heads, vdim, dim) or n_state.shape[1:] != (heads, dim) or m_state.shape[1:] != (heads,):
        raise ValueError("mlstm: the states do not fit heads, dim and vdim")
    if norm_weight.numel() != heads * vdim or i_bias.numel() != heads or f_bias.numel() != heads:
        raise ValueError("mlstm: a vector does not fit the head count")
    seqs = seq_starts.numel() - 1
    coef = _empty((tokens, heads, 4), torch.float32, proj.device)
    o = _empty((tokens * heads * (vdim + 1),), torch.float32, proj.device)     # numerators, then n . q per (token, head)
    out = _empty((tokens, heads * vdim), out_dtype, proj.device)
    fn = _fn("mlstm", "pkv_mlstm",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float,
              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
              c_int, c_void_p])
    _check(fn(_ptr(proj), ld, offsets["q"], offsets["k"], offsets["v"], offsets["g"], offsets["i"], offsets["f"],
              _ptr(i_bias), _ptr(f_bias), _ptr(norm_weight), float(cap), float(q_scale), float(eps), _ptr(s_state),
              _ptr(n_state), _ptr(m_state), _ptr(seq_starts), _ptr(state_slots), _ptr(coef), _ptr(o), _ptr(out),
              dtype_code(out_dtype), tokens, seqs, heads, dim, vdim, _stream()), "mlstm")
    ops.LAUNCHES["count"] += 2
    return out


def latent_rows_per_block() -> int:
    fn = ops.library("latent_attention").pkv_latent_rows_per_block
    fn.restype = c_int
    return int(fn())


def latent_prepare(fused: torch.Tensor, q_off: int, q_rank: int, kv_off: int, rank: int, rot: int, rot_dims: int,
                   q_weight: torch.Tensor, kv_weight: torch.Tensor, freq: torch.Tensor, eps: float, positions: torch.Tensor,
                   slots: torch.Tensor | None, pool: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """From the fused down-projections ``fused`` (float32 ``[tokens, ld]``): the RMS-normalised
    query latent ``[tokens, q_rank]`` (returned, in the pool's type; ``q_rank`` 0: there is none), and the cache row
    ``[normalised latent | rotated key part]`` written at ``slots`` (int32 per token, negative or
    ``None``: nothing is written) of ``pool [pages, 1, page_size, rank + rot]``."""
    _need(fused, torch.float32, "fused"); _need(pool, None, "pool"); _need(freq, torch.float32, "freq")
    _need(kv_weight, torch.float32, "kv_weight")
    if q_rank:
        _need(q_weight, torch.float32, "q_weight")
    tokens, ld = fused.shape
    if pool.shape[-1] != rank + rot:
        raise ValueError("the pool's rows must hold rank + rot values")
    pool_rows = pool.numel() // (rank + rot)
    c_q = _empty((tokens, q_rank), pool.dtype, fused.device)
    fn = _fn("latent_attention", "pkv_latent_prepare",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
              c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(fused), ld, q_off, q_rank, kv_off, rank, rot, rot_dims, _ptr(q_weight), _ptr(kv_weight), _ptr(freq),
              float(eps), _ptr(positions), _ptr(slots), _ptr(c_q), _ptr(pool), dtype_code(pool.dtype), pool_rows, tokens,
              _ptr(status), _stream()), "latent_prepare")
    return c_q


def latent_attention(q_lat: torch.Tensor, q: torch.Tensor, q_rot_offset: int, q_head_stride: int, pool: torch.Tensor,
                     block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor, work_seq: torch.Tensor,
                     work_row0: torch.Tensor, freq: torch.Tensor, gate: torch.Tensor | None, heads: int, rank: int, rot: int,
                     rot_dims: int, page_size: int, window: int, scale: float, status: torch.Tensor,
                     n_work: int | None = None) -> torch.Tensor:
    """Causal attention of absorbed queries over the cached latent. ``q_lat [heads, tokens, rank]``
    (float32, or the type of ``q``); the rotated part of head ``h`` of token ``t`` is read (and
    rotated) from ``q[t, h * q_head_stride + q_rot_offset :][:rot]``; ``gate`` float32 ``[tokens, >=
    heads]`` (a view with a row stride) multiplies the result by its sigmoid. Returns ``[heads,
    tokens, rank]`` in the type of ``q``: per head the softmax-weighted sum of the latents."""
    _need(q_lat, None, "q_lat"); _need(q, None, "q"); _need(pool, q.dtype, "pool")
    tokens = q.shape[0]
    if q_lat.shape != (heads, tokens, rank):
        raise ValueError("q_lat must be [heads, tokens, rank]")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.stride(1) != 1:
            raise ValueError("gate must be a float32 [tokens, heads] view with unit inner stride")
        gate_ld = gate.stride(0)
    out = _empty((heads, tokens, rank), q.dtype, q.device)
    num_pages = pool.numel() // (page_size * (rank + rot))
    fn = _fn("latent_attention", "pkv_latent_attention",
             [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
              c_int, c_void_p, c_void_p])
    q_rot = q.view(-1)[q_rot_offset:]
    _check(fn(_ptr(q_lat), dtype_code(q_lat.dtype), c_void_p(q_rot.data_ptr()), q.stride(0), q_head_stride, _ptr(out),
              dtype_code(q.dtype), _ptr(pool), dtype_code(pool.dtype), _ptr(block_table), block_table.shape[1],
              _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), _ptr(work_row0), work_seq.numel() if n_work is None else int(n_work), _ptr(freq), _ptr(gate),
              gate_ld, tokens, heads, rank, rot, rot_dims, page_size, int(window), float(scale), num_pages, _ptr(status),
              _stream()), "latent_attention")
    return out


def latent_mma_rows_per_block(rank: int, rot: int) -> int:
    """Rows of one block of the tensor-core kernel at these sizes (128, or 64 for wide latents)."""
    fn = ops.library("latent_attention").pkv_latent_mma_rows_per_block
    fn.restype = c_int
    fn.argtypes = [c_int, c_int]
    return int(fn(int(rank), int(rot)))


def latent_mma_supports(rank: int, rot: int) -> bool:
    """Whether the tensor-core kernel takes a latent of ``rank`` numbers with ``rot`` rotated ones
    behind them (multiples of 16 that fit its shared memory)."""
    fn = ops.library("latent_attention").pkv_latent_mma_supports
    fn.restype = c_int
    fn.argtypes = [c_int, c_int]
    return bool(fn(int(rank), int(rot)))


def latent_attention_mma(q_lat: torch.Tensor, q: torch.Tensor, q_rot_offset: int, q_head_stride: int, pool: torch.Tensor,
                         block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor, work_seq: torch.Tensor,
                         work_row0: torch.Tensor, freq: torch.Tensor, gate: torch.Tensor | None, heads: int, rank: int,
                         rot: int, rot_dims: int, page_size: int, window: int, scale: float, status: torch.Tensor,
                         n_work: int | None = None, num_splits: int = 1) -> torch.Tensor:
    """``latent_attention`` on the tensor cores, for bfloat16 queries and cache (``q_lat`` float32
    or bfloat16); the work list is in blocks of ``latent_mma_rows_per_block(rank, rot)`` rows.
    ``num_splits`` > 1 cuts every block's key range into that many parts that run side by side and
    are merged by a second kernel (for steps of few rows over long contexts)."""
    _need(q_lat, None, "q_lat"); _need(q, torch.bfloat16, "q"); _need(pool, torch.bfloat16, "pool")
    tokens = q.shape[0]
    if q_lat.shape != (heads, tokens, rank):
        raise ValueError("q_lat must be [heads, tokens, rank]")
    if (q.stride(0) * 2) % 4 or (q_head_stride * 2) % 2:
        raise ValueError("the query rows are not aligned")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.stride(1) != 1:
            raise ValueError("gate must be a float32 [tokens, heads] view with unit inner stride")
        gate_ld = gate.stride(0)
    out = _empty((heads, tokens, rank), torch.bfloat16, q.device)
    num_pages = pool.numel() // (page_size * (rank + rot))
    fn = _fn("latent_attention", "pkv_latent_attention_mma",
             [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
              c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    q_rot = q.view(-1)[q_rot_offset:]
    part_o = part_ml = None
    if num_splits > 1:
        part_o = _empty((num_splits, heads * tokens, rank), torch.float32, q.device)
        part_ml = _empty((num_splits, heads * tokens, 2), torch.float32, q.device)
    _check(fn(_ptr(q_lat), dtype_code(q_lat.dtype), c_void_p(q_rot.data_ptr()), q.stride(0), q_head_stride, _ptr(out),
              _ptr(pool), _ptr(block_table), block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq),
              _ptr(work_row0), work_seq.numel() if n_work is None else int(n_work), _ptr(freq), _ptr(gate), gate_ld, tokens,
              heads, rank, rot, rot_dims, page_size, int(window), float(scale), num_pages, _ptr(status), int(num_splits),
              _ptr(part_o), _ptr(part_ml), _stream()),
           "latent_attention_mma")
    if num_splits > 1:
        ops.LAUNCHES["count"] += 1
    return out


def token_side(hidden: torch.Tensor, delta: torch.Tensor | None, bias: torch.Tensor | None, gate_w: torch.Tensor,
               proj_w: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int, norm_w: torch.Tensor, eps: float,
               act: str, status: torch.Tensor, fed_back: torch.Tensor | None = None,
               fed_back_at: torch.Tensor | None = None) -> torch.Tensor:
    """The per-token side input in one kernel (one block a token; for the few rows of a decode
    step): ``hidden += delta + bias`` in place, then ``rmsnorm(proj_w (act(gate_w x) * table[ids,
    col0:col0 + dim])) * norm_w`` of the updated rows ``x``, float32 ``[tokens, width]``. ``gate_w
    [dim, width]``, ``proj_w [width, dim]`` and ``table`` share one type; the stages round as the
    separate kernels and products do."""
    _need(hidden, torch.float32, "hidden"); _need(gate_w, None, "gate_w"); _need(proj_w, gate_w.dtype, "proj_w")
    _need(table, gate_w.dtype, "table"); _need(norm_w, torch.float32, "norm_w"); _need(ids, torch.int32, "ids")
    tokens, width = hidden.shape
    dim = gate_w.shape[0]
    if gate_w.shape != (dim, width) or proj_w.shape != (width, dim) or norm_w.numel() != width:
        raise ValueError("token_side: sizes do not fit")
    if delta is not None:
        _need(delta, None, "delta")
        if delta.shape != hidden.shape:
            raise ValueError("delta and hidden differ in shape")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    out = _empty((tokens, width), torch.float32, hidden.device)
    fn = _fn("pointwise", "pkv_token_side",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
              c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(hidden), _ptr(delta), dtype_code(delta.dtype) if delta is not None else 0, _ptr(bias), _ptr(gate_w),
              _ptr(proj_w), _ptr(table), dtype_code(gate_w.dtype), table.shape[1], table.shape[0], _ptr(ids), int(col0),
              _ptr(norm_w), float(eps), _ptr(out), tokens, width, dim, ACTIVATIONS[act], _ptr(fed_back), _ptr(fed_back_at),
              _ptr(status), _stream()), "token_side")
    return out


def selective_scan(x: torch.Tensor, z: torch.Tensor, dt_pre: torch.Tensor, dt_bias: torch.Tensor, bc: torch.Tensor, b_at: int,
                   c_at: int, a: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, seq_starts: torch.Tensor,
                   state_slots: torch.Tensor) -> torch.Tensor:
    """The selective scan of a Mamba mixer over a ragged batch. ``x`` and ``z`` ``[tokens, inner]``
    in the compute type (column ranges of wider matrices are fine); ``dt_pre`` float32 ``[tokens,
    inner]`` (the step sizes before bias and softplus); ``bc`` float32 ``[tokens, ld]`` with
    ``B`` at column ``b_at`` and ``C`` at ``c_at``; ``a [inner, state]``, ``dt_bias`` and
    ``d_skip [inner]`` float32; ``state`` float32 ``[slots, inner, state]`` is read and brought up
    to date. Returns ``y * silu(z)`` ``[tokens, inner]`` in the type of ``x``."""
    for name, t in (("dt_pre", dt_pre), ("bc", bc)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be a float32 CUDA matrix whose rows are contiguous")
    for name, t in (("x", x), ("z", z)):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != x.dtype:
            raise ValueError(f"{name} must be a CUDA matrix whose rows are contiguous")
    for name, t in (("a", a), ("dt_bias", dt_bias), ("d_skip", d_skip), ("state", state)):
        _need(t, torch.float32, name)
    tokens, inner = x.shape
    n_state = a.shape[1]
    if a.shape != (inner, n_state) or z.shape != x.shape or dt_pre.shape[0] != tokens or dt_pre.shape[1] < inner or \
            dt_bias.numel() != inner or d_skip.numel() != inner or state.shape[1:] != (inner, n_state) or bc.shape[0] != tokens:
        raise ValueError("selective_scan: sizes do not fit")
    seqs = seq_starts.numel() - 1
    out = _empty((tokens, inner), x.dtype, x.device)

    def ld(t: torch.Tensor) -> int:
        return max(t.stride(0), t.shape[1])

    fn = _fn("selective_scan", "pkv_selective_scan",
             [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), ld(x), _ptr(z), ld(z), dtype_code(x.dtype), _ptr(dt_pre), ld(dt_pre), _ptr(dt_bias), _ptr(bc), ld(bc),
              int(b_at), int(c_at), _ptr(a), _ptr(d_skip), _ptr(state), _ptr(seq_starts), _ptr(state_slots), _ptr(out), tokens,
              seqs, inner, n_state, _stream()), "selective_scan")
    return out


def qkv_prepare(qkv: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor | None, rot_dims: int, rot_factor: float,
                eps: float, unit_norm: bool, k_pool: torch.Tensor, v_pool: torch.Tensor, slots: torch.Tensor | None,
                n_heads: int, n_kv: int, dim: int, vdim: int, page_size: int, status: torch.Tensor,
                v_other: torch.Tensor | None = None, blend: torch.Tensor | None = None,
                keep_values: torch.Tensor | None = None, q_weight: torch.Tensor | None = None,
                k_weight: torch.Tensor | None = None, bias: torch.Tensor | None = None, joint_norm: bool = False) -> None:
    """In ``qkv [tokens, >= H dim + G dim + G vdim]`` (columns ``[Q | K | V]``): rotate the first
    ``rot_dims`` coordinates of every query and key head (``freq [rot_dims / 2]`` float32 angular
    frequencies, cos and sin times ``rot_factor``), divide those heads by their root mean square
    (``unit_norm``) and multiply them by ``q_weight`` / ``k_weight`` (float32 ``[dim]``, the same for every
    head; ``None``: no factor), write the queries back in place and the keys into ``k_pool [pages, G,
    page_size, dim]`` at ``slots``; blend the values with ``v_other [tokens, G vdim]`` (weight
    ``blend``, a float32 tensor of one element: ``(1 - blend) v + blend v_other``) and write them
    into ``v_pool [pages, G, page_size, vdim]``. ``keep_values [tokens, G vdim]`` (type of ``qkv``)
    also receives the values as they are cached. ``bias`` (float32, one element per column ``[Q | K | V]``)
    is added to the columns first. ``joint_norm``: in place of the norm per head, all query columns of a
    token are divided by their joint root mean square and multiplied by ``q_weight [H dim]`` (the key
    columns likewise, ``k_weight [G dim]``) before the rotation."""
    _need(qkv, None, "qkv"); _need(positions, torch.int32, "positions"); _need(k_pool, None, "k_pool")
    _need(v_pool, k_pool.dtype, "v_pool")
    tokens, ld = qkv.shape
    if rot_dims:
        _need(freq, torch.float32, "freq")
        if freq.numel() != rot_dims // 2:
            raise ValueError("freq needs one element per rotated pair")
    ld_other = 0
    if v_other is not None:
        if v_other.dtype != qkv.dtype or v_other.dim() != 2 or v_other.stride(1) != 1 or v_other.shape != (tokens, n_kv * vdim):
            raise ValueError("v_other must be [tokens, G * vdim] in the type of qkv")
        _need(blend, torch.float32, "blend")
        ld_other = v_other.stride(0) if tokens > 1 else n_kv * vdim
    if k_pool.shape[-3:] != (n_kv, page_size, dim) or v_pool.shape[-3:] != (n_kv, page_size, vdim):
        raise ValueError("the pools do not fit heads, page size and head sizes")
    kept = keep_values
    if kept is not None:
        _need(kept, qkv.dtype, "keep_values")
        if kept.shape != (tokens, n_kv * vdim):
            raise ValueError("keep_values must be [tokens, G * vdim]")
    pool_slots = k_pool.numel() // (n_kv * dim)
    for name, t, heads_of in (("q_weight", q_weight, n_heads), ("k_weight", k_weight, n_kv)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != (heads_of * dim if joint_norm else dim):
                raise ValueError(f"{name} needs one element per coordinate of a head (per column with a joint norm)")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() < (n_heads + n_kv) * dim + n_kv * vdim:
            raise ValueError("bias needs one element per query, key and value column")
    if joint_norm and not unit_norm:
        raise ValueError("a joint norm is a norm")
    fn = _fn("attention_sink", "pkv_qkv_prepare",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p])
    _check(fn(_ptr(qkv), dtype_code(qkv.dtype), ld, _ptr(positions), _ptr(freq), int(rot_dims), float(rot_factor), float(eps),
              (2 if joint_norm else 1) if unit_norm else 0, _ptr(q_weight), _ptr(k_weight), _ptr(bias), _ptr(v_other), ld_other, _ptr(blend), _ptr(kept), _ptr(k_pool), _ptr(v_pool),
              dtype_code(k_pool.dtype), _ptr(slots), pool_slots, tokens, n_heads, n_kv, dim, vdim, page_size, _ptr(status),
              _stream()), "qkv_prepare")


def attention_sink_rows_per_block() -> int:
    fn = ops.library("attention_sink").pkv_attention_sink_rows_per_block
    fn.restype = c_int
    return int(fn())


def attention_sink(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                   seq_starts: torch.Tensor, first_pos: torch.Tensor, work_seq: torch.Tensor, work_row0: torch.Tensor,
                   n_heads: int, n_kv: int, dim: int, vdim: int, page_size: int, window: int, keep_first: int, scale: float,
                   softcap: float, status: torch.Tensor, head_scale: torch.Tensor | None = None,
                   distance_bias: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """Paged causal attention in float32 arithmetic: scores ``q.k * scale``, capped as ``softcap *
    tanh(score / softcap)`` (0: no cap); query position ``i`` sees key ``j <= i`` when ``i - j <
    window`` or ``j < keep_first`` (``window`` 0: every earlier key). ``head_scale`` (float32 ``[H]``)
    multiplies the score of its head before the cap; ``distance_bias = (a, b)`` (float32 ``[H]`` each)
    takes ``a[h] * log(1 + b[h] * (i - j))`` off it after the cap. Query head ``h`` of token
    ``t`` is ``q[t, h * dim : (h + 1) * dim]`` (``q`` may have further columns). Returns ``[tokens, H
    * vdim]`` in the type of ``q``. The work list is in blocks of ``attention_sink_rows_per_block()``
    rows per (entry, key/value head)."""
    _need(q, None, "q"); _need(k_pool, None, "k_pool"); _need(v_pool, k_pool.dtype, "v_pool")
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("work_row0", work_row0)):
        _need(t, torch.int32, name)
    tokens = q.shape[0]
    if q.shape[1] < n_heads * dim:
        raise ValueError("q is narrower than its heads")
    out = _empty((tokens, n_heads * vdim), q.dtype, q.device)
    num_pages = k_pool.numel() // (n_kv * page_size * dim)
    bias_a, bias_b = _per_head(head_scale, distance_bias, n_heads)
    fn = _fn("attention_sink", "pkv_attention_sink",
             [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p,
              c_int, c_void_p, c_void_p])
    _check(fn(_ptr(q), q.shape[1], _ptr(out), dtype_code(q.dtype), _ptr(k_pool), _ptr(v_pool), dtype_code(k_pool.dtype),
              _ptr(block_table), block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), _ptr(work_row0),
              work_seq.numel(), n_heads, n_kv, dim, vdim, page_size, int(window), int(keep_first), float(scale), float(softcap),
              _ptr(head_scale), _ptr(bias_a), _ptr(bias_b), num_pages, _ptr(status), _stream()), "attention_sink")
    return out


def _per_head(head_scale: torch.Tensor | None, distance_bias, n_heads: int):
    """Checks the per-head vectors of the two attention kernels; returns the bias pair (or two ``None``)."""
    bias_a, bias_b = distance_bias if distance_bias is not None else (None, None)
    for name, t in (("head_scale", head_scale), ("distance_bias[0]", bias_a), ("distance_bias[1]", bias_b)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n_heads:
                raise ValueError(f"{name} needs one element per query head")
    return bias_a, bias_b


def attention_sink_mma_supports(dim: int, vdim: int, q_row_stride: int) -> bool:
    """Whether the tensor-core form of ``attention_sink`` takes these sizes (bfloat16 only): key
    and value sizes that are multiples of 16 (keys up to 256, values up to 128)."""
    if dim % 16 or vdim % 16 or not 16 <= dim <= 256 or not 16 <= vdim <= 128 or q_row_stride % 8:
        return False     # known without building the library
    return True


def attention_sink_mma_rows() -> int:
    """Rows of one work item of ``attention_sink_mma``."""
    return 64


def attention_sink_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                       seq_starts: torch.Tensor, first_pos: torch.Tensor, work_seq: torch.Tensor, work_q0: torch.Tensor,
                       n_heads: int, n_kv: int, dim: int, vdim: int, page_size: int, window: int, keep_first: int, scale: float,
                       softcap: float, status: torch.Tensor, num_splits: int = 1, head_scale: torch.Tensor | None = None,
                       distance_bias: tuple[torch.Tensor, torch.Tensor] | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``attention_sink`` on the tensor cores (``mma.sync``, bfloat16 operands, float32 scores and
    accumulators) for head sizes that are multiples of 16. The rows of an (entry, key/value head)
    are (token, head in group) pairs, ``row = token * (H / G) + head in group``; the work list is in
    blocks of ``attention_sink_mma_rows()`` rows (``work_q0``: the block's first row) and must
    cover every token of the step when ``num_splits`` > 1: every block's key range is then
    cut into that many shares (at most 8) that run side by side and are merged by a second
    kernel (for steps of few rows over long contexts). With ``out`` the rows of the work list are
    written there (another kernel may serve the step's other rows) instead of into a new tensor."""
    _need(q, torch.bfloat16, "q"); _need(k_pool, torch.bfloat16, "k_pool"); _need(v_pool, torch.bfloat16, "v_pool")
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("work_q0", work_q0)):
        _need(t, torch.int32, name)
    tokens = q.shape[0]
    if q.shape[1] < n_heads * dim:
        raise ValueError("q is narrower than its heads")
    if out is None:
        out = _empty((tokens, n_heads * vdim), q.dtype, q.device)
    else:
        _need(out, torch.bfloat16, "out")
        if tuple(out.shape) != (tokens, n_heads * vdim):
            raise ValueError("out must have a row per token and the width of the heads' values")
    num_pages = k_pool.numel() // (n_kv * page_size * dim)
    part_o = part_ml = None
    if num_splits > 1:
        part_o = _empty((tokens * n_heads * num_splits, vdim), torch.float32, q.device)
        part_ml = _empty((tokens * n_heads * num_splits, 2), torch.float32, q.device)
    bias_a, bias_b = _per_head(head_scale, distance_bias, n_heads)
    fn = _fn("attention_sink", "pkv_attention_sink_mma",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
              c_int, c_void_p, c_void_p, c_longlong, c_void_p])
    _check(fn(_ptr(q), q.shape[1], _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
              _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), _ptr(work_q0), work_seq.numel(), n_heads, n_kv, dim, vdim,
              page_size, int(window), int(keep_first), float(scale), float(softcap), _ptr(head_scale), _ptr(bias_a), _ptr(bias_b),
              num_pages, _ptr(status), int(num_splits),
              _ptr(part_o), _ptr(part_ml), tokens, _stream()), "attention_sink_mma")
    if num_splits > 1:
        ops.LAUNCHES["count"] += 1
    return out


def layer_norm_step(hidden: torch.Tensor, update: torch.Tensor | None = None, post: tuple | None = None, mult: float = 1.0,
                    addend: torch.Tensor | None = None, pre: tuple | None = None, out_dtype: torch.dtype | None = None,
                    rows: torch.Tensor | None = None, eps: float = 1e-5) -> torch.Tensor | None:
    """What happens to a float32 stream between two sublayers of a block whose norms are layer
    norms with weight and bias, in one kernel and float32 arithmetic: ``hidden += mult *
    layer_norm(update; post)`` (with ``update``; ``post = (weight, bias)``), ``hidden += addend``
    (with ``addend``, float32 like the stream), and, with ``pre = (weight, bias)``, the layer norm
    of the updated stream in ``out_dtype`` (returned). With ``rows`` (int32 indices) only those
    rows are worked on, the stream itself stays as it is and the result has one row per index."""
    _need(hidden, torch.float32, "hidden")
    n, width = hidden.shape
    post_w = post_b = pre_w = pre_b = None
    if update is not None:
        _need(update, None, "update")
        if update.shape != hidden.shape or post is None:
            raise ValueError("update must have the stream's shape and come with its norm's weight and bias")
        post_w, post_b = post
        _need(post_w, torch.float32, "post weight"); _need(post_b, torch.float32, "post bias")
        if post_w.numel() != width or post_b.numel() != width:
            raise ValueError("the norm's weight and bias do not fit the stream's width")
    if addend is not None:
        _need(addend, torch.float32, "addend")
        if addend.shape != hidden.shape:
            raise ValueError("addend and hidden differ in shape")
    n_rows = n
    if rows is not None:
        _need(rows, torch.int32, "rows")
        n_rows = rows.numel()
    out = None
    if pre is not None:
        pre_w, pre_b = pre
        _need(pre_w, torch.float32, "pre weight"); _need(pre_b, torch.float32, "pre bias")
        if pre_w.numel() != width or pre_b.numel() != width:
            raise ValueError("the norm's weight and bias do not fit the stream's width")
        out = _empty((n_rows, width), out_dtype or torch.float32, hidden.device)
    fn = _fn("layernorm", "pkv_layer_norm_step",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
              c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(hidden), _ptr(update), dtype_code(update.dtype) if update is not None else 0, _ptr(post_w), _ptr(post_b),
              float(mult), _ptr(addend), _ptr(pre_w), _ptr(pre_b), _ptr(out), dtype_code(out.dtype) if out is not None else 0,
              _ptr(rows), n_rows, width, float(eps), _stream()), "layer_norm_step")
    return out


def token_shift(h: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, token_seq: torch.Tensor, seq_starts: torch.Tensor,
                state_slots: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``h[t] + (h[t - 1] - h[t]) * mix`` for a ragged batch: ``h`` float32 ``[tokens, width]``, ``mix``
    float32 ``[width]``; the row before an entry's first token is the request's row of ``state``
    (float32 ``[slots, width]``), which is then set to the entry's last row of ``h``."""
    _need(h, torch.float32, "h"); _need(mix, torch.float32, "mix"); _need(state, torch.float32, "state")
    tokens, width = h.shape
    if mix.numel() != width or state.dim() != 2 or state.shape[1] != width:
        raise ValueError("token_shift: sizes do not fit")
    out = _empty((tokens, width), out_dtype, h.device)
    fn = _fn("layernorm", "pkv_token_shift",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(h), _ptr(mix), _ptr(state), _ptr(token_seq), _ptr(seq_starts), _ptr(state_slots), _ptr(out),
              dtype_code(out_dtype), tokens, seq_starts.numel() - 1, width, _stream()), "token_shift")
    ops.LAUNCHES["count"] += 1
    return out


#: tokens of one entry up to which the linear-attention kernel walks them in a row
LIGHTNING_IN_A_ROW = 128
#: chunk sizes of the cut form: 64 tokens, or more so that a step has about 64 chunks at most
LIGHTNING_CHUNK, LIGHTNING_CHUNKS = 64, 64


def lightning_chunk(tokens: int, seqs: int) -> int:
    """Tokens per chunk for a step of ``tokens`` tokens in ``seqs`` entries (the host knows no more
    than these two numbers when a step is captured): 0 when no entry can be longer than
    ``LIGHTNING_IN_A_ROW``, else ``LIGHTNING_CHUNK`` or, for very long steps, a multiple of 16 that
    keeps the working memory at about ``LIGHTNING_CHUNKS`` states per head."""
    if tokens - (seqs - 1) <= LIGHTNING_IN_A_ROW:
        return 0
    return max(LIGHTNING_CHUNK, -(-tokens // (LIGHTNING_CHUNKS * 16)) * 16)


def lightning(proj: torch.Tensor, offsets: dict[str, int], decay: torch.Tensor, norm_weight: torch.Tensor, eps: float,
              state: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor, heads: int, dim: int, vdim: int,
              out_dtype: torch.dtype) -> torch.Tensor:
    """Linear attention with a fixed decay per head over a ragged batch. ``proj`` float32 ``[tokens,
    ld]`` holds the projections before their SiLU, q and k ``[heads, dim]``, v and the gate ``[heads,
    vdim]`` at ``offsets`` ("q", "k", "v", "g"); ``decay`` float32 ``[heads]``; ``state`` float32
    ``[slots, heads, vdim, dim]`` is read and brought up to date. Returns the heads' outputs after
    their joint RMS norm, its weight and the sigmoid gate, ``[tokens, heads * vdim]``.

    A step whose longest entry can exceed ``LIGHTNING_IN_A_ROW`` tokens is cut into chunks that run
    side by side (``lightning_chunk``); the others walk each entry's tokens in a row, one launch."""
    _need(proj, torch.float32, "proj"); _need(decay, torch.float32, "decay"); _need(norm_weight, torch.float32, "norm_weight")
    _need(state, torch.float32, "state")
    tokens, ld = proj.shape
    if state.shape[1:] != (heads, vdim, dim) or decay.numel() != heads or norm_weight.numel() != heads * vdim:
        raise ValueError("lightning: sizes do not fit")
    seqs = seq_starts.numel() - 1
    scratch = _empty((tokens, heads * vdim), torch.float32, proj.device)
    out = _empty((tokens, heads * vdim), out_dtype, proj.device)
    chunk = lightning_chunk(tokens, seqs)
    chunk_state = _empty((tokens // chunk + seqs, heads, vdim, dim), torch.float32, proj.device) if chunk else None
    fn = _fn("lightning", "pkv_lightning",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(proj), ld, offsets["q"], offsets["k"], offsets["v"], offsets["g"], _ptr(decay), _ptr(norm_weight), float(eps),
              _ptr(state), _ptr(seq_starts), _ptr(state_slots), _ptr(scratch), _ptr(out), dtype_code(out_dtype), tokens,
              seqs, heads, dim, vdim, chunk, _ptr(chunk_state) if chunk else None, _stream()), "lightning")
    ops.LAUNCHES["count"] += 3 if chunk else 1
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(x / cap)`` in place on a float32 tensor (returned)."""
    _need(x, torch.float32, "x")
    fn = _fn("pointwise", "pkv_softcap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(fn(_ptr(x), x.numel(), float(cap), _stream()), "softcap")
    return x


def route_scored(logits: torch.Tensor, experts: int, top: int, correction: torch.Tensor | None = None, groups: int = 1,
                 keep: int = 1, scale: float = 1.0) -> torch.Tensor:
    """Router weights ``[tokens, experts]`` (float32) from sigmoid scores: an expert is chosen by ``sigmoid(logit) +
    correction`` (the choice score), weighted by ``sigmoid(logit)`` alone. The experts form ``groups`` equal groups of
    neighbours; a group's score is the sum of its two largest choice scores, and only experts of the ``keep`` best
    groups can be chosen. The weights of the ``top`` chosen experts are their scores over the sum of those scores (plus
    ``1e-20``) times ``scale``; every other weight is zero. ``logits [tokens, >= experts]`` float32."""
    _need(logits, torch.float32, "logits")
    tokens, ld = logits.shape
    if correction is not None:
        _need(correction, torch.float32, "correction")
        if correction.numel() != experts:
            raise ValueError("the router's correction needs one element per expert")
    out = _empty((tokens, experts), torch.float32, logits.device)
    fn = _fn("pointwise", "pkv_route_scored",
             [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(logits), ld, _ptr(correction), _ptr(out), tokens, experts, top, int(groups), int(keep), float(scale),
              _stream()), "route_scored")
    return out


def gated_bias_act(gate_up: torch.Tensor, up_at: int, n: int, gate_bias: torch.Tensor | None, up_bias: torch.Tensor | None,
                   act: str) -> torch.Tensor:
    """``act(gate + gate_bias) * (up + up_bias)`` ``[tokens, n]`` for rows that hold the ``n`` gate columns and, ``up_at``
    columns further on, the up columns; the biases are float32 ``[n]`` or none."""
    _need(gate_up, None, "gate_up")
    tokens, ld = gate_up.shape
    for name, t in (("gate_bias", gate_bias), ("up_bias", up_bias)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n:
                raise ValueError(f"{name} needs one element per column")
    if up_at < n or ld < up_at + n:
        raise ValueError("gated_bias_act: sizes do not fit")
    out = _empty((tokens, n), gate_up.dtype, gate_up.device)
    fn = _fn("pointwise", "pkv_gated_bias_act", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), dtype_code(gate_up.dtype), ld, int(up_at), _ptr(gate_bias), _ptr(up_bias), _ptr(out), tokens, n,
              ACTIVATIONS[act], _stream()), "gated_bias_act")
    return out


def pair_rows(hidden: torch.Tensor, delta: torch.Tensor | None, other: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``hidden += delta`` in place (with ``delta``), then ``[hidden | other]`` row by row in ``out_dtype``: the float32
    stream beside a second float32 matrix of its shape, as the operand of one product, ``[tokens, 2 width]``."""
    _need(hidden, torch.float32, "hidden"); _need(other, torch.float32, "other")
    if other.shape != hidden.shape:
        raise ValueError("the two matrices differ in shape")
    if delta is not None:
        _need(delta, None, "delta")
        if delta.shape != hidden.shape:
            raise ValueError("delta and hidden differ in shape")
    rows, cols = hidden.shape
    out = _empty((rows, 2 * cols), out_dtype, hidden.device)
    fn = _fn("pointwise", "pkv_pair_rows", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(fn(_ptr(hidden), _ptr(delta), dtype_code(delta.dtype) if delta is not None else 0, _ptr(other), _ptr(out),
              dtype_code(out_dtype), rows, cols, _stream()), "pair_rows")
    return out


def assign_bias(hidden: torch.Tensor, value: torch.Tensor, bias: torch.Tensor | None) -> None:
    """``hidden = value + bias`` (all float32; ``bias [width]`` or none): the stream takes a new value in place."""
    _need(hidden, torch.float32, "hidden"); _need(value, torch.float32, "value")
    if value.shape != hidden.shape:
        raise ValueError("value and hidden differ in shape")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != hidden.shape[1]:
            raise ValueError("bias does not fit the stream's width")
    fn = _fn("pointwise", "pkv_assign_bias", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(_ptr(hidden), _ptr(value), _ptr(bias), hidden.shape[0], hidden.shape[1], _stream()), "assign_bias")


def combine_pair(a: torch.Tensor, b: torch.Tensor, factor_a: float, factor_b: float,
                 norm_weights: tuple[torch.Tensor, torch.Tensor] | None = None, eps: float = 1e-6) -> torch.Tensor:
    """One update from two float32 updates of the same shape: ``factor_a * a + factor_b * b``, or, with ``norm_weights =
    (wa, wb)`` (float32 ``[width]``), each first divided by its root mean square over the row (``eps`` inside the root)
    and multiplied by its weight. Float32 ``[tokens, width]``."""
    _need(a, torch.float32, "a"); _need(b, torch.float32, "b")
    if a.shape != b.shape:
        raise ValueError("the two updates differ in shape")
    wa = wb = None
    if norm_weights is not None:
        wa, wb = norm_weights
        _need(wa, torch.float32, "norm weight"); _need(wb, torch.float32, "norm weight")
        if wa.numel() != a.shape[1] or wb.numel() != a.shape[1]:
            raise ValueError("a norm's weight does not fit the width")
    out = _empty(tuple(a.shape), torch.float32, a.device)
    fn = _fn("pointwise", "pkv_combine_pair", [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p, c_int,
                                                c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), float(factor_a), float(factor_b), float(eps), _ptr(out), a.shape[0], a.shape[1],
              _stream()), "combine_pair")
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor | None, heads: int, vdim: int, factor: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """``x[t, h * vdim + j] * sigmoid(gate[t, h]) * factor`` for ``x [tokens, heads * vdim]``: in place, or written to
    ``out`` (a view of the same type whose rows may have a stride); returns where the result lies. ``gate`` is a view
    ``[tokens, heads]`` of the type of ``x`` whose rows may have a stride, or none (the factor alone)."""
    _need(x, None, "x")
    tokens = x.shape[0]
    n = heads * vdim
    if x.shape[1] != n:
        raise ValueError("x must hold heads * vdim columns")
    gate_ld = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != x.dtype or gate.dim() != 2 or gate.shape != (tokens, heads) or gate.stride(1) != 1:
            raise ValueError("gate must be a [tokens, heads] view of the type of x with unit inner stride")
        gate_ld = gate.stride(0) if tokens > 1 else max(gate.stride(0), heads)
    if out is None:
        out = x
    elif not out.is_cuda or out.dtype != x.dtype or out.dim() != 2 or out.shape != (tokens, n) or out.stride(1) != 1:
        raise ValueError("out must be a [tokens, heads * vdim] view of the type of x with unit inner stride")
    out_ld = out.stride(0) if tokens > 1 else max(out.stride(0), n)
    fn = _fn("pointwise", "pkv_head_gate", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(x), c_void_p(gate.data_ptr() if gate is not None else 0), dtype_code(x.dtype), gate_ld,
              c_void_p(out.data_ptr()), out_ld, tokens, heads, vdim, float(factor), _stream()), "head_gate")
    return out


#: tokens of one entry up to which ``linear_attention`` walks them in a row, and its chunk sizes (as for ``lightning``)
LINEAR_ATTENTION_IN_A_ROW = 128
LINEAR_ATTENTION_CHUNK, LINEAR_ATTENTION_CHUNKS = 64, 64


def linear_attention_chunk(tokens: int, seqs: int) -> int:
    """Tokens per chunk for a step of ``tokens`` tokens in ``seqs`` entries: 0 when no entry can be longer than
    ``LINEAR_ATTENTION_IN_A_ROW``, else ``LINEAR_ATTENTION_CHUNK`` or, for very long steps, a multiple of 16 that keeps
    the working memory at about ``LINEAR_ATTENTION_CHUNKS`` states per head."""
    if tokens - (seqs - 1) <= LINEAR_ATTENTION_IN_A_ROW:
        return 0
    return max(LINEAR_ATTENTION_CHUNK, -(-tokens // (LINEAR_ATTENTION_CHUNKS * 16)) * 16)


def linear_attention(proj: torch.Tensor, offsets: dict[str, int], state: torch.Tensor, seq_starts: torch.Tensor,
                     state_slots: torch.Tensor, heads: int, dim: int, vdim: int, out_dtype: torch.dtype, *,
                     head_decay: torch.Tensor | None = None, decay_pre: torch.Tensor | None = None,
                     decay_bias: torch.Tensor | None = None, inv_tau: float = 1.0,
                     q_scale: float = 1.0, k_scale: float = 1.0, rot_dims: int = 0, freq: torch.Tensor | None = None,
                     positions: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, eps: float = 1e-6,
                     out_factor: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Linear attention with a matrix state per head over a ragged batch: ``S_t = diag(a_t) S_(t-1) + k_t v_t^T``, ``o_t
    = S_t^T q_t``. ``proj`` float32 ``[tokens, ld]`` holds q and k ``[heads, dim]``, v and the output gate's
    pre-activation ``[heads, vdim]`` at ``offsets`` ("q", "k", "v", "g"). The decay is either ``head_decay`` (float32
    ``[heads]``, one fixed number per head) or, with ``decay_pre`` (float32 ``[tokens, heads * dim]``, rows may have a
    stride), ``sigmoid(decay_pre + decay_bias) ** inv_tau`` per token and key coordinate. Queries and keys are first
    rotated in their first ``rot_dims`` coordinates (coordinate ``i`` with ``i + rot_dims / 2``, angle ``positions[t] *
    freq[i]``), then multiplied by ``q_scale`` / ``k_scale``. ``state`` float32 ``[slots, heads, vdim, dim]`` is read and
    brought up to date. Returns, per head, the outputs divided by their root mean square over ``vdim``, times
    ``norm_weight`` (float32 ``[vdim]`` or none), the SiLU of the gate and ``out_factor``: ``[tokens, heads * vdim]`` in
    ``out_dtype``, or written into ``out`` (a view of that shape whose rows may have a stride). The kernel prepares its
    inputs in place: the query and key columns of ``proj`` and all of ``decay_pre`` are overwritten."""
    _need(proj, torch.float32, "proj"); _need(state, torch.float32, "state")
    tokens, ld = proj.shape
    if state.shape[1:] != (heads, vdim, dim):
        raise ValueError("linear_attention: the state does not fit heads, dim and vdim")
    a_ld = 0
    if decay_pre is None:
        _need(head_decay, torch.float32, "head_decay")
        if head_decay.numel() != heads:
            raise ValueError("one decay per head")
    else:
        if not decay_pre.is_cuda or decay_pre.dtype != torch.float32 or decay_pre.dim() != 2 or decay_pre.stride(1) != 1 \
                or decay_pre.shape[0] != tokens or decay_pre.shape[1] < heads * dim:
            raise ValueError("decay_pre must be float32 [tokens, >= heads * dim] with unit inner stride")
        a_ld = decay_pre.stride(0) if tokens > 1 else max(decay_pre.stride(0), heads * dim)
    if decay_bias is not None:
        _need(decay_bias, torch.float32, "decay_bias")
        if decay_bias.numel() != heads * dim:
            raise ValueError("the decay's bias needs one element per head and key coordinate")
    if norm_weight is not None:
        _need(norm_weight, torch.float32, "norm_weight")
        if norm_weight.numel() != vdim:
            raise ValueError("the norm's weight needs one element per value coordinate")
    if rot_dims:
        _need(freq, torch.float32, "freq"); _need(positions, torch.int32, "positions")
        if freq.numel() != rot_dims // 2:
            raise ValueError("freq needs one element per rotated pair")
    seqs = seq_starts.numel() - 1
    n = heads * vdim
    if out is None:
        out = _empty((tokens, n), out_dtype, proj.device)
    elif not out.is_cuda or out.dtype != out_dtype or out.dim() != 2 or out.shape != (tokens, n) or out.stride(1) != 1:
        raise ValueError("out must be [tokens, heads * vdim] of out_dtype with unit inner stride")
    out_ld = out.stride(0) if tokens > 1 else max(out.stride(0), n)
    scratch = _empty((tokens, n), torch.float32, proj.device)
    chunk = linear_attention_chunk(tokens, seqs)
    chunk_state = _empty((tokens // chunk + seqs, heads, vdim, dim), torch.float32, proj.device) if chunk else None
    chunk_decay = _empty((tokens // chunk + seqs, heads, dim), torch.float32, proj.device) if chunk and decay_pre is not None else None
    fn = _fn("linear_attention", "pkv_linear_attention",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_float, c_float, c_int,
              c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(proj), ld, offsets["q"], offsets["k"], offsets["v"], offsets["g"],
              c_void_p(decay_pre.data_ptr() if decay_pre is not None else 0), a_ld, _ptr(decay_bias), float(inv_tau),
              _ptr(head_decay), float(q_scale), float(k_scale), int(rot_dims), _ptr(freq), _ptr(positions), _ptr(norm_weight),
              float(eps), float(out_factor), _ptr(state), _ptr(seq_starts), _ptr(state_slots), _ptr(scratch),
              c_void_p(out.data_ptr()), dtype_code(out_dtype), out_ld, tokens, seqs, heads, dim, vdim, chunk,
              _ptr(chunk_state), _ptr(chunk_decay), _stream()), "linear_attention")
    prepared = decay_pre is not None or rot_dims or q_scale != 1.0 or k_scale != 1.0
    ops.LAUNCHES["count"] += (3 if chunk else 1) + (1 if prepared else 0)
    return out
