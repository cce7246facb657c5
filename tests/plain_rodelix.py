"""A plain, slow implementation of the Rodelix design in float64, one function per mechanism.

It shares no code with the package: plain PyTorch on the CPU, whole sequences at once, no cache,
no state carried between calls (``lightning`` walks the tokens in a Python loop). The tests
compare the engine with it. ``tensors`` maps the names of a model folder to tensors; ``config`` is
the nested dictionary of ``config.json``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """Mean and variance over the last axis (variance = mean of squared deviations)."""
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * weight.to(F64) + bias.to(F64)


def rms_weighted(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(F64)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """``h_t + (h_{t-1} - h_t) * mix`` with zeros in front of the first token."""
    previous = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (previous - h) * mix.to(F64)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotate the first ``dims`` coordinates of the last axis of ``x [tokens, ..., n]``; coordinate
    ``2i`` pairs with ``2i + 1``, the angle is ``position * base^(-2i/dims)``."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    angle = (positions.to(F64)[:, None] * freq[None, :]).reshape(shape)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    scores = scores.masked_fill(~mask, -math.inf)
    return torch.softmax(scores, dim=-1)


def latent_attention(h: torch.Tensor, p: dict, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are expanded from one latent per position; one rotated key
    part serves all heads."""
    n = h.shape[0]
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(n)
    q = (h @ p["q"].to(F64).T).view(n, heads, dim + rot_dim)
    down = h @ p["dkv"].to(F64).T
    c = rms_weighted(down[:, :rank], p["dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rank:], positions, m["rot"]["dims"], m["rot"]["base"])        # [n, rot_dim]
    q_plain = q[:, :, :dim]
    q_rot = rotate_pairs(q[:, :, dim:], positions, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ p["uk"].to(F64).T).view(n, heads, dim)
    v = (c @ p["uv"].to(F64).T).view(n, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    causal = torch.arange(n)[None, :] <= torch.arange(n)[:, None]
    w = softmax_rows(scores, causal[None])
    out = torch.einsum("hij,jhd->ihd", w, v).reshape(n, heads * vdim)
    return out @ p["o"].to(F64).T


def window_attention(h: torch.Tensor, p: dict, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention over a sliding window: weighted unit-norm queries and keys, a
    temperature per head, and a bias that grows with the logarithm of the distance."""
    n = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_weighted((h @ p["q"].to(F64).T).view(n, heads, dim), p["q.norm"], eps)
    k = rms_weighted((h @ p["k"].to(F64).T).view(n, groups, dim), p["k.norm"], eps)
    v = (h @ p["v"].to(F64).T).view(n, groups, vdim)
    per = heads // groups
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    distance = (i - j).clamp(min=0).to(F64)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"] * p["temp"].to(F64)[:, None, None]
    scores = scores - p["r1"].to(F64)[:, None, None] * torch.log1p(p["r2"].to(F64)[:, None, None] * distance[None])
    mask = (j <= i)
    size = (m.get("mask") or {}).get("size")
    if size:
        mask = mask & (i - j < size)
    w = softmax_rows(scores, mask[None])
    out = torch.einsum("hij,jhd->ihd", w, v).reshape(n, heads * vdim)
    return out @ p["o"].to(F64).T


def lightning(h: torch.Tensor, p: dict, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, token by token: ``S <- decay S + k v^T``,
    ``o = S^T q``; the heads together are RMS-normed, gated and projected."""
    n = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].to(F64).T).view(n, heads, dim)
    k = silu(h @ p["k"].to(F64).T).view(n, heads, dim)
    v = silu(h @ p["v"].to(F64).T).view(n, heads, vdim)
    decay = torch.tensor(m["decay"], dtype=F64)
    state = torch.zeros((heads, dim, vdim), dtype=F64)
    outs = []
    for t in range(n):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", state, q[t]).reshape(heads * vdim))
    o = torch.stack(outs, dim=0)
    o = rms_weighted(o, p["norm"], eps) * torch.sigmoid(h @ p["g"].to(F64).T)
    return o @ p["o"].to(F64).T


def dense_relu_squared(h: torch.Tensor, p: dict) -> torch.Tensor:
    z = torch.relu(h @ p["up"].to(F64).T)
    return (z * z) @ p["down"].to(F64).T


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "lightning": lightning}


def layer_params(tensors: dict, prefix: str) -> dict:
    """The tensors under ``prefix`` with the prefix taken off, as float64."""
    return {name[len(prefix):]: t.to(F64) for name, t in tensors.items() if name.startswith(prefix)}


def run_order(config: dict) -> list[tuple[int, bool]]:
    """``(layer, starts a repeated pass)`` in run order."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for pass_no in range(times):
        order += [(i, pass_no > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


def layer(x: torch.Tensor, tensors: dict, index: int, spec: dict, config: dict) -> torch.Tensor:
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    pre = f"l{index}."
    t = {k: v.to(F64) for k, v in tensors.items() if k.startswith(pre)}
    h = layer_norm(x, t[pre + "norm1"], t[pre + "norm1.b"], eps)
    h = token_shift(h, t[pre + "shift"])
    update = MIXERS[spec["type"]](h, layer_params(tensors, pre + "mix."), spec["mixer"], eps)
    x = x + mult * layer_norm(update, t[pre + "norm1b"], t[pre + "norm1b.b"], eps)
    if spec.get("mlp"):
        h = layer_norm(x, t[pre + "norm2"], t[pre + "norm2.b"], eps)
        update = dense_relu_squared(h, layer_params(tensors, pre + "mlp."))
        x = x + mult * layer_norm(update, t[pre + "norm2b"], t[pre + "norm2b.b"], eps)
    return x


def forward(tensors: dict, config: dict, token_ids: list[int], return_layers: bool = False):
    """Logits ``[tokens, vocab]`` (float64) of one whole sequence; with ``return_layers`` also the
    residual stream after every layer run."""
    ids = torch.tensor(token_ids, dtype=torch.long)
    embedded = tensors["embed"].to(F64)[ids]
    x = embedded
    streams = []
    for index, restart in run_order(config):
        if restart:
            x = x + embedded
        x = layer(x, tensors, index, config["layers"][index], config)
        streams.append(x)
    eps = float(config["norm"]["eps"])
    y = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = y @ tensors["head"].to(F64).T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
