"""A plain, slow implementation of the Segetar design in float64 on the CPU, one function per mechanism.

It shares no code with the package: tensors come as a dict name -> torch tensor under the names of a model
folder, the configuration as the nested dict of ``config.json``. Everything is written token by token or as
dense matrices over a whole sequence, whichever is plainer.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def widen(tensors):
    return {k: (v.to(F) if v.is_floating_point() else v) for k, v in tensors.items()}


def under(tensors, prefix):
    """The tensors whose names begin with ``prefix``, with the prefix taken off."""
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def run_order(config):
    """(layer, number of the pass that starts in front of it or None) in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for number in range(loop["times"]):
        order += [(i, number if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], count)]


def angles(positions, dims, base):
    """[tokens, dims / 2]: position times base^(-2i / dims)."""
    i = torch.arange(dims // 2, dtype=F)
    return positions.to(F)[:, None] * base ** (-2.0 * i / dims)[None, :]


def rotate_neighbours(x, positions, dims, base):
    """x [tokens, heads, size]: coordinates 2i and 2i + 1 of the first ``dims`` turn together."""
    if not dims:
        return x
    a = angles(positions, dims, base)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * torch.cos(a) - odd * torch.sin(a)
    out[..., 1:dims:2] = odd * torch.cos(a) + even * torch.sin(a)
    return out


def rotate_halves(x, positions, dims, base):
    """x [tokens, heads, size]: coordinates i and i + dims / 2 of the first ``dims`` turn together."""
    if not dims:
        return x
    a = angles(positions, dims, base)[:, None, :]
    lo, hi = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.clone()
    out[..., :dims // 2] = lo * torch.cos(a) - hi * torch.sin(a)
    out[..., dims // 2:dims] = hi * torch.cos(a) + lo * torch.sin(a)
    return out


def window_attention(h, p, m, eps, positions, full):
    """The attention side of a two-sided mixer. ``full``: biases, rotation of neighbours, a gate per head."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if full:
        q, k, v = q + p["q.b"], k + p["k.b"], v + p["v.b"]
    q = unit_rms(q, eps) * p["q.norm"]                   # over all heads at once
    k = unit_rms(k, eps) * p["k.norm"]
    q, k, v = q.view(n, H, D), k.view(n, G, D), v.view(n, G, V)
    rot = m.get("rot") or {}
    if full and rot.get("dims"):
        q = rotate_neighbours(q, positions, rot["dims"], rot["base"])
        k = rotate_neighbours(k, positions, rot["dims"], rot["base"])
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    size = (m.get("mask") or {}).get("size")
    if size is not None:
        seen = seen & (distance < size)
    out = torch.zeros((n, H, V), dtype=F)
    for head in range(H):
        kv = head // (H // G)
        score = (q[:, head] @ k[:, kv].T) * m["scale"]
        weights = torch.softmax(score.masked_fill(~seen, float("-inf")), dim=-1)
        out[:, head] = weights @ v[:, kv]
    if full:
        out = out * torch.sigmoid(h @ p["g"].T)[:, :, None]
    return out.reshape(n, H * V) @ p["o"].T


def matrix_state_scan(q, k, v, decay):
    """q, k [tokens, heads, D], v [tokens, heads, V], decay [tokens, heads, D]: the state S [heads, D, V] starts at
    zero; every token first shrinks row d of S by decay[d], then adds k v^T, then reads S^T q."""
    n, H, D = q.shape
    S = torch.zeros((H, D, v.shape[-1]), dtype=F)
    out = torch.zeros((n, H, v.shape[-1]), dtype=F)
    for t in range(n):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def gated_linear_attention(h, p, m, eps):
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(n, H, D) / math.sqrt(D)
    k = (h @ p["k"].T).view(n, H, D)
    v = (h @ p["v"].T).view(n, H, V)
    decay = torch.sigmoid((h @ p["a1"].T) @ p["a2"].T + p["a2.b"]) ** (1.0 / m["tau"])
    o = matrix_state_scan(q, k, v, decay.view(n, H, D))
    o = unit_rms(o, eps) * p["norm"]
    return (o.reshape(n, H * V) * silu(h @ p["g"].T)) @ p["o"].T


def retention(h, p, m, eps, positions):
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(n, H, D)
    k = (h @ p["k"].T).view(n, H, D)
    v = (h @ p["v"].T).view(n, H, V)
    rot = m.get("rot") or {}
    if rot.get("dims"):
        q = rotate_halves(q, positions, rot["dims"], rot["base"])
        k = rotate_halves(k, positions, rot["dims"], rot["base"])
    k = k / math.sqrt(D)
    decay = torch.tensor(m["decay"], dtype=F)[None, :, None].expand(n, H, D)
    o = unit_rms(matrix_state_scan(q, k, v, decay), eps)
    return (o.reshape(n, H * V) * silu(h @ p["g"].T)) @ p["o"].T


def two_sided(h, p, kind, m, eps, positions):
    left = window_attention(h, under(p, "left."), m["left"], eps, positions, full=kind == "parallel")
    if kind == "parallel":
        right = gated_linear_attention(h, under(p, "right."), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    right = retention(h, under(p, "right."), m["right"], eps, positions)
    return 0.5 * (unit_rms(left, eps) * p["left.out"] + unit_rms(right, eps) * p["right.out"])


def mamba(h, p, m):
    n = h.shape[0]
    inner, N, rank, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    both = h @ p["in"].T
    x, z = both[:, :inner], both[:, inner:]
    padded = torch.cat([torch.zeros((taps - 1, inner), dtype=F), x])
    x = silu(sum(padded[j:j + n] * p["conv"][:, j] for j in range(taps)) + p["conv.b"])
    low = x @ p["x"].T
    dt = torch.nn.functional.softplus(low[:, :rank] @ p["dt"].T + p["dt.b"])
    B, C = low[:, rank:rank + N], low[:, rank + N:rank + 2 * N]
    A = -torch.exp(p["A_log"])
    S = torch.zeros((inner, N), dtype=F)
    y = torch.zeros((n, inner), dtype=F)
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + p["D"] * x[t]
    return (y * silu(z)) @ p["o"].T


def dense_feed_forward(h, p):
    return (gelu_tanh(h @ p["gate"].T + p["gate.b"]) * (h @ p["up"].T + p["up.b"])) @ p["down"].T + p["down.b"]


def router_weights(h, p, router):
    """[tokens, experts]: zero but for the chosen experts."""
    E, top = router["experts"], router["top"]
    score = torch.sigmoid(h @ p["router"].T)
    choice = score + p["correction"]
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"]:
        per = E // groups["count"]
        grouped = choice.view(-1, groups["count"], per)
        group_score = grouped.topk(min(2, per), dim=-1).values.sum(dim=-1)
        kept = torch.zeros_like(group_score, dtype=torch.bool)
        kept.scatter_(1, group_score.topk(groups["keep"], dim=-1).indices, True)
        choice = grouped.masked_fill(~kept[:, :, None], float("-inf")).reshape(-1, E)
    chosen = choice.topk(top, dim=-1).indices
    picked = score.gather(1, chosen)
    picked = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * router.get("scale", 1.0)
    return torch.zeros_like(score).scatter_(1, chosen, picked)


def expert_mixture(h, p, mlp):
    weights = router_weights(h, p, mlp["router"])
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows = weights[:, e] != 0
        if rows.any():
            x = h[rows]
            y = (silu(x @ p[f"e{e}.gate"].T) * (x @ p[f"e{e}.up"].T)) @ p[f"e{e}.down"].T
            out[rows] += weights[rows, e][:, None] * y
    return out


def forward(tensors, config, tokens, return_layers=False):
    """Logits [tokens, vocab] of one sequence from position 0 (and the stream after every layer run)."""
    w = widen(tensors)
    eps = config["norm"]["eps"]
    positions = torch.arange(len(tokens))
    first = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    x = first
    streams = []
    for index, number in run_order(config):
        if number is not None:
            x = torch.cat([x, first], dim=-1) @ w["loop.in"].T + w["loop.step"][number]
        layer = config["layers"][index]
        p = under(w, f"l{index}.")
        h = unit_rms(x, eps) * p["norm1"]
        if layer["type"] == "mamba1":
            x = x + mamba(h, under(p, "mix."), layer["mixer"])
        else:
            x = x + two_sided(h, under(p, "mix."), layer["type"], layer["mixer"], eps, positions)
        mlp = layer.get("mlp")
        if mlp:
            h = unit_rms(x, eps) * p["norm2"]
            x = x + (dense_feed_forward(h, under(p, "mlp.")) if mlp.get("kind", "dense") == "dense"
                     else expert_mixture(h, under(p, "mlp."), mlp))
        streams.append(x)
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, streams) if return_layers else logits
