"""Prefill and decode throughput of one architecture at layer sizes of a real model (random
weights), with the time of every kernel of a step against its roofline. ``bench.py --design``
runs it for the Revupel, the Tiburax, the Rodelix or the Segetar design and, at equal sizes, for the models it is compared with.

A step runs through ``ModelRunner.step``. For the kernel table one eager step is run with every
kernel call of ``ops`` / ``ops.mixer_ops`` and every library product bracketed by CUDA events on
the launching stream; a kernel's roofline time is the larger of its bytes over the measured copy
bandwidth (its tensor arguments and results, or for attention the cache it must read) and its
flops over the measured matrix peak.
"""

from __future__ import annotations

import numpy as np
import torch

__all__ = ["RODELIX_SIZES", "SEGETAR_SIZES", "SIZES", "TIBURAX_SIZES", "llama_like", "measure", "revupel_config", "rodelix_config",
           "segetar_config", "tiburax_config"]

#: name -> sizes of a Revupel model whose layers resemble a served model's (latent attention of
#: the kind with a compressed cache, an mLSTM block, eight experts of which two run, a dense block)
SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=256, m_heads=4, m_dim=256,
               m_vdim=512, ff=8192, experts=8, top=2, expert_ff=2048, shared_ff=2048, vocab=32000, side=64, pairs=2),
    "7b": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512, m_heads=8, m_dim=256,
               m_vdim=512, ff=14336, experts=8, top=2, expert_ff=3584, shared_ff=3584, vocab=32000, side=64, pairs=2),
}


def revupel_config(size: str) -> dict:
    z = SIZES[size]
    attention = {"type": "latent_attention", "mixer": {
        "heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "q_rank": z["q_rank"],
        "kv_rank": z["kv_rank"], "scale": (z["dim"] + z["rot_dim"]) ** -0.5, "rot": {"base": 10000.0, "dims": z["rot_dim"]}}}
    recurrent = {"type": "mlstm", "mixer": {"heads": z["m_heads"], "dim": z["m_dim"], "vdim": z["m_vdim"], "gate_cap": 15.0}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    dense = {"kind": "dense", "ff": z["ff"]}
    layers = []
    for _ in range(z["pairs"]):
        layers += [{**attention, "mlp": moe}, {**recurrent, "mlp": dense}]
    return {"architecture": "Revupel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "token_side": {"dim": z["side"]}, "layers": layers}


#: name -> sizes of a Tiburax model at the same width, layer count and expert sizes: attention over
#: a window with kept first tokens (grouped keys, heads of 128), a Mamba block with 16 state
#: coordinates per channel, eight gated experts of which two run beside a shared one
TIBURAX_SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep=4, inner=4096, state=16, dt_rank=128,
               experts=8, top=2, expert_ff=2048, shared_ff=2048, vocab=32000, pairs=2),
    "7b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, keep=4, inner=8192, state=16, dt_rank=256,
               experts=8, top=2, expert_ff=3584, shared_ff=3584, vocab=32000, pairs=2),
}


def tiburax_config(size: str) -> dict:
    z = TIBURAX_SIZES[size]
    attention = {"type": "attention", "mixer": {
        "heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
        "softcap": 30.0, "v_mix": True, "mask": {"size": z["window"], "keep_first": z["keep"]},
        "rot": {"base": 10000.0, "dims": z["dim"], "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}}
    recurrent = {"type": "mamba1", "mixer": {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": 4}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    layers = []
    for _ in range(z["pairs"]):
        layers += [{**attention, "mlp": moe}, {**recurrent, "mlp": moe}]
    return {"architecture": "Tiburax", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": float(z["width"]) ** 0.5}, "layers": layers}


#: name -> sizes of a Rodelix model at the same width and layer count: attention over a cached latent,
#: linear attention with a decay per head (heads of 128 by 128), grouped-query attention over a
#: window of 1,024 (heads of 128), dense feed-forwards
RODELIX_SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, rot_dim=64, vdim=128, kv_rank=256, window=1024, l_heads=16, l_dim=128,
               l_vdim=128, ff=8192, vocab=32000),
    "7b": dict(width=4096, heads=32, kv_heads=8, dim=128, rot_dim=64, vdim=128, kv_rank=512, window=1024, l_heads=32, l_dim=128,
               l_vdim=128, ff=14336, vocab=32000),
}


def rodelix_config(size: str) -> dict:
    z = RODELIX_SIZES[size]
    latent = {"type": "latent_attention", "mixer": {
        "heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
        "scale": (z["dim"] + z["rot_dim"]) ** -0.5, "rot": {"base": 10000.0, "dims": z["rot_dim"]}}}
    window = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                                             "scale": z["dim"] ** -0.5, "mask": {"size": z["window"]}}}
    decays = [1.0 - 2.0 ** (-5.0 - 3.0 * a / max(z["l_heads"] - 1, 1)) for a in range(z["l_heads"])]
    linear = {"type": "lightning", "mixer": {"heads": z["l_heads"], "dim": z["l_dim"], "vdim": z["l_vdim"], "decay": decays}}
    dense = {"kind": "dense", "ff": z["ff"]}
    layers = [{**latent, "mlp": dense}, {**linear, "mlp": dense}, {**window, "mlp": dense}, {**linear, "mlp": dense}]
    return {"architecture": "Rodelix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_softcap": 30.0, "layers": layers}


#: name -> sizes of a Segetar model at the same width and layer count: a Mamba block, window attention (grouped keys,
#: heads of 128, window 1,024) beside gated linear attention (keys of 128, values of 256), window attention beside
#: retention, a Mamba block again; a dense gated feed-forward and eight gated experts of which two run, chosen within
#: two of four groups; the four layers are one span with a pass input in front
SEGETAR_SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, r_heads=8, r_dim=128, r_vdim=256, rank=16,
               inner=4096, state=16, dt_rank=128, ff=5632, experts=8, top=2, expert_ff=2048, vocab=32000),
    "7b": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, r_heads=16, r_dim=128, r_vdim=256, rank=32,
               inner=8192, state=16, dt_rank=256, ff=9728, experts=8, top=2, expert_ff=3584, vocab=32000),
}


def segetar_config(size: str) -> dict:
    z = SEGETAR_SIZES[size]

    def attention(rotated: bool) -> dict:
        side = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                "mask": {"size": z["window"]}}
        if rotated:
            side["rot"] = {"base": 1000000.0, "dims": z["dim"]}
        return side

    decays = [1.0 - 2.0 ** (-5.0 - 3.0 * a / max(z["r_heads"] - 1, 1)) for a in range(z["r_heads"])]
    gated = {"type": "parallel", "mixer": {
        "left": attention(True), "right": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"], "tau": 8.0, "rank": z["rank"]},
        "left_scale": 1.0, "right_scale": 0.7}}
    retentive = {"type": "parallel_2", "mixer": {
        "left": attention(False), "right": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"], "decay": decays,
                                            "rot": {"base": 10000.0, "dims": z["r_dim"]}}}}
    recurrent = {"type": "mamba1", "mixer": {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": 4}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    dense = {"kind": "dense", "ff": z["ff"]}
    layers = [{**recurrent, "mlp": dense}, {**gated, "mlp": moe}, {**retentive, "mlp": moe}, {**recurrent, "mlp": moe}]
    return {"architecture": "Segetar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "loop": {"start": 0, "stop": len(layers), "times": 1}, "layers": layers}


def llama_like(size: str) -> dict:
    """The Llama-style decoder at the same width, layer count and head count; its gated
    feed-forward has the parameter count of the dense block above."""
    z = SIZES[size]
    return {"architecture": "LlamaToyDecoder", "vocab_size": z["vocab"], "d_model": z["width"], "n_layers": 2 * z["pairs"],
            "n_heads": z["heads"], "n_kv_heads": max(1, z["heads"] // 4), "head_dim": 128, "d_ff": z["ff"] * 2 // 3 // 128 * 128,
            "max_seq_len": 8192, "rope_theta": 10000.0, "norm_eps": 1e-6, "tie_embeddings": False}


def _bytes_of(values) -> int:
    return sum(v.numel() * v.element_size() for v in values if isinstance(v, torch.Tensor))


class _KernelTimes:
    """Brackets every kernel call of a step with CUDA events."""

    def __init__(self, attention_cost) -> None:
        self.records: list = []
        self.attention_cost = attention_cost
        self._undo: list = []

    def _wrap(self, owner, name, kind):
        original = getattr(owner, name)

        def timed(*args, **kwargs):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = original(*args, **kwargs)
            stop.record()
            outs = out if isinstance(out, (tuple, list)) else (out,)
            moved, flops = _bytes_of(args) + _bytes_of(outs), 0.0
            if kind == "product":
                a, b = args[0], args[1]
                flops = 2.0 * a.numel() * b.shape[-1]
            elif name in self.attention_cost:
                moved, flops = self.attention_cost[name](tuple(args) + (kwargs,), out)     # (keyword arguments ride last)
            self.records.append((name, start, stop, moved, flops))
            return out

        setattr(owner, name, timed)
        self._undo.append((owner, name, original))

    def __enter__(self):
        from paged_kv_serving_b200 import ops
        from paged_kv_serving_b200.ops import gemm, mixer_ops

        for name in ("embedding_gather", "add_rmsnorm", "silu_mul", "rope_kv_store", "attention_prefill_tcgen05",
                     "attention_prefill_bf16", "attention_decode_tma", "attention_decode_flat", "attention_decode_bf16",
                     "gemm_small_m", "gemm_tcgen05", "finish_norm"):
            self._wrap(ops, name, "kernel")
        for name in ("bias_act", "residual_add", "act_times_table", "route_top", "expert_act", "conv_residual", "mlstm",
                     "latent_prepare", "latent_attention", "latent_attention_mma", "norm_residual", "expert_gated_act",
                     "qkv_prepare", "attention_sink", "attention_sink_mma", "selective_scan", "layer_norm_step", "token_shift",
                     "lightning", "softcap", "linear_attention", "route_scored", "gated_bias_act", "pair_rows", "assign_bias",
                     "combine_pair", "head_gate"):
            self._wrap(mixer_ops, name, "kernel")
        self._wrap(gemm, "matmul", "product")
        self._wrap(torch, "bmm", "product")
        return self

    def __exit__(self, *exc):
        for owner, name, original in reversed(self._undo):
            setattr(owner, name, original)

    def table(self, peaks: dict) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, start, stop, moved, flops in self.records:
            row = out.setdefault(name, {"calls": 0, "ms": 0.0, "roofline_ms": 0.0})
            row["calls"] += 1
            row["ms"] += start.elapsed_time(stop)
            row["roofline_ms"] += 1e3 * max(moved / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12))
        for row in out.values():
            row["of_roofline"] = round(row["roofline_ms"] / row["ms"], 4) if row["ms"] > 0 else None
            row["ms"], row["roofline_ms"] = round(row["ms"], 4), round(row["roofline_ms"], 4)
        return out


def measure(config: dict, peaks: dict, *, prefill_tokens: int = 2048, batch: int = 8, context: int = 1024, steps: int = 32,
            warmup: int = 4) -> dict:
    """Prefill (one prompt in one step) and decode (``batch`` requests with ``context`` cached
    tokens, one token each a step, captured graph) of a random-weights model of ``config``."""
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
    from paged_kv_serving_b200.engine.runner import ModelRunner
    from paged_kv_serving_b200.models.decoder import DecoderModel

    arch = registry.architecture(config["architecture"])
    typed = getattr(arch, "config_class", None)
    if typed is None:
        from paged_kv_serving_b200.config import ModelConfig as typed
    model = DecoderModel.from_random(typed.from_dict(config), seed=0, dtype="bfloat16", device="cuda:0")
    block = 16
    room = warmup + steps + 8
    pages_per_seq = -(-(context + 2 * room + 64) // block)
    prefill_pages = -(-prefill_tokens // block)
    runner = ModelRunner(model, num_blocks=batch * pages_per_seq + prefill_pages, block_size=block, max_running_seqs=batch + 1)
    groups = len(runner.groups)
    rng = np.random.default_rng(0)
    vocab = model.layout.vocab_size
    has_state = runner.num_state_slots > 0

    def entry(name, ids, first, table, want, slot):
        return BatchEntry(name, tuple(int(t) for t in ids), first, tuple(table for _ in range(groups)), want,
                          slot if has_state else None)

    def timed(fn, repeat):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for i in range(repeat):
            fn(i)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / repeat

    # attention's algorithmic cost, from the sizes of the step at hand
    cost = {}
    shape = {"tokens": 0, "keys": 0.0}

    def window_keys(window: int, keep: int) -> float:
        """(query, key) pairs a window with kept first tokens lets through, for the step at hand."""
        if shape["tokens"] == shape["cache_tokens"]:              # one prompt from position 0
            n = shape["tokens"]
            if not window or window >= n:
                return n * (n + 1) / 2.0
            return window * (window + 1) / 2.0 + (n - window) * float(window + keep)
        per_row = shape["cache_tokens"] / max(shape["tokens"], 1)
        return shape["tokens"] * float(min(per_row, window + keep) if window else per_row)

    def latent_cost(args, out):
        heads, rank = out.shape[0], out.shape[2]
        dk = args[4].shape[-1]
        flops = 2.0 * heads * shape["keys"] * (dk + rank)
        moved = shape["cache_tokens"] * dk * 2 + _bytes_of((args[0], out))
        return moved, flops

    def llama_prefill_cost(args, out):
        heads, hd, window, keep = args[9], args[11], args[13], args[-1].get("keep_first", 0)
        return _bytes_of((args[0], out)), 4.0 * heads * hd * window_keys(window, keep)

    def llama_decode_cost(args, out):
        kv, hd, window, keep = args[10], args[11], args[13], args[-1].get("keep_first", 0)
        pairs = window_keys(window, keep)
        return pairs * kv * hd * 2 * 2 + _bytes_of((args[0], out)), 4.0 * args[9] * hd * pairs

    def mlstm_cost(args, out):
        heads, dim, vdim = args[13], args[14], args[15]
        return _bytes_of((args[0], out)) * 2, 4.0 * args[0].shape[0] * heads * dim * vdim

    def sink_cost(args, out):
        # attention_sink(q, k_pool, v_pool, table, starts, first, work_seq, work_row0, H, G, dim, vdim, page, window, keep, ...)
        heads, groups, dim, vdim, window, keep = args[8], args[9], args[10], args[11], args[13], args[14]
        pairs = window_keys(window, keep)
        cached = shape["cache_tokens"]                            # a prompt reads every key of its cache once
        if shape["tokens"] != shape["cache_tokens"]:
            per_row = shape["cache_tokens"] / max(shape["tokens"], 1)
            cached = shape["tokens"] * (min(per_row, window + keep) if window else per_row)
        moved = cached * groups * (dim + vdim) * 2 + out.numel() * out.element_size() * 2
        return moved, 2.0 * heads * (dim + vdim) * pairs

    def scan_cost(args, out):
        # per token and channel: 2 state updates and sums per state coordinate on the float32 pipe; bytes: x, z, dt, out
        x, dt_pre, a = args[0], args[2], args[7]
        moved = x.numel() * (2 * x.element_size() + 4) + out.numel() * out.element_size()
        return moved, 0.0

    def lightning_cost(args, out):
        # lightning(proj, offsets, decay, norm_weight, eps, state, starts, slots, heads, dim, vdim, out_dtype)
        heads, dim, vdim = args[8], args[9], args[10]
        return _bytes_of((args[0], out)) + out.numel() * 8, 4.0 * args[0].shape[0] * heads * dim * vdim

    def linear_attention_cost(args, out):
        # linear_attention(proj, offsets, state, starts, slots, heads, dim, vdim, out_dtype, ...)
        heads, dim, vdim = args[5], args[6], args[7]
        return _bytes_of((args[0], out)) + out.numel() * 8, 4.0 * args[0].shape[0] * heads * dim * vdim

    cost["linear_attention"] = linear_attention_cost
    cost["lightning"] = lightning_cost
    cost.update({"attention_sink": sink_cost, "attention_sink_mma": sink_cost, "selective_scan": scan_cost})
    cost.update({"latent_attention": latent_cost, "latent_attention_mma": latent_cost,
                 "attention_prefill_tcgen05": llama_prefill_cost, "attention_prefill_bf16": llama_prefill_cost,
                 "attention_decode_tma": llama_decode_cost, "attention_decode_flat": llama_decode_cost,
                 "attention_decode_bf16": llama_decode_cost, "mlstm": mlstm_cost})

    # ---- prefill ---------------------------------------------------------------------------------
    table = tuple(range(batch * pages_per_seq, batch * pages_per_seq + prefill_pages))
    prompt = rng.integers(0, vocab, size=prefill_tokens)
    prefill_batch = ExecutionBatch((entry("p", prompt, 0, table, (prefill_tokens - 1,), batch),))
    for _ in range(3):
        runner.step(prefill_batch, clear_state_slots=[batch] if has_state else None)
    prefill_ms = timed(lambda i: runner.step(prefill_batch, clear_state_slots=[batch] if has_state else None), 3)
    shape.update(tokens=prefill_tokens, keys=prefill_tokens * (prefill_tokens + 1) / 2.0, cache_tokens=prefill_tokens)
    with _KernelTimes(cost) as times:
        runner.step(prefill_batch, clear_state_slots=[batch] if has_state else None)
    prefill_kernels = times.table(peaks)

    # ---- decode ----------------------------------------------------------------------------------
    tables = [tuple(j * batch + i for j in range(pages_per_seq)) for i in range(batch)]
    ids = rng.integers(0, vocab, size=(batch, context + 2 * room + 64))
    for i in range(batch):
        runner.step(ExecutionBatch((entry(f"s{i}", ids[i, :context], 0, tables[i], (), i),)),
                    clear_state_slots=[i] if has_state else None)

    def one(k, offset=0):
        position = context + offset + k
        runner.step(ExecutionBatch(tuple(entry(f"s{i}", (ids[i, position],), position, tables[i], (0,), i)
                                         for i in range(batch))))

    for k in range(warmup):
        one(k)
    decode_ms = timed(lambda k: one(k, warmup), steps)
    position = context + warmup + steps
    shape.update(tokens=batch, keys=float(batch * (position + 1)), cache_tokens=batch * (position + 1))
    runner.use_graphs = False
    with _KernelTimes(cost) as times:
        one(0, warmup + steps)
    decode_kernels = times.table(peaks)
    weight_bytes = model.weight_bytes_read_per_step()
    cache_bytes_per_token = sum((2 if g.values else 1) * len(g.entries) * g.n_kv_heads * g.head_dim * 2 for g in runner.groups)
    step_bytes = weight_bytes + batch * position * cache_bytes_per_token
    return {
        "parameters": model.layout.parameter_count(),
        "prefill": {"tokens": prefill_tokens, "ms": round(prefill_ms, 3), "tok_s": round(prefill_tokens / (prefill_ms / 1e3)),
                    "kernels": prefill_kernels},
        "decode": {"batch": batch, "context": context, "ms_per_step": round(decode_ms, 4),
                   "tok_s": round(batch / (decode_ms / 1e3)), "step_bytes": step_bytes,
                   "of_copy_bandwidth": round(step_bytes / (decode_ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4),
                   "kernels_eager": decode_kernels},
    }
