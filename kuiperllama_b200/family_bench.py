"""`bench.py --family fobolorn | kikunex | vurazen | bukuvik`: prefill and decode throughput of a batched family (sequence-batch
engine) at sizes that resemble a real model's layers, random weights, beside the closest existing model at equal width,
heads, active feed-forward size and number of layer runs: Fobolorn beside the Llama family of the single-sequence decoder,
Kikunex beside Fobolorn, Vurazen beside Kikunex, Bukuvik beside Vurazen.

What is timed.  A step is the call a server makes: kllm_seq_step() with token ids in host memory and the greedy ids
read back to host memory, blocking -- so every number here is end to end.  Between timed steps a buffer larger than
L2 is written.  Per-phase device times come from the engine's own events (kllm_seq_profile) in a separate step.
Roofline fractions use MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16) and say which.

Like kernels side by side (same shapes, CUDA events, L2 flushed):
   token-block product   kllm_seq_gemm bf16 (tcgen05 kind::f16)   vs   kllm_gemm_tf32 (tcgen05 kind::tf32)
   one-row product       kllm_seq_gemm, 1 token (rows kernel)     vs   kllm_gemv_f32
"""
from __future__ import annotations

import json
import statistics
import time
from pathlib import Path

from .sequence import BF16, BukuvikShape, F32, FobolornShape, KikunexShape, SeqEngine, VurazenShape, load_seq_library

ROOT = Path(__file__).resolve().parent.parent

SIZES = {
    # width 1024: 16 heads of 64 over 4 kv heads, 16 experts of 512 (2 active) + shared 1024; 4 layers, 2 of them twice
    "s": FobolornShape("fobolorn-s", 1024, 32000, 4, (1, 3, 2), 16, 4, 64, 64, 16, 2, 512, 1024),
    # width 2048: 16 heads of 128 over 4 kv heads, 32 experts of 768 (4 active) + shared 2048
    "m": FobolornShape("fobolorn-m", 2048, 32000, 4, (1, 3, 2), 16, 4, 128, 128, 32, 4, 768, 2048),
    "debug": FobolornShape("fobolorn-debug", 256, 4096, 3, (1, 3, 2), 4, 2, 64, 64, 8, 2, 128, 256),
}


_KP = (("lightning", "dense"), ("latent", "moe"), ("lightning", "moe"), ("latent", "moe"))
KIKUNEX_SIZES = {
    # the sizes of SIZES, layer for layer: same width, head counts, experts and layer runs; latent attention with a
    # key/value rank of two head sizes and a window of a quarter of the prompt, linear attention with square states
    "s": KikunexShape("kikunex-s", 1024, 32000, _KP, (1, 3, 2), 16, 64, 32, 64, 384, 128, 512, 16, 64, 64, 2048, 16, 2, 512),
    "m": KikunexShape("kikunex-m", 2048, 32000, _KP, (1, 3, 2), 16, 128, 64, 128, 768, 256, 512, 16, 128, 128, 4096, 32, 4, 768),
    "debug": KikunexShape("kikunex-debug", 256, 4096, _KP[:3], (1, 3, 2), 4, 32, 16, 32, 96, 64, 96, 4, 32, 32, 512, 8, 2, 128),
}


_VP = (("mamba", "dense"), ("parallel", "moe"), ("lightning", "moe"), ("parallel", "moe"))
VURAZEN_SIZES = {
    # the sizes of KIKUNEX_SIZES, layer for layer: same width, experts and layer runs; a selective scan of twice the width
    # with 16 states, window attention of the same heads over 4 key heads (window 512, 4 kept tokens) beside a delta rule
    # with square states, the same linear attention, gated dense layers and experts with a shared expert
    "s": VurazenShape("vurazen-s", 1024, 32000, _VP, (1, 3, 2), 2048, 16, 64, 16, 64, 64, 16, 4, 64, 512, 4, 32,
                      16, 16, 64, 64, 64, 2048, 16, 2, 512, 1024),
    "m": VurazenShape("vurazen-m", 2048, 32000, _VP, (1, 3, 2), 4096, 16, 128, 16, 128, 128, 16, 4, 128, 512, 4, 64,
                      16, 16, 128, 128, 128, 4096, 32, 4, 768, 2048),
    "debug": VurazenShape("vurazen-debug", 256, 4096, _VP[:3], (1, 3, 2), 512, 8, 16, 4, 32, 32, 4, 2, 32, 96, 2, 16,
                          4, 2, 32, 32, 16, 512, 8, 2, 128, 256),
}


def _bp(ff):
    return (("parallel", ff), ("attention", ff), ("attention", ff), ("parallel", ff), ("parallel", ff), ("attention", ff))


BUKUVIK_SIZES = {
    # the sizes of VURAZEN_SIZES: same width, head counts and number of layer runs (six layers, none looped); differential
    # attention with 16 heads of 2 x 64 (values 128) over 4 key heads and a window of 1024; in the pair a unit-normed
    # attention with the window of Vurazen's (512, 4 kept tokens) beside a duality mixer as wide as Vurazen's scan
    # (inner = 2 x width) with heads of 64 and 128 states; dense feed-forwards of 4 x width
    "s": BukuvikShape("bukuvik-s", 1024, 32000, _bp(4096), 16, 4, 64, 128, 1024, 32, 16, 4, 64, 64, 512, 4, 32,
                      32, 64, 128, 2, 2),
    "m": BukuvikShape("bukuvik-m", 2048, 32000, _bp(8192), 16, 4, 128, 128, 1024, 64, 16, 4, 128, 128, 512, 4, 64,
                      64, 64, 128, 2, 2),
    "debug": BukuvikShape("bukuvik-debug", 256, 4096, _bp(512)[:3], 4, 2, 32, 64, 96, 16, 4, 2, 32, 32, 64, 2, 16,
                          8, 32, 16, 2, 2),
}


def bukuvik_costs(shape, prompt_len):
    """FLOPs of a prompt step by phase class of the engine's profile."""
    W, T = shape.width, prompt_len
    n_att = sum(1 for m, _ in shape.pattern if m == "attention")
    n_par = shape.layers - n_att

    def pairs(window, keep):
        win = min(window, T)
        return T * win - win * (win - 1) / 2 + max(0, T - win) * keep
    # two maps per head, each with its own scores and its own weighted sum of the values
    attn_diff = 2 * pairs(shape.window, 0) * 2 * shape.heads * (shape.dim + shape.vdim)
    attn_left = 2 * pairs(shape.l_window, shape.l_keep_first) * shape.l_heads * (shape.l_dim + shape.l_vdim)
    # per token, head and state element: decay, update, read-out (multiply-adds)
    attn_right = T * shape.s_heads * 6 * shape.s_vdim * shape.s_state
    return {"in_proj": 2 * T * W * (n_att * shape.n_in("attention") + n_par * (shape.n_in("left") + shape.n_in("right"))),
            "attention": n_att * attn_diff + n_par * (attn_left + attn_right),
            "out_proj": 2 * T * W * (n_att * shape.n_out("attention") + n_par * (shape.n_out("left") + shape.n_out("right"))),
            "experts": 2 * T * sum(2 * (f or 0) * W for _, f in shape.pattern),
            "head": 2 * shape.vocab * W}


def bukuvik_decode_bytes(shape, B, ctx, es):
    """Bytes a decode step must move, by phase class: weights once per step, the windows' keys and values, the states."""
    W = shape.width
    n_att = sum(1 for m, _ in shape.pattern if m == "attention")
    n_par = shape.layers - n_att
    return {"in_proj": (n_att * shape.n_in("attention") + n_par * (shape.n_in("left") + shape.n_in("right"))) * W * es,
            "out_proj": (n_att * shape.n_out("attention") + n_par * (shape.n_out("left") + shape.n_out("right"))) * W * es,
            "experts": sum(2 * (f or 0) * W for _, f in shape.pattern) * es,
            "attention": shape.state_bytes_per_step(B, ctx, es), "head": shape.vocab * W * es}


def vurazen_costs(shape, prompt_len):
    """FLOPs of a prompt step by phase class of the engine's profile."""
    W, T = shape.width, prompt_len
    runs = [shape.pattern[i] for i, _, _ in shape.run_order()]
    n = {k: sum(1 for m, _ in runs if m == k) for k in ("mamba", "lightning", "parallel")}
    win = min(shape.window, T)
    pairs = T * win - win * (win - 1) / 2 + max(0, T - win) * shape.keep_first
    attn_left = 2 * pairs * shape.heads * 2 * shape.dim
    # per token and head of the delta rule: decay, prediction, update and read-out over a dim x vdim state; its low-rank
    # decay and gate projections; per token and channel of the scan: the step size and 3 multiply-adds per state
    attn_right = T * shape.d_heads * (8 * shape.d_dim * shape.d_vdim + 2 * shape.d_rank * (shape.d_dim + shape.d_vdim))
    attn_scan = T * shape.inner * (2 * shape.dt_rank + 6 * shape.state)
    chunk = 32
    attn_lin = 2 * T * shape.lin_heads * (chunk / 2 * (shape.lin_dim + shape.lin_vdim) + 2 * shape.lin_dim * shape.lin_vdim)
    lin_in = 2 * shape.lin_heads * (shape.lin_dim + shape.lin_vdim)
    par_in = (shape.heads + shape.kv_heads) * shape.dim + shape.delta_in()
    moe_runs = sum(1 for _, f in runs if f == "moe")
    return {"in_proj": 2 * T * W * (n["mamba"] * 2 * shape.inner + n["lightning"] * lin_in + n["parallel"] * par_in),
            "qk_prepare": 2 * T * n["mamba"] * (shape.dt_rank + 2 * shape.state) * shape.inner,
            "attention": n["parallel"] * (attn_left + attn_right) + n["mamba"] * attn_scan + n["lightning"] * attn_lin,
            "out_proj": 2 * T * W * (n["mamba"] * shape.inner + n["lightning"] * shape.lin_heads * shape.lin_vdim +
                                     n["parallel"] * (shape.heads * shape.dim + shape.d_heads * shape.d_vdim)),
            "experts": 2 * T * sum(3 * shape.dense_ff * W if f == "dense" else shape.top * 3 * shape.ff * W if f == "moe" else 0
                                   for _, f in runs),
            "shared": 2 * T * moe_runs * 3 * shape.shared_ff * W,
            "head": 2 * shape.vocab * W}


def vurazen_decode_bytes(shape, B, ctx, es):
    """Bytes a decode step must move, by phase class: weights once per step, states read and written, the window's keys."""
    W = shape.width
    runs = [shape.pattern[i] for i, _, _ in shape.run_order()]
    state = shape.state_bytes_per_step(B, ctx, es)
    lin_in = 2 * shape.lin_heads * (shape.lin_dim + shape.lin_vdim)
    par_in = (shape.heads + shape.kv_heads) * shape.dim + shape.delta_in()
    n_in = {"mamba": 2 * shape.inner, "lightning": lin_in, "parallel": par_in}
    n_out = {"mamba": shape.inner, "lightning": shape.lin_heads * shape.lin_vdim,
             "parallel": shape.heads * shape.dim + shape.d_heads * shape.d_vdim}
    pairs = min(B * shape.top, shape.experts)
    return {"in_proj": sum(n_in[m] for m, _ in runs) * W * es,
            "qk_prepare": sum((shape.dt_rank + 2 * shape.state) * shape.inner * es for m, _ in runs if m == "mamba"),
            "out_proj": sum(n_out[m] for m, _ in runs) * W * es,
            "experts": sum(3 * shape.dense_ff * W if f == "dense" else pairs * 3 * shape.ff * W if f == "moe" else 0
                           for _, f in runs) * es,
            "shared": sum(3 * shape.shared_ff * W for _, f in runs if f == "moe") * es,
            "attention": state, "head": shape.vocab * W * es}


def kikunex_costs(shape, prompt_len):
    """FLOPs of a prompt step and bytes of a decode step, by phase class of the engine's profile."""
    W = shape.width
    runs = [shape.pattern[i] for i, _, _ in shape.run_order()]
    n_lat = sum(1 for m, _ in runs if m == "latent")
    n_lin = len(runs) - n_lat
    win = min(shape.window, prompt_len)
    pairs = prompt_len * win - win * (win - 1) / 2  # (query, key) pairs inside the window
    H, r, dr = shape.heads, shape.kv_rank, shape.rot_dim
    # latent attention in its per-head form: scores over dim + rot_dim, sums over vdim, and the two up-projections of
    # every token's latent (W_uk c, W_uv c); the absorbed form the engine uses beyond fresh prompts costs more
    attn_lat = 2 * pairs * H * (shape.dim + dr + shape.vdim) + 2 * prompt_len * H * r * (shape.dim + shape.vdim)
    chunk = 32
    attn_lin = 2 * prompt_len * shape.lin_heads * (chunk / 2 * (shape.lin_dim + shape.lin_vdim) +
                                                    2 * shape.lin_dim * shape.lin_vdim)
    flops = {"in_proj": 2 * prompt_len * W * (n_lat * shape.n_in("latent") + n_lin * shape.n_in("lightning")),
             "qk_prepare": 2 * prompt_len * n_lat * H * (shape.dim + dr) * shape.q_rank,
             "attention": n_lat * attn_lat + n_lin * attn_lin,
             "out_proj": 2 * prompt_len * W * (n_lat * H * shape.vdim + n_lin * shape.lin_heads * shape.lin_vdim),
             "experts": 2 * prompt_len * sum(shape.ff_weight_elems(f, shape.top) - (shape.experts * W if f == "moe" else 0)
                                             for _, f in runs),
             "head": 2 * shape.vocab * W}
    return flops


def fobolorn_costs(shape, prompt_len):
    W = shape.width
    R = shape.runs
    return {"in_proj": 2 * prompt_len * W * shape.n_in() * R,
            "attention": 2 * prompt_len * prompt_len / 2 * (shape.dim + shape.vdim) * shape.heads * R,
            "out_proj": 2 * prompt_len * W * shape.heads * shape.vdim * R,
            "experts": 2 * prompt_len * shape.top * 3 * shape.ff * W * R,
            "shared": 2 * prompt_len * 3 * shape.shared_ff * W * R,
            "head": 2 * shape.vocab * W}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class Flusher:
    def __init__(self, torch):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.add_(1)


def time_events(torch, fn, flush, reps=5, warm=3):
    for _ in range(warm):
        fn()
    ms = []
    for _ in range(reps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    return statistics.median(ms)


def bench_engine(torch, shape, dtype, prompt_len, ctx, batches, steps, warm, flush, hbm, tf):
    es = 2 if dtype == BF16 else 4
    eng = SeqEngine(shape, dtype, max_tokens=max(prompt_len, max(batches) * (ctx + steps + warm + 8)) + 64,
                    max_seqs=max(batches) + 1, seed=7)
    g = torch.Generator().manual_seed(1)

    def toks(n):
        return torch.randint(0, shape.vocab, (n,), generator=g).tolist()
    out = {"dtype": "bf16" if dtype == BF16 else "fp32"}
    # ---- prefill: one sequence of prompt_len tokens per step -----------------------------------------------------
    times = []
    for i in range(warm + steps):
        s = eng.open()
        t = toks(prompt_len)
        flush()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.step([(s, t)])
        dt = time.perf_counter() - t0
        eng.close_seq(s)
        if i >= warm:
            times.append(dt)
    s = eng.open()
    _, ph = eng.step([(s, toks(prompt_len))], profile=True)
    launches = eng.launches()
    eng.close_seq(s)
    sec = statistics.median(times)
    kiku = isinstance(shape, KikunexShape)
    vura = isinstance(shape, VurazenShape)
    buku = isinstance(shape, BukuvikShape)
    phase_flops = (bukuvik_costs if buku else vurazen_costs if vura else kikunex_costs if kiku else
                   fobolorn_costs)(shape, prompt_len)
    flops = sum(phase_flops.values())
    out["prefill"] = {"tokens": prompt_len, "tok_s": prompt_len / sec, "ms": sec * 1e3, "launches": launches,
                      "tflops": flops / sec / 1e12, "frac_of_bf16_peak": flops / sec / 1e12 / tf if dtype == BF16 else None,
                      "phase_ms": ph,
                      "phase_tflops": {k: (v / (ph[k] * 1e-3) / 1e12 if ph.get(k, 0) > 0 else None)
                                       for k, v in phase_flops.items()}}
    # ---- decode: B sequences at context ctx, one token each per step ---------------------------------------------
    out["decode"] = {}
    for B in batches:
        seqs = [eng.open() for _ in range(B)]
        eng.step([(q, toks(ctx)) for q in seqs])
        times = []
        for i in range(warm + steps):
            ent = [(q, toks(1)) for q in seqs]
            flush()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.step(ent)
            dt = time.perf_counter() - t0
            if i >= warm:
                times.append(dt)
        _, ph = eng.step([(q, toks(1)) for q in seqs], profile=True)
        launches = eng.launches()
        for q in seqs:
            eng.close_seq(q)
        sec = statistics.median(times)
        # bytes a step must read: the active weights (distinct experts per token, an upper bound when tokens share
        # experts) and the cached keys / values
        W = shape.width
        if vura or buku:
            phase_bytes = (bukuvik_decode_bytes if buku else vurazen_decode_bytes)(shape, B, ctx, es)
            bytes_step = shape.weight_elems_per_step(B) * es + phase_bytes["attention"]
            out["decode"][str(B)] = {
                "batch": B, "context": ctx, "tok_s": B / sec, "ms_per_step": sec * 1e3, "launches": launches,
                "bytes_per_step": bytes_step, "frac_of_hbm_peak": bytes_step / sec / 1e9 / hbm, "phase_ms": ph,
                "phase_frac_of_hbm_peak": {k: (v / (ph[k] * 1e-3) / 1e9 / hbm if ph.get(k, 0) > 0 else None)
                                           for k, v in phase_bytes.items()}}
            continue
        if kiku:
            runs = [shape.pattern[i] for i, _, _ in shape.run_order()]
            state = shape.state_bytes_per_step(B, ctx, es)
            bytes_step = shape.weight_elems_per_step(B) * es + state
            phase_bytes = {"in_proj": sum(shape.n_in(m) for m, _ in runs) * W * es,
                           "out_proj": sum(shape.heads * shape.vdim if m == "latent" else shape.lin_heads * shape.lin_vdim
                                           for m, _ in runs) * W * es,
                           "experts": sum(shape.ff_weight_elems(f, B * shape.top) - (shape.experts * W if f == "moe" else 0)
                                          for _, f in runs) * es,
                           "attention": state + sum(shape.heads * shape.vdim * shape.kv_rank for m, _ in runs if m == "latent") * es,
                           "head": shape.vocab * W * es}
            out["decode"][str(B)] = {
                "batch": B, "context": ctx, "tok_s": B / sec, "ms_per_step": sec * 1e3, "launches": launches,
                "bytes_per_step": bytes_step, "frac_of_hbm_peak": bytes_step / sec / 1e9 / hbm, "phase_ms": ph,
                "phase_frac_of_hbm_peak": {k: (v / (ph[k] * 1e-3) / 1e9 / hbm if ph[k] > 0 else None)
                                           for k, v in phase_bytes.items()}}
            continue
        per_run_shared = (shape.n_in() * W + W * shape.heads * shape.vdim + 3 * shape.shared_ff * W) * es + shape.experts * W * 4
        per_run_experts = min(B * shape.top, shape.experts) * 3 * shape.ff * W * es
        kv = B * ctx * shape.kv_heads * (shape.dim + shape.vdim) * es
        bytes_step = (per_run_shared + per_run_experts + kv) * shape.runs + shape.vocab * W * es
        phase_bytes = {"in_proj": shape.n_in() * W * es * shape.runs, "out_proj": W * shape.heads * shape.vdim * es * shape.runs,
                       "experts": per_run_experts * shape.runs, "shared": 3 * shape.shared_ff * W * es * shape.runs,
                       "attention": kv * shape.runs, "head": shape.vocab * W * es}
        out["decode"][str(B)] = {
            "batch": B, "context": ctx, "tok_s": B / sec, "ms_per_step": sec * 1e3, "launches": launches,
            "bytes_per_step": bytes_step, "frac_of_hbm_peak": bytes_step / sec / 1e9 / hbm, "phase_ms": ph,
            "phase_frac_of_hbm_peak": {k: (v / (ph[k] * 1e-3) / 1e9 / hbm if ph[k] > 0 else None)
                                       for k, v in phase_bytes.items()}}
    eng.close()
    return out


def bench_llama(torch, shape, ctx, steps, warm, hbm, tf):
    """The closest existing model at equal size: fp32 Llama through the single-sequence decoder."""
    from . import Decoder, ModelShape, synth_weights
    ls = ModelShape(f"llama-like-{shape.name}", shape.width, shape.top * shape.ff + shape.shared_ff, shape.runs,
                    shape.heads, shape.kv_heads, shape.vocab, 2 * ctx)
    import os
    w = synth_weights(ls, "cuda", 11)
    bytes_tok = ls.weight_bytes_per_token()

    def decode_rate(dec):
        dec.generate(1, 0, ctx)  # fill the cache
        reps = []
        for i in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            dec.generate(1, ctx, steps)
            b.record()
            torch.cuda.synchronize()
            reps.append(a.elapsed_time(b) * 1e-3)
        sec = statistics.median(reps) / steps
        return {"batch": 1, "context": ctx, "engine": dec.engine, "tok_s": 1 / sec, "ms_per_step": sec * 1e3,
                "bytes_per_step": bytes_tok, "frac_of_hbm_peak": bytes_tok / sec / 1e9 / hbm}
    # the family's other decode engine, a CUDA graph of one fused kernel per phase: the like of the batched engine's
    # decode step (a graph of small kernels); the persistent kernel is the default
    old_env = os.environ.get("KLLM_ENGINE")
    os.environ["KLLM_ENGINE"] = "graph"
    try:
        dec = Decoder(ls, w)
        graph_rate = decode_rate(dec)
        dec.close()
    finally:
        if old_env is None:
            del os.environ["KLLM_ENGINE"]
        else:
            os.environ["KLLM_ENGINE"] = old_env
    dec = Decoder(ls, w)
    res = {"model": ls.name, "dtype": "fp32", "engine": dec.engine, "decode": decode_rate(dec),
           "decode_graph_engine": graph_rate}
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, shape.vocab, (ctx,), generator=g).tolist()
    try:
        times = []
        for i in range(warm + 3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            dec.prefill_tf32(prompt, 0)
            torch.cuda.synchronize()
            if i >= warm:
                times.append(time.perf_counter() - t0)
        sec = statistics.median(times)
        flops = 2 * (bytes_tok / 4 - shape.vocab * shape.width) * ctx + \
            2 * ctx * ctx / 2 * 2 * (shape.width // shape.heads) * shape.heads * shape.runs
        res["prefill"] = {"tokens": ctx, "tok_s": ctx / sec, "ms": sec * 1e3, "tflops": flops / sec / 1e12,
                          "frac_of_tf32_peak": flops / sec / 1e12 / (tf / 2), "multiply": "tf32"}
    except Exception as e:  # noqa: BLE001
        res["prefill"] = {"unavailable": str(e)[:200]}
    dec.close()
    return res


def bench_kernels(torch, shape, flush, hbm, tf):
    """The like kernels of the two families at this size's projection shapes."""
    import ctypes
    from . import load_library
    seq = load_seq_library()
    core = load_library()
    W, N, T = shape.width, shape.n_in(), 2048
    res = {}
    a16 = torch.randn(T, W, device="cuda").bfloat16()
    w16 = torch.randn(N, W, device="cuda").bfloat16()
    a32, w32 = a16.float(), w16.float()
    out = torch.empty(T, N, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    fl = 2.0 * T * W * N
    ms = time_events(torch, lambda: seq.kllm_seq_gemm(BF16, p(a16), p(w16), p(out), T, W, N, None), flush)
    res["block_product_bf16_tcgen05"] = {"shape": [T, W, N], "ms": ms, "tflops": fl / ms / 1e9,
                                         "frac_of_bf16_peak": fl / ms / 1e9 / tf}
    ms = time_events(torch, lambda: core.kllm_gemm_tf32(p(a32), p(w32), p(out), T, W, N, None), flush)
    res["block_product_tf32_tcgen05_llama"] = {"shape": [T, W, N], "ms": ms, "tflops": fl / ms / 1e9,
                                               "frac_of_tf32_peak": fl / ms / 1e9 / (tf / 2)}
    ms = time_events(torch, lambda: seq.kllm_seq_gemm(F32, p(a32), p(w32), p(out), T, W, N, None), flush)
    res["block_product_fp32_fma"] = {"shape": [T, W, N], "ms": ms, "tflops": fl / ms / 1e9}
    # one row: the weights are streamed once
    Nv = shape.vocab
    wv16 = torch.randn(Nv, W, device="cuda").bfloat16()
    wv32 = wv16.float()
    o1 = torch.empty(Nv, device="cuda")
    ms = time_events(torch, lambda: seq.kllm_seq_gemm(BF16, p(a16), p(wv16), p(o1), 1, W, Nv, None), flush)
    res["row_product_bf16"] = {"shape": [1, W, Nv], "ms": ms, "frac_of_hbm_peak": Nv * W * 2 / ms / 1e6 / hbm}
    ms = time_events(torch, lambda: seq.kllm_seq_gemm(F32, p(a32), p(wv32), p(o1), 1, W, Nv, None), flush)
    res["row_product_fp32"] = {"shape": [1, W, Nv], "ms": ms, "frac_of_hbm_peak": Nv * W * 4 / ms / 1e6 / hbm}
    ms = time_events(torch, lambda: core.kllm_gemv_f32(p(a32), p(wv32), p(o1), W, Nv, None), flush)
    res["row_product_fp32_llama"] = {"shape": [1, W, Nv], "ms": ms, "frac_of_hbm_peak": Nv * W * 4 / ms / 1e6 / hbm}
    return res


def run(args, emit):
    import torch
    torch.cuda.set_device(0)
    hbm, tf, src = peaks()
    flush = Flusher(torch)
    sizes = [s for s in (args.family_sizes.split(",") if args.family_sizes else ["s", "m"])]
    steps, warm = max(3, min(args.steps, 16)), max(3, min(args.warmup, 8))
    if args.family == "kikunex":
        return run_kikunex(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src)
    if args.family == "vurazen":
        return run_vurazen(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src)
    if args.family == "bukuvik":
        return run_bukuvik(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src)
    line = {"family": "fobolorn", "metric": "prefill_and_decode_tokens_per_s", "n_gpus": 1, "steps": steps, "warmup": warm,
            "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "config": {"l2": "a 256 MiB buffer is written between timed steps", "timing": "wall clock around the blocking "
                       "step call (token ids from host memory, greedy ids back to host memory); phases by CUDA events"},
            "sizes": {}}
    for name in sizes:
        shape = SIZES[name]
        ctx, prompt = (256, 512) if name == "debug" else (1024, 2048)
        entry = {"shape": shape.__dict__ | {"runs": shape.runs}, "fobolorn": [], "closest": None, "kernels": None}
        for dtype in (BF16, F32):
            entry["fobolorn"].append(bench_engine(torch, shape, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
        entry["closest"] = bench_llama(torch, shape, ctx, max(steps, 32), warm, hbm, tf)
        entry["kernels"] = bench_kernels(torch, shape, flush, hbm, tf)
        line["sizes"][name] = entry
    emit(line)


def run_kikunex(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src):
    """Kikunex beside its closest existing model, Fobolorn (the same engine), at equal width, heads, experts and layer
    runs: whole steps end to end, and the engine's phase classes side by side."""
    line = {"family": "kikunex", "metric": "prefill_and_decode_tokens_per_s", "n_gpus": 1, "steps": steps, "warmup": warm,
            "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "config": {"l2": "a 256 MiB buffer is written between timed steps", "timing": "wall clock around the blocking "
                       "step call (token ids from host memory, greedy ids back to host memory); phases by CUDA events"},
            "sizes": {}}
    for name in sizes:
        shape, close = KIKUNEX_SIZES[name], SIZES[name]
        ctx, prompt = (256, 512) if name == "debug" else (1024, 2048)
        entry = {"shape": {k: v for k, v in shape.__dict__.items()} | {"runs": shape.runs}, "kikunex": [], "closest": []}
        for dtype in (BF16, F32):
            entry["kikunex"].append(bench_engine(torch, shape, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
            entry["closest"].append(bench_engine(torch, close, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
        entry["closest_model"] = close.name
        line["sizes"][name] = entry
    emit(line)


def run_vurazen(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src):
    """Vurazen beside its closest existing model, Kikunex (the same engine: linear attention, a windowed softmax
    attention, routed experts, a loop), at equal width, heads, experts and layer runs: whole steps end to end, and the
    engine's phase classes side by side."""
    line = {"family": "vurazen", "metric": "prefill_and_decode_tokens_per_s", "n_gpus": 1, "steps": steps, "warmup": warm,
            "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "config": {"l2": "a 256 MiB buffer is written between timed steps", "timing": "wall clock around the blocking "
                       "step call (token ids from host memory, greedy ids back to host memory); phases by CUDA events"},
            "sizes": {}}
    for name in sizes:
        shape, close = VURAZEN_SIZES[name], KIKUNEX_SIZES[name]
        ctx, prompt = (256, 512) if name == "debug" else (1024, 2048)
        entry = {"shape": {k: v for k, v in shape.__dict__.items()} | {"runs": shape.runs}, "vurazen": [], "closest": []}
        for dtype in (BF16, F32):
            entry["vurazen"].append(bench_engine(torch, shape, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
            entry["closest"].append(bench_engine(torch, close, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
        entry["closest_model"] = close.name
        line["sizes"][name] = entry
    emit(line)


def run_bukuvik(args, emit, torch, sizes, steps, warm, flush, hbm, tf, src):
    """Bukuvik beside its closest existing model, Vurazen (the same engine: a windowed softmax attention that keeps the
    first tokens beside a recurrent mixer with a short convolution in one layer, a scan with input-dependent decays), at
    equal width, head counts and layer runs: whole steps end to end, and the engine's phase classes side by side."""
    line = {"family": "bukuvik", "metric": "prefill_and_decode_tokens_per_s", "n_gpus": 1, "steps": steps, "warmup": warm,
            "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
            "config": {"l2": "a 256 MiB buffer is written between timed steps", "timing": "wall clock around the blocking "
                       "step call (token ids from host memory, greedy ids back to host memory); phases by CUDA events"},
            "sizes": {}}
    for name in sizes:
        shape, close = BUKUVIK_SIZES[name], VURAZEN_SIZES[name]
        ctx, prompt = (256, 512) if name == "debug" else (1024, 2048)
        entry = {"shape": {k: v for k, v in shape.__dict__.items()} | {"runs": shape.runs}, "bukuvik": [], "closest": []}
        for dtype in (BF16, F32):
            entry["bukuvik"].append(bench_engine(torch, shape, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
            entry["closest"].append(bench_engine(torch, close, dtype, prompt, ctx, [1, 8], steps, warm, flush, hbm, tf))
        entry["closest_model"] = close.name
        line["sizes"][name] = entry
    emit(line)
