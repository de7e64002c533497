"""A slow float64 restatement of the Vurazen family, one function per mechanism.

It shares no code with the product path: numpy only, whole sequences, no cache and no state (every function sees the
complete sequence).  `weights` maps tensor names to float64 arrays; `config` is the parsed config.json.

    tokens --embed * scale--> layer runs --> layer norm --> head --> cap * tanh(. / cap)

    layer:  h = LN(x; norm1);  x += mixer(h) + ff(h)        (one norm, both sublayers read it; ff optional)
    loop:   layers start..stop-1 run `times` times; before pass t > 0 the embedding output is added to x, and before
            every pass row t of 'loop.step'
    mixers: 'mamba1' (selective scan), 'lightning' (linear attention with a fixed decay per head), 'parallel' (a
            windowed softmax attention whose values are its keys, beside a gated delta rule; a weighted sum of both)
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ------------------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def short_conv(u, taps_w, bias=None):
    """Causal convolution over time per channel.  u [T, C]; taps_w [C, taps], the last column weighs the current row;
    rows before the start count as zero."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = np.vstack([np.zeros((taps - 1, C)), u])
    out = np.zeros((T, C))
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j]
    return out if bias is None else out + bias


def rotate_pairs(v, positions, dims, base):
    """Rotary positions on the first `dims` coordinates of v [T, heads, n]: coordinate 2i pairs with 2i + 1."""
    out = v.copy()
    for i in range(dims // 2):
        ang = positions * base ** (-2.0 * i / dims)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------------
def mamba(h, w, p, m, eps):
    """Selective scan.  h [T, width]; p: tensor prefix '<layer>.mix.'; m: the mixer's configuration."""
    T = h.shape[0]
    inner, n, rank = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(short_conv(x, w[p + "conv"], w[p + "conv.b"]))
    low = x @ w[p + "x"].T
    dt = softplus(low[:, :rank] @ w[p + "dt"].T + w[p + "dt.b"])          # [T, inner]
    B, C = low[:, rank:rank + n], low[:, rank + n:rank + 2 * n]
    A = -np.exp(w[p + "A_log"])                                           # [inner, n]
    S = np.zeros((inner, n))
    y = np.zeros((T, inner))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


def lightning(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    decay = m["decay"] if isinstance(m["decay"], (list, tuple)) else [m["decay"]] * H
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[hd] * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = rms_unit(out.reshape(T, H * dv), eps) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def window_attention(h, w, p, m, eps):
    """Softmax attention over a sliding window plus the first tokens, values = keys before rotation, capped scores,
    one sink per head in the denominator."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    assert m["vdim"] == d
    pos = np.arange(T, dtype=np.float64)
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).reshape(T, H, d)
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).reshape(T, G, d)
    v = k
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rotate_pairs(q, pos, rot["dims"], rot["base"]), rotate_pairs(k, pos, rot["dims"], rot["base"])
    mask = m.get("mask") or {"size": T + 1, "keep_first": 0}
    cap = m.get("softcap")
    out = np.zeros((T, H, d))
    for i in range(T):
        seen = [j for j in range(i + 1) if i - j < mask["size"] or j < mask.get("keep_first", 0)]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[seen, g] @ q[i, hd]) * m["scale"]
            if cap:
                s = cap * np.tanh(s / cap)
            sink = w[p + "sink"][hd]
            top = max(s.max(), sink)
            e = np.exp(s - top)
            out[i, hd] = (e @ v[seen, g]) / (e.sum() + math.exp(sink - top))
    return out.reshape(T, H * d) @ w[p + "o"].T


def gated_delta(h, w, p, m, eps):
    """Gated delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    rate = np.exp(w[p + "A_log"])                                           # [H]
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, dk)
    decay = np.exp(-rate[None, :, None] * step)                             # [T, H, dk]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


def parallel(h, w, p, m, eps):
    return m["left_scale"] * window_attention(h, w, p + "left.", m["left"], eps) + \
        m["right_scale"] * gated_delta(h, w, p + "right.", m["right"], eps)


# ---- feed-forward ------------------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return (np.maximum(h @ w[p + "gate"].T, 0.0) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, r):
    """Returns (chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen ones."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :r["top"]]
    zc = np.take_along_axis(z, idx, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def moe_ff(h, w, p, c):
    idx, wt = route(h, w, p, c["router"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t]):
            out[t] += wt[t, j] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", c["expert"]["limit"])[0]
    if c.get("shared"):
        out += clamped_expert(h, w, p + "shared.", c["shared"]["limit"])
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------
MIXERS = {"mamba1": mamba, "lightning": lightning, "parallel": parallel}


def layer_runs(config):
    """[(layer, pass number or None)]: pass number on the first layer of each pass of the loop."""
    n = len(config["layers"])
    lp = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(config, weights, tokens):
    """Returns (logits [T, vocab], residual stream after every layer run [runs, T, width])."""
    w, eps = weights, config["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    x = x0.copy()
    trace = []
    for i, t in layer_runs(config):
        L = config["layers"][i]
        pre = f"l{i}."
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        h = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
        y = MIXERS[L["type"]](h, w, pre + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            y = y + (dense_ff(h, w, pre + "mlp.") if L["mlp"]["kind"] == "dense" else moe_ff(h, w, pre + "mlp.", L["mlp"]))
        x = x + y
        trace.append(x.copy())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return logits, np.stack(trace)


def greedy(config, weights, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence (lowest index on ties)."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        logits, _ = forward(config, weights, seq)
        out.append(int(np.argmax(logits[-1])))
        seq.append(out[-1])
    return out


# ---- small random models for the tests ------------------------------------------------------------------------------------
def mamba_mixer(inner=24, state=5, dt_rank=3, conv=3):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def lightning_mixer(heads=3, dim=8, vdim=12, decay=None):
    decay = [math.exp(-1.0 / (2.0 + 7.0 * h)) for h in range(heads)] if decay is None else decay
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def left_mixer(heads=4, kv_heads=2, dim=12, conv=3, window=16, keep_first=2, rot_dims=8, base=10000.0, scale=None,
               softcap=20.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv,
            "mask": {"size": window, "keep_first": keep_first}, "rot": {"base": base, "dims": rot_dims},
            "scale": dim ** -0.5 if scale is None else scale, "softcap": softcap}


def right_mixer(heads=4, kv_heads=2, dim=10, vdim=6, conv=2):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel_mixer(left=None, right=None, left_scale=0.7, right_scale=0.4):
    return {"type": "parallel", "mixer": {"left": left or left_mixer(), "right": right or right_mixer(),
                                          "left_scale": left_scale, "right_scale": right_scale}}


def dense_mlp(ff=40):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, top=2, ff=16, limit=1.25, shared=(12, 0.75)):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def make_config(width=48, vocab=61, layers=(), loop=None, eps=3e-6, logit_softcap=12.0, embed_scale=1.5):
    """layers: [(mixer dict, mlp dict or None)]."""
    cfg = {"architecture": "Vurazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": logit_softcap,
           "embedding": {"scale": embed_scale}, "layers": [dict(m, mlp=f) for m, f in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7fff + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


def make_weights(cfg, seed=0, sharp=1.0):
    """Random bf16-representable weights.  `sharp` multiplies the attention's query weights: > 1 makes the softmax
    peaky, so that single keys (those at a window's edge too) carry the output."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, std=1.0, mean=0.0):
        return bf16_round(mean + std * rng.standard_normal(shape))

    def fan(rows, cols, gain=1.0):
        return rnd(rows, cols, std=gain * cols ** -0.5)
    w = {"embed": rnd(V, W), "head": fan(V, W), "final.norm": rnd(W, mean=1.0, std=0.1), "final.norm.b": rnd(W, std=0.1)}
    if cfg.get("loop"):
        w["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.5)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = rnd(W, mean=1.0, std=0.1)
        w[p + "norm1.b"] = rnd(W, std=0.1)
        q = p + "mix."
        if L["type"] == "mamba1":
            n, r, c = m["inner"], m["dt_rank"], m["state"]
            w[q + "in"] = fan(2 * n, W)
            w[q + "conv"] = rnd(n, m["conv"], std=0.6)
            w[q + "conv.b"] = rnd(n, std=0.2)
            w[q + "x"] = fan(r + 2 * c, n)
            w[q + "dt"] = fan(n, r)
            w[q + "dt.b"] = rnd(n, mean=-1.0, std=0.7)
            w[q + "A_log"] = bf16_round(np.log(rng.uniform(0.05, 4.0, (n, c))))
            w[q + "D"] = rnd(n)
            w[q + "o"] = fan(W, n)
        elif L["type"] == "lightning":
            H = m["heads"]
            for nme, rows in (("q", H * m["dim"]), ("k", H * m["dim"]), ("v", H * m["vdim"]), ("g", H * m["vdim"])):
                w[q + nme] = fan(rows, W)
            w[q + "norm"] = rnd(H * m["vdim"], mean=1.0, std=0.1)
            w[q + "o"] = fan(W, H * m["vdim"])
        else:
            a, l = m["left"], q + "left."
            w[l + "q"] = fan(a["heads"] * a["dim"], W, sharp)
            w[l + "k"] = fan(a["kv_heads"] * a["dim"], W, 1.5)
            w[l + "q.b"] = rnd(a["heads"] * a["dim"], std=0.2)
            w[l + "k.b"] = rnd(a["kv_heads"] * a["dim"], std=0.2)
            w[l + "q.conv"] = rnd(a["heads"] * a["dim"], a["conv"], std=0.6)
            w[l + "k.conv"] = rnd(a["kv_heads"] * a["dim"], a["conv"], std=0.6)
            w[l + "sink"] = rnd(a["heads"])
            w[l + "o"] = fan(W, a["heads"] * a["vdim"])
            d, r = m["right"], q + "right."
            low = max(2, d["dim"] // 4)
            for nme, rows in (("q", d["kv_heads"] * d["dim"]), ("k", d["kv_heads"] * d["dim"]), ("v", d["heads"] * d["vdim"])):
                w[r + nme] = fan(rows, W, 2.0)
                w[r + nme + ".conv"] = rnd(rows, d["conv"], std=0.6)
            w[r + "b"] = fan(d["heads"], W, 2.0)
            w[r + "A_log"] = bf16_round(np.log(rng.uniform(0.02, 2.0, d["heads"])))
            w[r + "norm"] = rnd(d["vdim"], mean=1.0, std=0.1)
            w[r + "a1"] = fan(low, W)
            w[r + "a2"] = fan(d["heads"] * d["dim"], low, 2.0)
            w[r + "dt_bias"] = rnd(d["heads"] * d["dim"], mean=-1.0, std=0.7)
            w[r + "g1"] = fan(low, W)
            w[r + "g2"] = fan(d["heads"] * d["vdim"], low, 2.0)
            w[r + "o"] = fan(W, d["heads"] * d["vdim"])
        f = L.get("mlp")
        if not f:
            continue
        q = p + "mlp."
        if f["kind"] == "dense":
            w[q + "gate"], w[q + "up"], w[q + "down"] = fan(f["ff"], W), fan(f["ff"], W), fan(W, f["ff"])
        else:
            names = [f"e{e}" for e in range(f["router"]["experts"])] + (["shared"] if f.get("shared") else [])
            for nme in names:
                ff = f["shared"]["ff"] if nme == "shared" else f["expert"]["ff"]
                w[f"{q}{nme}.gate"], w[f"{q}{nme}.up"], w[f"{q}{nme}.down"] = fan(ff, W, 1.5), fan(ff, W, 1.5), fan(W, ff)
            w[q + "router"] = fan(f["router"]["experts"], W, 2.0)
            w[q + "router.b"] = rnd(f["router"]["experts"], std=0.5)
    return w


def write_model(folder, cfg, weights):
    """config.json and model.safetensors (bfloat16) in `folder`."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    header, blobs, at = {}, [], 0
    for name, a in weights.items():
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        assert not (u & 0xffff).any(), f"{name} is not bf16-representable"
        raw = (u >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder
