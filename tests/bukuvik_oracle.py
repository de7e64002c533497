"""A slow float64 restatement of the Bukuvik family, one function per mechanism.

It shares no code with the product path: numpy only, whole sequences, no cache and no state (every function sees the
complete sequence).  `weights` maps tensor names to float64 arrays; `config` is the parsed config.json.

    tokens --embed * scale--> layers --> RMS norm --> embed^T

    layer:  x += m * ls1 * RMS(mixer(x); norm1);  x += m * ls2 * RMS(ff(x); norm2)   (nothing is normed BEFORE a sublayer)
    mixers: 'attention' (differential: two softmax maps per head over the same values, a1 - lambda a2),
            'parallel'  (an attention with rescaled rotary positions and unit-normed q / k, beside a state-space-duality
                         recurrence; the mean of their RMS-normed outputs)
    ff:     down(relu(up x)^2)
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ------------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def short_conv(u, taps_w, bias):
    """u [T, C], taps_w [C, taps]: out[t] = bias + sum_k taps_w[:, k] * u[t - (taps - 1) + k], zeros before the start."""
    T, taps = u.shape[0], taps_w.shape[1]
    out = np.tile(np.asarray(bias, dtype=np.float64), (T, 1))
    for k in range(taps):
        back = taps - 1 - k
        if back < T:
            out[back:] += u[:T - back] * taps_w[:, k]
    return out


def rotary_frequencies(rot):
    """Frequencies of the rot["dims"] / 2 rotated pairs and the factor on cos and sin.  With rot["scaling"], waves that
    make fewer than `slow` turns over the original length are slowed by `factor`, those with more than `fast` turns are
    kept, and the coordinates between them are blended linearly."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def coordinate(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(coordinate(sc["fast"])), 0)
    hi = min(math.ceil(coordinate(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_halves(v, positions, rot):
    """v [T, heads, dim]: coordinate i < dims / 2 is paired with coordinate i + dims / 2; the rest pass."""
    if not rot or rot["dims"] == 0:
        return v
    half = rot["dims"] // 2
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = v.copy()
    a, b = v[..., :half], v[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


def visible(T, window, keep_first):
    """[T, T] mask: row i sees column j <= i when i - j < window (window 0: all) or j < keep_first."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    near = (i - j < window) if window else np.ones((T, T), dtype=bool)
    return (j <= i) & (near | (j < keep_first))


def softmax_map(q, k, v, scale, softcap, mask):
    """One attention map: q [T, dim], k [T, dim], v [T, vdim]."""
    s = q @ k.T * scale
    if softcap:
        s = softcap * np.tanh(s / softcap)
    s = np.where(mask, s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    return (p / p.sum(-1, keepdims=True)) @ v


# ---- mixers ------------------------------------------------------------------------------------------------------------
def differential_lambda(w, p, diff):
    return math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + diff


def differential_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, 2, D)
    k = (h @ w[p + "k"].T).reshape(T, G, 2, D)
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    q = rotate_halves(q.reshape(T, 2 * H, D), pos, m.get("rot")).reshape(T, H, 2, D)
    k = rotate_halves(k.reshape(T, 2 * G, D), pos, m.get("rot")).reshape(T, G, 2, D)
    mask = visible(T, m["mask"]["size"] if m.get("mask") else 0, (m.get("mask") or {}).get("keep_first", 0))
    lam = differential_lambda(w, p, m["diff"])
    out = np.zeros((T, H, V))
    for hh in range(H):
        g = hh // (H // G)
        a1 = softmax_map(q[:, hh, 0], k[:, g, 0], v[:, g], m["scale"], m.get("softcap"), mask)
        a2 = softmax_map(q[:, hh, 1], k[:, g, 1], v[:, g], m["scale"], m.get("softcap"), mask)
        out[:, hh] = rms_unit(a1 - lam * a2, eps) * (1.0 - m["diff"])
    gated = out.reshape(T, H * V) * sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T


def unit_attention(h, w, p, m, eps):
    """The left mixer of a 'parallel' layer."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = rotate_halves((h @ w[p + "q"].T).reshape(T, H, D), pos, m.get("rot"))
    k = rotate_halves((h @ w[p + "k"].T).reshape(T, G, D), pos, m.get("rot"))
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    mask = visible(T, m["mask"]["size"] if m.get("mask") else 0, (m.get("mask") or {}).get("keep_first", 0))
    out = np.zeros((T, H, V))
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = softmax_map(q[:, hh], k[:, g], v[:, g], m["scale"], m.get("softcap"), mask)
    gated = out.reshape(T, H * V) * sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T


def duality(h, w, p, m, eps):
    """The right mixer of a 'parallel' layer: a matrix state per head, one decay per head and token."""
    T = h.shape[0]
    nh, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * V
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, nh, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = -np.exp(w[p + "A_log"])
    y = np.zeros((T, nh, V))
    for hh in range(nh):
        g = hh // (nh // G)
        S = np.zeros((N, V))
        for t in range(T):
            S = math.exp(rate[hh] * dt[t, hh]) * S + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + w[p + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel(h, w, p, m, eps):
    left = rms_unit(unit_attention(h, w, p + "left.", m["left"], eps), eps) * w[p + "left.out"]
    right = rms_unit(duality(h, w, p + "right.", m["right"], eps), eps) * w[p + "right.out"]
    return 0.5 * (left + right)


def dense_ff(h, w, p):
    return np.maximum(h @ w[p + "up"].T, 0.0) ** 2 @ w[p + "down"].T


# ---- the model ---------------------------------------------------------------------------------------------------------
def forward(config, weights, tokens):
    """Returns (logits [T, vocab], residual stream after every layer [layers, T, width])."""
    w, eps, mult = weights, config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"][np.asarray(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    trace = []
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        if L["type"] == "attention":
            y = differential_attention(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * w[p + "ls1"] * (rms_unit(y, eps) * w[p + "norm1"])
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "dense"
            f = dense_ff(x, w, p + "mlp.")
            x = x + mult * w[p + "ls2"] * (rms_unit(f, eps) * w[p + "norm2"])
        trace.append(x.copy())
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["embed"].T
    return logits, np.stack(trace)


def greedy(config, weights, prompt, n_new):
    """n_new greedy tokens after `prompt` (lowest index on ties), recomputing the whole sequence every time."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(np.argmax(forward(config, weights, seq)[0][-1])))
    return seq[len(prompt):]


# ---- small configurations and random weights for the tests ---------------------------------------------------------------
def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        factor, original, fast, slow = scaling
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def diff_mixer(heads=4, kv_heads=2, dim=12, vdim=10, window=16, rot_dims=4, base=1000.0, scale=None, softcap=20.0, diff=0.25):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
         "rot": rot(rot_dims, base), "scale": dim ** -0.5 if scale is None else scale, "diff": diff}
    if softcap:
        m["softcap"] = softcap
    return m


def left_mixer(heads=4, kv_heads=2, dim=12, vdim=8, window=14, keep_first=3, rot_dims=8, base=10000.0,
               scaling=(4.0, 64, 16.0, 1.0), scale=None):
    mask = {"size": window}
    if keep_first:
        mask["keep_first"] = keep_first
    # unit-normed q and k: q . k is about dim * cos(angle), so the default scale is a bit sharper than dim^-0.5
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": mask,
            "rot": rot(rot_dims, base, scaling), "scale": 2.0 * dim ** -0.5 if scale is None else scale}


def right_mixer(heads=4, vdim=6, state=5, groups=2, conv=3, norm_groups=2):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel_mixer(left=None, right=None):
    return {"left": left or left_mixer(), "right": right or right_mixer()}


def make_config(width=48, vocab=61, layers=(), eps=3e-6, embed_scale=2.0, residual_mult=0.8):
    """layers: (mixer, ff size or None); the mixer's kind is read off its keys."""
    out = []
    for mixer, ff in layers:
        out.append({"type": "parallel" if "left" in mixer else "attention", "mixer": mixer,
                    "mlp": {"kind": "dense", "ff": ff} if ff else None})
    return {"architecture": "Bukuvik", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "residual_mult": residual_mult, "layers": out}


def bf16_round(a):
    """Round float64 values to the nearest bfloat16 (ties to even); the result is exactly representable."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7fff + ((u >> 16) & 1)) & 0xffff0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def make_weights(cfg, seed=0, sharp=1.0):
    """Random bf16-representable weights.  `sharp` multiplies the attentions' query weights: > 1 makes the softmax
    peaky, so that single keys (those at a window's edge too) carry the output."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, std=1.0, mean=0.0):
        return bf16_round(mean + std * rng.standard_normal(shape))

    def fan(rows, cols, gain=1.0):
        return rnd(rows, cols, std=gain * cols ** -0.5)

    def attention(p, a, maps):
        w[p + "q"] = fan(maps * a["heads"] * a["dim"], W, sharp)
        w[p + "k"] = fan(maps * a["kv_heads"] * a["dim"], W, 1.5)
        w[p + "v"] = fan(a["kv_heads"] * a["vdim"], W)
        w[p + "g"] = fan(a["heads"] * a["vdim"], W, 2.0)
        w[p + "o"] = fan(W, a["heads"] * a["vdim"])
    w = {"embed": rnd(V, W, std=0.5), "final.norm": rnd(W, mean=1.0, std=0.1)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = rnd(W, mean=1.0, std=0.1)
        w[p + "ls1"] = rnd(W, mean=0.8, std=0.2)
        q = p + "mix."
        if L["type"] == "attention":
            attention(q, m, 2)
            w[q + "q.norm"] = rnd(m["dim"], mean=1.0, std=0.2)
            w[q + "k.norm"] = rnd(m["dim"], mean=1.0, std=0.2)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[q + n] = rnd(m["dim"], std=0.7 * m["dim"] ** -0.5)
        else:
            attention(q + "left.", m["left"], 1)
            d, r = m["right"], q + "right."
            inner, bc = d["heads"] * d["vdim"], d["groups"] * d["state"]
            w[r + "in"] = fan(2 * inner + 2 * bc + d["heads"], W, 1.5)
            w[r + "conv"] = rnd(inner + 2 * bc, d["conv"], std=0.6)
            w[r + "conv.b"] = rnd(inner + 2 * bc, std=0.2)
            w[r + "dt_bias"] = rnd(d["heads"], mean=-1.0, std=0.7)
            w[r + "A_log"] = bf16_round(np.log(rng.uniform(0.05, 4.0, d["heads"])))
            w[r + "D"] = rnd(d["heads"])
            w[r + "norm"] = rnd(inner, mean=1.0, std=0.1)
            w[r + "o"] = fan(W, inner)
            w[q + "left.out"] = rnd(W, mean=1.0, std=0.2)
            w[q + "right.out"] = rnd(W, mean=1.0, std=0.2)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            w[p + "norm2"] = rnd(W, mean=1.0, std=0.1)
            w[p + "ls2"] = rnd(W, mean=0.8, std=0.2)
            w[p + "mlp.up"] = fan(ff, W)
            w[p + "mlp.down"] = fan(W, ff)
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
