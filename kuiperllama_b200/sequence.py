"""ctypes loader of the sequence-batch engine (include/kllm_seq.h) for bench.py and tests: torch tensors are the
device memory, the engine and every kernel are the product library's.  Like the rest of this package it has no
fallback: without libkllm_seq.so (or libkllm_b200.so, which carries the same symbols) it raises.

`FobolornShape` / `KikunexShape` / `VurazenShape` / `BukuvikShape` + `SeqEngine` build a random-weight model of a family directly in device memory
(no model folder), for measurements at sizes that resemble a real model's layers.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import POINTER, c_float, c_int32, c_void_p
from dataclasses import dataclass

F32, BF16 = 0, 1
PHASES = ["norm", "in_proj", "qk_prepare", "attention", "out_proj", "router", "experts", "shared", "head"]


class Norm(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("b", c_void_p), ("kind", c_int32)]


class Attention(ctypes.Structure):
    _fields_ = [("heads", c_int32), ("kv_heads", c_int32), ("dim", c_int32), ("vdim", c_int32), ("scale", c_float),
                ("temp_coef", c_float), ("temp_every", c_int32), ("qk_norm", c_int32), ("gate", c_int32),
                ("w_in", c_void_p), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("w_out", c_void_p),
                ("window", c_int32), ("keep_first", c_int32), ("softcap", c_float), ("sink", c_void_p),
                ("in_bias", c_void_p), ("conv_taps", c_int32), ("conv_w", c_void_p), ("rope_dims", c_int32),
                ("rope_base", c_float), ("rope_pairing", c_int32), ("values_are_keys", c_int32),
                ("rope_freq", c_void_p), ("rope_mag", c_float), ("differential", c_int32), ("diff_lambda", c_float),
                ("diff_out_scale", c_float)]


class Moe(ctypes.Structure):
    _fields_ = [("experts", c_int32), ("top", c_int32), ("ff", c_int32), ("router_scale", c_float),
                ("w_router", c_void_p), ("gate_up", c_void_p), ("down", c_void_p), ("shared_ff", c_int32),
                ("shared_gate_up", c_void_p), ("shared_down", c_void_p), ("w_shared_gate", c_void_p),
                ("router_kind", c_int32), ("correction", c_void_p), ("groups", c_int32), ("groups_keep", c_int32),
                ("act", c_int32), ("router_bias", c_void_p), ("act_limit", c_float), ("act_alpha", c_float),
                ("shared_act_limit", c_float)]


class Latent(ctypes.Structure):
    _fields_ = [("heads", c_int32), ("dim", c_int32), ("rot_dim", c_int32), ("vdim", c_int32), ("q_rank", c_int32),
                ("kv_rank", c_int32), ("scale", c_float), ("window", c_int32), ("rope_dims", c_int32),
                ("rope_base", c_float), ("w_in", c_void_p), ("q_norm_w", c_void_p), ("kv_norm_w", c_void_p),
                ("w_uq", c_void_p), ("w_uk", c_void_p), ("w_uv", c_void_p), ("sink", c_void_p), ("w_out", c_void_p)]


class Linear(ctypes.Structure):
    _fields_ = [("heads", c_int32), ("dim", c_int32), ("vdim", c_int32), ("decay", c_void_p), ("w_in", c_void_p),
                ("out_norm_w", c_void_p), ("w_out", c_void_p)]


class Dense(ctypes.Structure):
    _fields_ = [("ff", c_int32), ("act", c_int32), ("act_a", c_float), ("act_b", c_float), ("up", c_void_p),
                ("down", c_void_p)]


class Ssm(ctypes.Structure):
    _fields_ = [("inner", c_int32), ("state", c_int32), ("dt_rank", c_int32), ("conv_taps", c_int32), ("w_in", c_void_p),
                ("conv_w", c_void_p), ("conv_b", c_void_p), ("w_x", c_void_p), ("w_dt", c_void_p), ("dt_b", c_void_p),
                ("a", c_void_p), ("d", c_void_p), ("w_out", c_void_p)]


class Delta(ctypes.Structure):
    _fields_ = [("heads", c_int32), ("kv_heads", c_int32), ("dim", c_int32), ("vdim", c_int32), ("conv_taps", c_int32),
                ("decay_rank", c_int32), ("gate_rank", c_int32), ("w_in", c_void_p), ("conv_w", c_void_p),
                ("w_low2", c_void_p), ("dt_bias", c_void_p), ("rate", c_void_p),
                ("out_norm_w", c_void_p), ("w_out", c_void_p)]


class Ssd(ctypes.Structure):
    _fields_ = [("heads", c_int32), ("vdim", c_int32), ("state", c_int32), ("groups", c_int32), ("conv_taps", c_int32),
                ("norm_groups", c_int32), ("w_in", c_void_p), ("conv_w", c_void_p), ("conv_b", c_void_p),
                ("dt_bias", c_void_p), ("a", c_void_p), ("d", c_void_p), ("out_norm_w", c_void_p), ("w_out", c_void_p)]


class Layer(ctypes.Structure):
    _fields_ = [("mixer_kind", c_int32), ("ff_kind", c_int32), ("pre_mixer", Norm), ("post_mixer", Norm),
                ("pre_ff", Norm), ("post_ff", Norm), ("attn", Attention), ("moe", Moe), ("shift", c_void_p),
                ("latent", Latent), ("linear", Linear), ("dense", Dense), ("ssm", Ssm), ("delta", Delta),
                ("mixer2_kind", c_int32), ("mixer_scale", c_float), ("mixer2_scale", c_float), ("parallel_ff", c_int32),
                ("ssd", Ssd), ("mixer_out_norm", Norm), ("mixer2_out_norm", Norm)]


class Desc(ctypes.Structure):
    _fields_ = [("dtype", c_int32), ("width", c_int32), ("vocab", c_int32), ("norm_eps", c_float),
                ("n_layers", c_int32), ("layers", POINTER(Layer)), ("n_runs", c_int32), ("run_layer", POINTER(c_int32)),
                ("run_add", POINTER(c_int32)), ("run_vectors", c_void_p), ("embed", c_void_p), ("final_norm", Norm),
                ("head", c_void_p), ("max_tokens", c_int32), ("max_seqs", c_int32), ("page_tokens", c_int32),
                ("embed_norm", Norm), ("run_embed", POINTER(c_int32)), ("logit_scale", c_float), ("embed_scale", c_float),
                ("logit_softcap", c_float)]


class SeqError(RuntimeError):
    pass


def load_seq_library():
    from . import build
    lib = ctypes.CDLL(str(build.build_seq()))
    lib.kllm_seq_create.argtypes = [POINTER(Desc), c_void_p, POINTER(c_void_p)]
    lib.kllm_seq_destroy.argtypes = [c_void_p]
    lib.kllm_seq_destroy.restype = None
    lib.kllm_seq_open.argtypes = [c_void_p, POINTER(c_int32)]
    lib.kllm_seq_close.argtypes = [c_void_p, c_int32]
    lib.kllm_seq_length.argtypes = [c_void_p, c_int32]
    lib.kllm_seq_step.argtypes = [c_void_p, c_int32, POINTER(c_int32), POINTER(c_int32), POINTER(c_int32), c_int32,
                                  POINTER(c_int32), c_void_p, c_void_p]
    lib.kllm_seq_profile.argtypes = [c_void_p, POINTER(c_float)]
    lib.kllm_seq_last_launches.argtypes = [c_void_p]
    lib.kllm_seq_gemm.argtypes = [c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]
    lib.kllm_error_string.restype = ctypes.c_char_p
    return lib


def _check(lib, rc, what):
    if rc != 0:
        raise SeqError(f"{what}: {lib.kllm_error_string(rc).decode()} ({rc})")


@dataclass
class FobolornShape:
    name: str
    width: int
    vocab: int
    layers: int          # distinct layers
    loop: tuple          # (start, stop, times)
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    experts: int
    top: int
    ff: int
    shared_ff: int
    temp: tuple = (0.25, 512)
    eps: float = 1e-5

    @property
    def runs(self):
        s, e, t = self.loop
        return s + (e - s) * t + (self.layers - e)

    def run_order(self):
        s, e, t = self.loop
        order = [(i, -1) for i in range(s)]
        for p in range(t):
            order += [(i, p if i == s else -1) for i in range(s, e)]
        return order + [(i, -1) for i in range(e, self.layers)]

    def n_in(self):
        return self.heads * self.dim + self.kv_heads * (self.dim + self.vdim) + self.heads

    def active_weight_elems_per_token(self):
        """Matrix elements one decoded token of one sequence reads, per layer run and for the head."""
        W = self.width
        per_run = self.n_in() * W + W * self.heads * self.vdim + self.experts * W + \
            self.top * 3 * self.ff * W + 3 * self.shared_ff * W
        return per_run * self.runs + self.vocab * W

    def flops_per_token(self):
        return 2 * self.active_weight_elems_per_token()


@dataclass
class KikunexShape:
    """A Kikunex model: `pattern` lists the layers ("lightning" | "latent", "dense" | "moe" | None)."""
    name: str
    width: int
    vocab: int
    pattern: tuple
    loop: tuple          # (start, stop, times)
    heads: int           # latent attention
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    window: int
    lin_heads: int       # linear attention
    lin_dim: int
    lin_vdim: int
    dense_ff: int
    experts: int
    top: int
    ff: int
    groups: tuple = (4, 2)
    eps: float = 1e-5

    @property
    def layers(self):
        return len(self.pattern)

    def run_order(self):
        s, e, t = self.loop
        order = [(i, -1, 0) for i in range(s)]
        for p in range(t):
            order += [(i, p if i == s else -1, 1 if i == s and p > 0 else 0) for i in range(s, e)]
        return order + [(i, -1, 0) for i in range(e, self.layers)]

    @property
    def runs(self):
        return len(self.run_order())

    def n_in(self, kind):
        if kind == "latent":
            return self.q_rank + self.kv_rank + self.rot_dim + self.heads
        return 2 * self.lin_heads * (self.lin_dim + self.lin_vdim)

    def mixer_weight_elems(self, kind):
        W = self.width
        if kind == "latent":
            return self.n_in(kind) * W + self.heads * (self.dim + self.rot_dim) * self.q_rank + \
                self.heads * (self.dim + self.vdim) * self.kv_rank + W * self.heads * self.vdim
        return self.n_in(kind) * W + W * self.lin_heads * self.lin_vdim

    def ff_weight_elems(self, kind, pairs):
        W = self.width
        if kind == "dense":
            return 2 * self.dense_ff * W
        if kind == "moe":
            return self.experts * W + min(pairs, self.experts) * 2 * self.ff * W
        return 0

    def weight_elems_per_step(self, batch):
        """Matrix elements a decode step of `batch` sequences reads (distinct experts: an upper bound)."""
        total = self.vocab * self.width
        for i, _, _ in self.run_order():
            m, f = self.pattern[i]
            total += self.mixer_weight_elems(m) + self.ff_weight_elems(f, batch * self.top)
        return total

    def flops_per_token(self):
        total = self.vocab * self.width
        for i, _, _ in self.run_order():
            m, f = self.pattern[i]
            total += self.mixer_weight_elems(m) + self.ff_weight_elems(f, self.top) - (self.experts * 0 if f != "moe" else 0)
        return 2 * total

    def state_bytes_per_step(self, batch, ctx, es):
        """Cache and state a decode step touches: the window's latents, the linear-attention state (read and written)."""
        total = 0
        for i, _, _ in self.run_order():
            m, _ = self.pattern[i]
            if m == "latent":
                total += batch * min(ctx, self.window) * (self.kv_rank + self.rot_dim) * es
            else:
                total += batch * 2 * self.lin_heads * self.lin_dim * self.lin_vdim * 4
        return total


@dataclass
class VurazenShape:
    """A Vurazen model: `pattern` lists the layers ("mamba" | "lightning" | "parallel", "dense" | "moe" | None)."""
    name: str
    width: int
    vocab: int
    pattern: tuple
    loop: tuple          # (start, stop, times)
    inner: int           # selective scan
    state: int
    dt_rank: int
    lin_heads: int       # linear attention
    lin_dim: int
    lin_vdim: int
    heads: int           # window attention (values = keys)
    kv_heads: int
    dim: int
    window: int
    keep_first: int
    rot_dims: int
    d_heads: int         # delta rule
    d_kv_heads: int
    d_dim: int
    d_vdim: int
    d_rank: int
    dense_ff: int
    experts: int
    top: int
    ff: int
    shared_ff: int
    taps: int = 4
    eps: float = 1e-5

    @property
    def layers(self):
        return len(self.pattern)

    def run_order(self):
        s, e, t = self.loop
        order = [(i, -1, 0) for i in range(s)]
        for p in range(t):
            order += [(i, p if i == s else -1, 1 if i == s and p > 0 else 0) for i in range(s, e)]
        return order + [(i, -1, 0) for i in range(e, self.layers)]

    @property
    def runs(self):
        return len(self.run_order())

    def delta_in(self):
        return 2 * self.d_kv_heads * self.d_dim + self.d_heads * self.d_vdim + self.d_heads + 2 * self.d_rank

    def mixer_weight_elems(self, kind):
        W = self.width
        if kind == "mamba":
            return 2 * self.inner * W + (self.dt_rank + 2 * self.state) * self.inner + self.inner * self.dt_rank + W * self.inner
        if kind == "lightning":
            return 2 * self.lin_heads * (self.lin_dim + self.lin_vdim) * W + W * self.lin_heads * self.lin_vdim
        left = (self.heads + self.kv_heads) * self.dim * W + W * self.heads * self.dim
        right = self.delta_in() * W + self.d_heads * (self.d_dim + self.d_vdim) * self.d_rank + W * self.d_heads * self.d_vdim
        return left + right

    def ff_weight_elems(self, kind, pairs):
        W = self.width
        if kind == "dense":
            return 3 * self.dense_ff * W
        if kind == "moe":
            return self.experts * W + min(pairs, self.experts) * 3 * self.ff * W + 3 * self.shared_ff * W
        return 0

    def weight_elems_per_step(self, batch):
        """Matrix elements a decode step of `batch` sequences reads (distinct experts: an upper bound)."""
        total = self.vocab * self.width
        for i, _, _ in self.run_order():
            m, f = self.pattern[i]
            total += self.mixer_weight_elems(m) + self.ff_weight_elems(f, batch * self.top)
        return total

    def flops_per_token(self):
        total = self.vocab * self.width
        for i, _, _ in self.run_order():
            m, f = self.pattern[i]
            total += self.mixer_weight_elems(m) + self.ff_weight_elems(f, self.top)
        return 2 * total

    def state_bytes_per_step(self, batch, ctx, es):
        """Cache and state a decode step touches: the window's keys and values, the recurrent states (read and written)."""
        total = 0
        for i, _, _ in self.run_order():
            m, _ = self.pattern[i]
            if m == "mamba":
                total += batch * 2 * self.inner * self.state * 4
            elif m == "lightning":
                total += batch * 2 * self.lin_heads * self.lin_dim * self.lin_vdim * 4
            else:
                total += batch * min(ctx, self.window + self.keep_first) * 2 * self.kv_heads * self.dim * es
                total += batch * 2 * self.d_heads * self.d_dim * self.d_vdim * 4
        return total


@dataclass
class BukuvikShape:
    """A Bukuvik model: `pattern` lists the layers ("attention" | "parallel", feed-forward size or None)."""
    name: str
    width: int
    vocab: int
    pattern: tuple
    heads: int           # differential attention
    kv_heads: int
    dim: int
    vdim: int
    window: int
    rot_dims: int
    l_heads: int         # the pair's attention (unit-normed, rescaled rotation, kept first tokens)
    l_kv_heads: int
    l_dim: int
    l_vdim: int
    l_window: int
    l_keep_first: int
    l_rot_dims: int
    s_heads: int         # the pair's duality mixer
    s_vdim: int
    s_state: int
    s_groups: int
    s_norm_groups: int
    taps: int = 4
    softcap: float = 30.0
    diff: float = 0.2
    eps: float = 1e-5

    @property
    def layers(self):
        return len(self.pattern)

    @property
    def runs(self):
        return len(self.pattern)

    def run_order(self):
        return [(i, -1, 0) for i in range(self.layers)]

    def n_in(self, kind):
        if kind == "attention":
            return 2 * (self.heads + self.kv_heads) * self.dim + (self.kv_heads + self.heads) * self.vdim
        if kind == "left":
            return (self.l_heads + self.l_kv_heads) * self.l_dim + (self.l_kv_heads + self.l_heads) * self.l_vdim
        return 2 * self.s_heads * self.s_vdim + 2 * self.s_groups * self.s_state + self.s_heads

    def n_out(self, kind):
        return {"attention": self.heads * self.vdim, "left": self.l_heads * self.l_vdim, "right": self.s_heads * self.s_vdim}[kind]

    def mixer_weight_elems(self, kind):
        parts = ("attention",) if kind == "attention" else ("left", "right")
        return sum((self.n_in(k) + self.n_out(k)) * self.width for k in parts)

    def weight_elems_per_step(self, batch):
        return self.vocab * self.width + sum(self.mixer_weight_elems(m) + 2 * (f or 0) * self.width for m, f in self.pattern)

    def flops_per_token(self):
        return 2 * self.weight_elems_per_step(1)

    def state_bytes_per_step(self, batch, ctx, es):
        """Cache and state a decode step touches: the windows' keys and values, the duality state (read and written)."""
        total = 0
        for m, _ in self.pattern:
            if m == "attention":
                total += batch * min(ctx, self.window) * self.kv_heads * (2 * self.dim + self.vdim) * es
            else:
                total += batch * min(ctx, self.l_window + self.l_keep_first) * self.l_kv_heads * (self.l_dim + self.l_vdim) * es
                total += batch * 2 * self.s_heads * self.s_vdim * self.s_state * 4
        return total


class SeqEngine:
    """A random-weight model (Fobolorn, Kikunex, Vurazen or Bukuvik, by the shape's class) in device memory behind the engine's C-ABI."""

    def __init__(self, shape, dtype=BF16, max_tokens=4096, max_seqs=16, page=0, seed=1):
        import torch
        self.torch = torch
        self.lib = load_seq_library()
        self.shape, self.dtype = shape, dtype
        if isinstance(shape, KikunexShape):
            self._init_kikunex(shape, dtype, max_tokens, max_seqs, page, seed)
            return
        if isinstance(shape, VurazenShape):
            self._init_vurazen(shape, dtype, max_tokens, max_seqs, page, seed)
            return
        if isinstance(shape, BukuvikShape):
            self._init_bukuvik(shape, dtype, max_tokens, max_seqs, page, seed)
            return
        td = torch.bfloat16 if dtype == BF16 else torch.float32
        g = torch.Generator(device="cuda").manual_seed(seed)
        keep = self._keep = []
        W = shape.width

        def rnd(*dims, std, t=td):
            x = (torch.randn(*dims, device="cuda", generator=g) * std).to(t).contiguous()
            keep.append(x)
            return x

        def norm():
            w = rnd(W, std=0.05, t=torch.float32)
            w += 1
            return Norm(w.data_ptr(), rnd(W, std=0.05, t=torch.float32).data_ptr())

        layers = (Layer * shape.layers)()
        for L in layers:
            L.mixer_kind, L.ff_kind = 1, 1
            L.pre_mixer, L.post_mixer, L.pre_ff, L.post_ff = norm(), norm(), norm(), norm()
            a = L.attn
            a.heads, a.kv_heads, a.dim, a.vdim = shape.heads, shape.kv_heads, shape.dim, shape.vdim
            a.scale, a.temp_coef, a.temp_every, a.qk_norm, a.gate = shape.dim ** -0.5, shape.temp[0], shape.temp[1], 1, 1
            a.w_in = rnd(shape.n_in(), W, std=W ** -0.5).data_ptr()
            ones = rnd(shape.dim, std=0.05, t=torch.float32)
            ones += 1
            a.q_norm_w = a.k_norm_w = ones.data_ptr()
            a.w_out = rnd(W, shape.heads * shape.vdim, std=(shape.heads * shape.vdim) ** -0.5).data_ptr()
            m = L.moe
            m.experts, m.top, m.ff, m.router_scale = shape.experts, shape.top, shape.ff, 1.0
            m.w_router = rnd(shape.experts, W, std=W ** -0.5, t=torch.float32).data_ptr()
            m.gate_up = rnd(shape.experts, 2 * shape.ff, W, std=W ** -0.5).data_ptr()
            m.down = rnd(shape.experts, W, shape.ff, std=shape.ff ** -0.5).data_ptr()
            m.shared_ff = shape.shared_ff
            if shape.shared_ff:
                m.shared_gate_up = rnd(2 * shape.shared_ff, W, std=W ** -0.5).data_ptr()
                m.shared_down = rnd(W, shape.shared_ff, std=shape.shared_ff ** -0.5).data_ptr()
                m.w_shared_gate = rnd(W, std=W ** -0.5, t=torch.float32).data_ptr()
        order = shape.run_order()
        run_layer = (c_int32 * len(order))(*[i for i, _ in order])
        run_add = (c_int32 * len(order))(*[p for _, p in order])
        d = Desc()
        d.dtype, d.width, d.vocab, d.norm_eps = dtype, W, shape.vocab, shape.eps
        d.n_layers, d.layers = shape.layers, layers
        d.n_runs, d.run_layer, d.run_add = len(order), run_layer, run_add
        d.run_vectors = rnd(max(1, shape.loop[2]), W, std=0.1, t=torch.float32).data_ptr()
        d.embed = rnd(shape.vocab, W, std=1.0).data_ptr()
        d.final_norm = norm()
        d.head = rnd(shape.vocab, W, std=W ** -0.5).data_ptr()
        d.max_tokens, d.max_seqs, d.page_tokens = max_tokens, max_seqs, page
        self._desc = (d, layers, run_layer, run_add)
        self.handle = c_void_p()
        torch.cuda.synchronize()  # the engine runs on a stream of its own: the weights must be complete first
        _check(self.lib, self.lib.kllm_seq_create(ctypes.byref(d), None, ctypes.byref(self.handle)), "kllm_seq_create")

    def _init_kikunex(self, shape, dtype, max_tokens, max_seqs, page, seed):
        torch = self.torch
        td = torch.bfloat16 if dtype == BF16 else torch.float32
        g = torch.Generator(device="cuda").manual_seed(seed)
        keep = self._keep = []
        W = shape.width

        def rnd(*dims, std, t=td, mean=0.0):
            x = (torch.randn(*dims, device="cuda", generator=g) * std + mean).to(t).contiguous()
            keep.append(x)
            return x

        def f32(*dims, std, mean=0.0):
            return rnd(*dims, std=std, t=torch.float32, mean=mean)

        def norm():
            w = torch.full((W,), 1.0 + 0.05 * float(torch.randn((), generator=torch.Generator().manual_seed(len(keep)))),
                           device="cuda")
            keep.append(w)
            return Norm(w.data_ptr(), None, 1)

        layers = (Layer * shape.layers)()
        for L, (mix, ff) in zip(layers, shape.pattern):
            L.pre_mixer = norm()
            L.shift = f32(W, std=0.2, mean=0.5).data_ptr()
            if mix == "latent":
                L.mixer_kind = 2
                a = L.latent
                a.heads, a.dim, a.rot_dim, a.vdim = shape.heads, shape.dim, shape.rot_dim, shape.vdim
                a.q_rank, a.kv_rank, a.window = shape.q_rank, shape.kv_rank, shape.window
                a.scale, a.rope_dims, a.rope_base = (shape.dim + shape.rot_dim) ** -0.5, shape.rot_dim, 10000.0
                a.w_in = rnd(shape.n_in("latent"), W, std=W ** -0.5).data_ptr()
                a.q_norm_w = f32(shape.q_rank, std=0.05, mean=1.0).data_ptr()
                a.kv_norm_w = f32(shape.kv_rank, std=0.05, mean=1.0).data_ptr()
                a.w_uq = rnd(shape.heads * (shape.dim + shape.rot_dim), shape.q_rank, std=shape.q_rank ** -0.5).data_ptr()
                a.w_uk = rnd(shape.heads * shape.dim, shape.kv_rank, std=shape.kv_rank ** -0.5).data_ptr()
                a.w_uv = rnd(shape.heads * shape.vdim, shape.kv_rank, std=shape.kv_rank ** -0.5).data_ptr()
                a.sink = f32(shape.heads, std=1.0).data_ptr()
                a.w_out = rnd(W, shape.heads * shape.vdim, std=(shape.heads * shape.vdim) ** -0.5).data_ptr()
            else:
                L.mixer_kind = 3
                a = L.linear
                a.heads, a.dim, a.vdim = shape.lin_heads, shape.lin_dim, shape.lin_vdim
                decay = torch.tensor([math.exp(-1.0 / (4.0 * (h + 1))) for h in range(shape.lin_heads)], device="cuda")
                keep.append(decay)
                a.decay = decay.data_ptr()
                a.w_in = rnd(shape.n_in("lightning"), W, std=W ** -0.5).data_ptr()
                a.out_norm_w = f32(shape.lin_heads * shape.lin_vdim, std=0.05, mean=1.0).data_ptr()
                a.w_out = rnd(W, shape.lin_heads * shape.lin_vdim, std=(shape.lin_heads * shape.lin_vdim) ** -0.5).data_ptr()
            L.ff_kind = {None: 0, "moe": 1, "dense": 2}[ff]
            if ff is not None:
                L.pre_ff = norm()
            if ff == "dense":
                d = L.dense
                d.ff, d.act, d.act_a, d.act_b = shape.dense_ff, 2, 0.6, 1.1
                d.up = rnd(shape.dense_ff, W, std=W ** -0.5).data_ptr()
                d.down = rnd(W, shape.dense_ff, std=0.3 * shape.dense_ff ** -0.5).data_ptr()
            elif ff == "moe":
                m = L.moe
                m.experts, m.top, m.ff, m.router_scale = shape.experts, shape.top, shape.ff, 1.5
                m.router_kind, m.act = 1, 1
                m.groups, m.groups_keep = shape.groups
                m.w_router = f32(shape.experts, W, std=W ** -0.5).data_ptr()
                m.correction = f32(shape.experts, std=0.1).data_ptr()
                m.gate_up = rnd(shape.experts, shape.ff, W, std=W ** -0.5).data_ptr()
                m.down = rnd(shape.experts, W, shape.ff, std=0.3 * shape.ff ** -0.5).data_ptr()
        order = shape.run_order()
        run_layer = (c_int32 * len(order))(*[i for i, _, _ in order])
        run_add = (c_int32 * len(order))(*[p for _, p, _ in order])
        run_embed = (c_int32 * len(order))(*[x for _, _, x in order])
        d = Desc()
        d.dtype, d.width, d.vocab, d.norm_eps = dtype, W, shape.vocab, shape.eps
        d.n_layers, d.layers = shape.layers, layers
        d.n_runs, d.run_layer, d.run_add, d.run_embed = len(order), run_layer, run_add, run_embed
        d.run_vectors = f32(max(1, shape.loop[2]), W, std=0.1).data_ptr()
        d.embed = rnd(shape.vocab, W, std=1.0).data_ptr()
        d.embed_norm, d.final_norm = norm(), norm()
        d.head = rnd(shape.vocab, W, std=W ** -0.5).data_ptr()
        d.logit_scale = 0.5
        d.max_tokens, d.max_seqs, d.page_tokens = max_tokens, max_seqs, page
        self._desc = (d, layers, run_layer, run_add, run_embed)
        self.handle = c_void_p()
        torch.cuda.synchronize()
        _check(self.lib, self.lib.kllm_seq_create(ctypes.byref(d), None, ctypes.byref(self.handle)), "kllm_seq_create")

    def _init_vurazen(self, shape, dtype, max_tokens, max_seqs, page, seed):
        torch = self.torch
        td = torch.bfloat16 if dtype == BF16 else torch.float32
        g = torch.Generator(device="cuda").manual_seed(seed)
        keep = self._keep = []
        W = shape.width

        def rnd(*dims, std, t=td, mean=0.0):
            x = (torch.randn(*dims, device="cuda", generator=g) * std + mean).to(t).contiguous()
            keep.append(x)
            return x

        def f32(*dims, std, mean=0.0):
            return rnd(*dims, std=std, t=torch.float32, mean=mean)

        def norm():
            return Norm(f32(W, std=0.05, mean=1.0).data_ptr(), f32(W, std=0.05).data_ptr(), 0)

        layers = (Layer * shape.layers)()
        for L, (mix, ff) in zip(layers, shape.pattern):
            L.pre_mixer = norm()
            L.mixer_scale = L.mixer2_scale = 1.0
            if mix == "mamba":
                L.mixer_kind = 4
                a = L.ssm
                n = shape.inner
                a.inner, a.state, a.dt_rank, a.conv_taps = n, shape.state, shape.dt_rank, shape.taps
                a.w_in = rnd(2 * n, W, std=W ** -0.5).data_ptr()
                a.conv_w = f32(n, shape.taps, std=0.5).data_ptr()
                a.conv_b = f32(n, std=0.1).data_ptr()
                a.w_x = rnd(shape.dt_rank + 2 * shape.state, n, std=n ** -0.5).data_ptr()
                a.w_dt = f32(n, shape.dt_rank, std=shape.dt_rank ** -0.5).data_ptr()
                a.dt_b = f32(n, std=0.5, mean=-2.0).data_ptr()
                rates = -torch.rand(n, shape.state, device="cuda", generator=g) * 4.0 - 0.05
                keep.append(rates)
                a.a = rates.data_ptr()
                a.d = f32(n, std=1.0).data_ptr()
                a.w_out = rnd(W, n, std=0.5 * n ** -0.5).data_ptr()
            elif mix == "lightning":
                L.mixer_kind = 3
                a = L.linear
                a.heads, a.dim, a.vdim = shape.lin_heads, shape.lin_dim, shape.lin_vdim
                decay = torch.tensor([math.exp(-1.0 / (4.0 * (h + 1))) for h in range(shape.lin_heads)], device="cuda")
                keep.append(decay)
                a.decay = decay.data_ptr()
                a.w_in = rnd(2 * shape.lin_heads * (shape.lin_dim + shape.lin_vdim), W, std=W ** -0.5).data_ptr()
                a.out_norm_w = f32(shape.lin_heads * shape.lin_vdim, std=0.05, mean=1.0).data_ptr()
                a.w_out = rnd(W, shape.lin_heads * shape.lin_vdim, std=(shape.lin_heads * shape.lin_vdim) ** -0.5).data_ptr()
            else:
                L.mixer_kind, L.mixer2_kind = 1, 5
                L.mixer_scale, L.mixer2_scale = 0.6, 0.5
                a = L.attn
                a.heads, a.kv_heads, a.dim, a.vdim = shape.heads, shape.kv_heads, shape.dim, shape.dim
                C = (shape.heads + shape.kv_heads) * shape.dim
                a.scale, a.softcap, a.window, a.keep_first = shape.dim ** -0.5, 30.0, shape.window, shape.keep_first
                a.conv_taps, a.rope_dims, a.rope_base, a.rope_pairing, a.values_are_keys = shape.taps, shape.rot_dims, 1e4, 1, 1
                a.w_in = rnd(C, W, std=W ** -0.5).data_ptr()
                a.in_bias = f32(C, std=0.1).data_ptr()
                a.conv_w = f32(C, shape.taps, std=0.5).data_ptr()
                a.sink = f32(shape.heads, std=1.0).data_ptr()
                a.w_out = rnd(W, shape.heads * shape.dim, std=(shape.heads * shape.dim) ** -0.5).data_ptr()
                b = L.delta
                b.heads, b.kv_heads, b.dim, b.vdim = shape.d_heads, shape.d_kv_heads, shape.d_dim, shape.d_vdim
                b.conv_taps, b.decay_rank, b.gate_rank = shape.taps, shape.d_rank, shape.d_rank
                Cd = 2 * shape.d_kv_heads * shape.d_dim + shape.d_heads * shape.d_vdim
                b.w_in = rnd(shape.delta_in(), W, std=W ** -0.5).data_ptr()
                b.conv_w = f32(Cd, shape.taps, std=0.5).data_ptr()
                low2 = torch.zeros(shape.d_heads * (shape.d_dim + shape.d_vdim), 2 * shape.d_rank, device="cuda")
                low2[:shape.d_heads * shape.d_dim, :shape.d_rank] = torch.randn(
                    shape.d_heads * shape.d_dim, shape.d_rank, device="cuda", generator=g) * shape.d_rank ** -0.5
                low2[shape.d_heads * shape.d_dim:, shape.d_rank:] = torch.randn(
                    shape.d_heads * shape.d_vdim, shape.d_rank, device="cuda", generator=g) * shape.d_rank ** -0.5
                low2 = low2.to(td).contiguous()
                keep.append(low2)
                b.w_low2 = low2.data_ptr()
                b.dt_bias = f32(shape.d_heads * shape.d_dim, std=0.5, mean=-2.0).data_ptr()
                rate = torch.rand(shape.d_heads, device="cuda", generator=g) * 2.0 + 0.02
                keep.append(rate)
                b.rate = rate.data_ptr()
                b.out_norm_w = f32(shape.d_vdim, std=0.05, mean=1.0).data_ptr()
                b.w_out = rnd(W, shape.d_heads * shape.d_vdim, std=(shape.d_heads * shape.d_vdim) ** -0.5).data_ptr()
            L.ff_kind = {None: 0, "moe": 1, "dense": 2}[ff]
            L.parallel_ff = 0 if ff is None else 1
            if ff == "dense":
                d = L.dense
                d.ff, d.act = shape.dense_ff, 3
                d.up = rnd(2 * shape.dense_ff, W, std=W ** -0.5).data_ptr()
                d.down = rnd(W, shape.dense_ff, std=0.3 * shape.dense_ff ** -0.5).data_ptr()
            elif ff == "moe":
                m = L.moe
                m.experts, m.top, m.ff, m.router_scale = shape.experts, shape.top, shape.ff, 1.0
                m.router_kind, m.act, m.act_limit, m.act_alpha, m.shared_act_limit = 2, 4, 7.0, 1.702, 7.0
                m.w_router = f32(shape.experts, W, std=W ** -0.5).data_ptr()
                m.router_bias = f32(shape.experts, std=0.1).data_ptr()
                m.gate_up = rnd(shape.experts, 2 * shape.ff, W, std=W ** -0.5).data_ptr()
                m.down = rnd(shape.experts, W, shape.ff, std=0.3 * shape.ff ** -0.5).data_ptr()
                m.shared_ff = shape.shared_ff
                if shape.shared_ff:
                    m.shared_gate_up = rnd(2 * shape.shared_ff, W, std=W ** -0.5).data_ptr()
                    m.shared_down = rnd(W, shape.shared_ff, std=0.3 * shape.shared_ff ** -0.5).data_ptr()
        order = shape.run_order()
        run_layer = (c_int32 * len(order))(*[i for i, _, _ in order])
        run_add = (c_int32 * len(order))(*[p for _, p, _ in order])
        run_embed = (c_int32 * len(order))(*[x for _, _, x in order])
        d = Desc()
        d.dtype, d.width, d.vocab, d.norm_eps = dtype, W, shape.vocab, shape.eps
        d.n_layers, d.layers = shape.layers, layers
        d.n_runs, d.run_layer, d.run_add, d.run_embed = len(order), run_layer, run_add, run_embed
        d.run_vectors = f32(max(1, shape.loop[2]), W, std=0.1).data_ptr()
        d.embed = rnd(shape.vocab, W, std=1.0).data_ptr()
        d.final_norm = norm()
        d.head = rnd(shape.vocab, W, std=W ** -0.5).data_ptr()
        d.embed_scale, d.logit_softcap = 1.0, 30.0
        d.max_tokens, d.max_seqs, d.page_tokens = max_tokens, max_seqs, page
        self._desc = (d, layers, run_layer, run_add, run_embed)
        self.handle = c_void_p()
        torch.cuda.synchronize()
        _check(self.lib, self.lib.kllm_seq_create(ctypes.byref(d), None, ctypes.byref(self.handle)), "kllm_seq_create")

    def _init_bukuvik(self, shape, dtype, max_tokens, max_seqs, page, seed):
        torch = self.torch
        td = torch.bfloat16 if dtype == BF16 else torch.float32
        g = torch.Generator(device="cuda").manual_seed(seed)
        keep = self._keep = []
        W = shape.width

        def rnd(*dims, std, t=td, mean=0.0):
            x = (torch.randn(*dims, device="cuda", generator=g) * std + mean).to(t).contiguous()
            keep.append(x)
            return x

        def f32(*dims, std, mean=0.0):
            return rnd(*dims, std=std, t=torch.float32, mean=mean)

        def out_norm(scale=1.0):
            return Norm(f32(W, std=0.05 * scale, mean=scale).data_ptr(), None, 1)

        def frequencies(dims, base, factor=None):
            f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], device="cuda")
            if factor:  # the slow half of the waves is stretched
                f[dims // 4:] /= factor
            keep.append(f)
            return f.data_ptr()

        def attention(a, heads, kv_heads, dim, vdim, window, rot_dims, n_in):
            a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window = heads, kv_heads, dim, vdim, dim ** -0.5, window
            a.gate, a.rope_dims, a.rope_base, a.rope_pairing = 2, rot_dims, 1e4, 0
            a.w_in = rnd(n_in, W, std=W ** -0.5).data_ptr()
            a.w_out = rnd(W, heads * vdim, std=(heads * vdim) ** -0.5).data_ptr()

        layers = (Layer * shape.layers)()
        for L, (mix, ff) in zip(layers, shape.pattern):
            L.pre_mixer, L.pre_ff = Norm(None, None, 2), Norm(None, None, 2)
            L.post_mixer = out_norm(0.8)
            L.mixer_scale = L.mixer2_scale = 1.0
            if mix == "attention":
                L.mixer_kind = 1
                a = L.attn
                attention(a, shape.heads, shape.kv_heads, shape.dim, shape.vdim, shape.window, shape.rot_dims,
                          shape.n_in("attention"))
                a.qk_norm, a.softcap, a.differential = 1, shape.softcap, 1
                a.q_norm_w = f32(shape.dim, std=0.05, mean=1.0).data_ptr()
                a.k_norm_w = f32(shape.dim, std=0.05, mean=1.0).data_ptr()
                a.rope_freq, a.rope_mag = frequencies(shape.rot_dims, 1e6), 1.0
                a.diff_lambda, a.diff_out_scale = 0.8, 1.0 - shape.diff
            else:
                L.mixer_kind, L.mixer2_kind = 1, 6
                L.mixer_scale = L.mixer2_scale = 0.5
                L.mixer_out_norm, L.mixer2_out_norm = out_norm(), out_norm()
                a = L.attn
                attention(a, shape.l_heads, shape.l_kv_heads, shape.l_dim, shape.l_vdim, shape.l_window, shape.l_rot_dims,
                          shape.n_in("left"))
                a.qk_norm, a.keep_first = 2, shape.l_keep_first
                a.scale = 2.0 * shape.l_dim ** -0.5
                a.rope_freq, a.rope_mag = frequencies(shape.l_rot_dims, 1e4, 4.0), 0.1 * math.log(4.0) + 1.0
                b = L.ssd
                b.heads, b.vdim, b.state, b.groups = shape.s_heads, shape.s_vdim, shape.s_state, shape.s_groups
                b.conv_taps, b.norm_groups = shape.taps, shape.s_norm_groups
                inner, ch = shape.s_heads * shape.s_vdim, shape.s_heads * shape.s_vdim + 2 * shape.s_groups * shape.s_state
                b.w_in = rnd(shape.n_in("right"), W, std=W ** -0.5).data_ptr()
                b.conv_w = f32(ch, shape.taps, std=0.5).data_ptr()
                b.conv_b = f32(ch, std=0.1).data_ptr()
                b.dt_bias = f32(shape.s_heads, std=0.5, mean=-2.0).data_ptr()
                rates = -torch.rand(shape.s_heads, device="cuda", generator=g) * 4.0 - 0.05
                keep.append(rates)
                b.a = rates.data_ptr()
                b.d = f32(shape.s_heads, std=1.0).data_ptr()
                b.out_norm_w = f32(inner, std=0.05, mean=1.0).data_ptr()
                b.w_out = rnd(W, inner, std=inner ** -0.5).data_ptr()
            L.ff_kind = 2 if ff else 0
            if ff:
                L.post_ff = out_norm(0.8)
                d = L.dense
                d.ff, d.act = ff, 1
                d.up = rnd(ff, W, std=W ** -0.5).data_ptr()
                d.down = rnd(W, ff, std=ff ** -0.5).data_ptr()
        order = shape.run_order()
        run_layer = (c_int32 * len(order))(*[i for i, _, _ in order])
        run_add = (c_int32 * len(order))(*[p for _, p, _ in order])
        run_embed = (c_int32 * len(order))(*[x for _, _, x in order])
        d = Desc()
        d.dtype, d.width, d.vocab, d.norm_eps = dtype, W, shape.vocab, shape.eps
        d.n_layers, d.layers = shape.layers, layers
        d.n_runs, d.run_layer, d.run_add, d.run_embed = len(order), run_layer, run_add, run_embed
        d.embed = rnd(shape.vocab, W, std=1.0).data_ptr()
        d.final_norm = out_norm()
        d.head = d.embed  # the classifier is the embedding table
        d.embed_scale = W ** 0.5
        d.max_tokens, d.max_seqs, d.page_tokens = max_tokens, max_seqs, page
        self._desc = (d, layers, run_layer, run_add, run_embed)
        self.handle = c_void_p()
        torch.cuda.synchronize()
        _check(self.lib, self.lib.kllm_seq_create(ctypes.byref(d), None, ctypes.byref(self.handle)), "kllm_seq_create")

    def open(self):
        s = c_int32(-1)
        _check(self.lib, self.lib.kllm_seq_open(self.handle, ctypes.byref(s)), "kllm_seq_open")
        return s.value

    def close_seq(self, s):
        _check(self.lib, self.lib.kllm_seq_close(self.handle, s), "kllm_seq_close")

    def step(self, entries, want_last=True, profile=False):
        """entries: [(seq, [tokens])].  Returns (greedy ids of the last row of every entry, phase ms or None).
        Token ids go in from host memory and the ids come back to host memory: the call a server makes."""
        seqs = (c_int32 * len(entries))(*[s for s, _ in entries])
        counts = (c_int32 * len(entries))(*[len(t) for _, t in entries])
        flat = [x for _, t in entries for x in t]
        toks = (c_int32 * len(flat))(*flat)
        want, at = [], 0
        for _, t in entries:
            at += len(t)
            want.append(at - 1)
        n_want = len(want) if want_last else 0
        wantv = (c_int32 * max(1, len(want)))(*want)
        out = (c_int32 * max(1, len(want)))()
        ph = (c_float * len(PHASES))()
        if profile:
            self.lib.kllm_seq_profile(self.handle, ph)
        _check(self.lib, self.lib.kllm_seq_step(self.handle, len(entries), seqs, counts, toks, n_want, wantv, None, out),
               "kllm_seq_step")
        return list(out)[:n_want], (dict(zip(PHASES, ph)) if profile else None)

    def launches(self):
        return self.lib.kllm_seq_last_launches(self.handle)

    def close(self):
        if self.handle:
            self.lib.kllm_seq_destroy(self.handle)
            self.handle = c_void_p()
