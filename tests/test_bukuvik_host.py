"""Bukuvik without a GPU: the float64 restatement's own pieces against closed forms, the model-folder checks of the loader."""
import math
import subprocess

import numpy as np
import pytest

import bukuvik_oracle as bo


@pytest.fixture(scope="module")
def tools():
    from kuiperllama_b200 import build
    return build.build_seq_tools()


def small():
    cfg = bo.make_config(layers=[(bo.parallel_mixer(), 20), (bo.diff_mixer(), None)])
    return cfg, bo.make_weights(cfg)


def trace_cmd(tools, d, out):
    return [str(tools / "kuiper_trace"), "--model", str(d), "--out", str(out), "--dtype", "float32"]


def test_missing_tensors_and_unknown_kinds_are_reported(tools, tmp_path):
    cfg, w = small()
    for missing in ("l0.mix.left.g", "l0.mix.left.out", "l0.mix.right.A_log", "l0.mix.right.conv.b", "l0.ls2", "l0.norm2",
                    "l1.mix.k.norm", "l1.mix.lq2", "l1.mix.g", "l1.ls1", "final.norm", "embed"):
        d = bo.write_model(tmp_path / missing, cfg, {k: v for k, v in w.items() if k != missing})
        r = subprocess.run(trace_cmd(tools, d, tmp_path), capture_output=True, text=True)
        assert r.returncode == 2 and missing in r.stderr, (missing, r.stderr)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="convolution")])
    r = subprocess.run(trace_cmd(tools, bo.write_model(tmp_path / "bad", bad, w), tmp_path), capture_output=True, text=True)
    assert r.returncode == 2 and "convolution" in r.stderr
    bad = dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "routed", "ff": 20})])
    r = subprocess.run(trace_cmd(tools, bo.write_model(tmp_path / "bad2", bad, w), tmp_path), capture_output=True, text=True)
    assert r.returncode == 2 and "routed" in r.stderr


def test_short_convolution():
    # three taps: the last column weighs the current row, zeros before the start
    u = np.array([[1.0], [2.0], [4.0]])
    assert np.allclose(bo.short_conv(u, np.array([[100.0, 10.0, 1.0]]), [0.0])[:, 0], [1.0, 12.0, 124.0])
    assert np.allclose(bo.short_conv(u, np.array([[1.0]]), [0.5])[:, 0], [1.5, 2.5, 4.5])


def test_rotation_pairs_a_coordinate_with_the_one_half_the_rotated_size_on():
    v = (np.arange(6, dtype=np.float64) + 1).reshape(1, 1, 6)
    r = bo.rotate_halves(v, np.array([3.0]), bo.rot(4, 100.0))[0, 0]
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(r[:4], [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                               3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)])
    assert np.allclose(r[4:], [5.0, 6.0])
    assert np.allclose(bo.rotate_halves(v, np.array([3.0]), bo.rot(0)), v)


def test_rescaled_frequencies():
    """Eight pairs over base 10000, original length 64: waves with more than 4 turns over it stay, those with fewer
    than 1 turn are slowed by the factor, the pairs between are blended; cos and sin grow by 0.1 ln(factor) + 1."""
    r = bo.rot(16, 10000.0, (4.0, 64, 4.0, 1.0))
    f, mag = bo.rotary_frequencies(r)
    plain = 10000.0 ** (-2.0 * np.arange(8) / 16)
    turns = 64 * plain / (2 * math.pi)
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    assert np.allclose(f[turns > 4.0], plain[turns > 4.0])
    slow = turns < 1.0
    lo = math.floor(16 * math.log(64 / (2 * math.pi * 4.0)) / (2 * math.log(10000.0)))
    hi = math.ceil(16 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(10000.0)))
    assert np.allclose(f[hi:], plain[hi:] / 4.0) and slow[hi:].all()
    mid = np.arange(8)[lo + 1:hi]
    assert ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 4.0)).all()
    # without scaling: the plain table and a factor of one
    f0, mag0 = bo.rotary_frequencies(bo.rot(16, 10000.0))
    assert np.allclose(f0, plain) and mag0 == 1.0


def test_window_and_kept_tokens():
    m = bo.visible(6, 2, 1)
    want = np.array([[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 0, 1, 1, 0, 0], [1, 0, 0, 1, 1, 0],
                     [1, 0, 0, 0, 1, 1]], dtype=bool)
    assert (m == want).all()
    assert (bo.visible(4, 0, 0) == np.tril(np.ones((4, 4), dtype=bool))).all()
    assert (bo.visible(4, 1, 0) == np.eye(4, dtype=bool)).all()


def test_uniform_maps_cancel_in_a_differential_head():
    """Zero queries make both maps the running mean of the values: a1 - lambda a2 = (1 - lambda) mean, and the unit norm
    that follows leaves its direction; lambda > 1 flips the sign."""
    cfg = bo.make_config(width=8, vocab=5, layers=[(bo.diff_mixer(heads=1, kv_heads=1, dim=4, vdim=8, window=100, rot_dims=0), None)])
    w = bo.make_weights(cfg, seed=2)
    p = "l0.mix."
    w[p + "q"] = np.zeros_like(w[p + "q"])
    w[p + "g"] = np.zeros_like(w[p + "g"])   # gate 1/2 everywhere
    w[p + "o"] = np.eye(8)
    h = np.random.default_rng(0).standard_normal((5, 8))
    for lq, sign in ((0.0, 1.0), (1.0, -1.0)):   # lambda = diff, then e - 1 + diff > 1
        w[p + "lq1"], w[p + "lk1"] = np.full(4, lq), np.full(4, 0.25)
        w[p + "lq2"], w[p + "lk2"] = np.zeros(4), np.zeros(4)
        lam = bo.differential_lambda(w, p, 0.25)
        assert math.isclose(lam, math.exp(lq) - 1.0 + 0.25)
        out = bo.differential_attention(h, w, p, cfg["layers"][0]["mixer"], 1e-30)
        mean = np.cumsum(h @ w[p + "v"].T, axis=0) / np.arange(1, 6)[:, None]
        want = sign * mean / np.sqrt((mean ** 2).mean(-1, keepdims=True)) * 0.75 * 0.5
        assert np.allclose(out, want)


def test_duality_recurrence_in_closed_form():
    """One head, one state, one value, no filter: S_t = exp(-A dt) S_(t-1) + dt B_t x_t and y_t = C_t S_t + D x_t with a
    constant step size is a geometric sum."""
    m = bo.right_mixer(heads=1, vdim=1, state=1, groups=1, conv=1, norm_groups=1)
    W = 3
    w_in = np.zeros((5, W))            # z | x | B | C | dt
    w_in[0, 0], w_in[1, 1], w_in[2, 2], w_in[3, 2] = 1.0, 1.0, 1.0, 1.0
    w = {"p.in": w_in, "p.conv": np.ones((3, 1)), "p.conv.b": np.zeros(3), "p.dt_bias": np.array([0.3]),
         "p.A_log": np.array([math.log(0.5)]), "p.D": np.array([2.0]), "p.norm": np.ones(1), "p.o": np.ones((1, 1))}
    h = np.array([[0.7, 1.0, 0.5], [0.7, -2.0, 1.5], [0.7, 0.25, -1.0]])
    dt = math.log1p(math.exp(0.3))
    dec = math.exp(-0.5 * dt)
    x, bc = bo.silu(h[:, 1]), bo.silu(h[:, 2])
    S, ys = 0.0, []
    for t in range(3):
        S = dec * S + dt * bc[t] * x[t]
        ys.append(bc[t] * S + 2.0 * x[t])
    gated = np.array(ys) * bo.silu(0.7)
    want = gated / np.sqrt(gated ** 2 + 1e-3)   # a norm part of one value
    assert np.allclose(bo.duality(h, w, "p.", m, 1e-3)[:, 0], want)
