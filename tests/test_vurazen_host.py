"""Vurazen without a GPU: the float64 restatement's own pieces against closed forms, the model-folder checks of the loader."""
import math
import subprocess

import numpy as np
import pytest

import vurazen_oracle as vo


@pytest.fixture(scope="module")
def tools():
    from kuiperllama_b200 import build
    return build.build_seq_tools()


def small():
    layers = [(vo.mamba_mixer(), vo.moe_mlp()), (vo.parallel_mixer(), vo.dense_mlp()), (vo.lightning_mixer(), None)]
    cfg = vo.make_config(layers=layers, loop=(0, 1, 2))
    return cfg, vo.make_weights(cfg)


def test_missing_tensors_and_unknown_mixers_are_reported(tools, tmp_path):
    cfg, w = small()
    for missing in ("l0.mix.A_log", "l0.norm1.b", "l1.mix.left.k.b", "l1.mix.right.dt_bias", "l2.mix.norm",
                    "l0.mlp.e3.down", "l0.mlp.shared.up", "l0.mlp.router.b", "l1.mlp.gate", "final.norm.b"):
        d = vo.write_model(tmp_path / missing, cfg, {k: v for k, v in w.items() if k != missing})
        r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                           capture_output=True, text=True)
        assert r.returncode == 2 and missing in r.stderr, (missing, r.stderr)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="convolution")])
    d = vo.write_model(tmp_path / "bad", bad, w)
    r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "convolution" in r.stderr


def test_layer_runs():
    cfg = vo.make_config(layers=[(vo.lightning_mixer(), None)] * 4, loop=(1, 3, 3))
    assert vo.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert vo.layer_runs(vo.make_config(layers=[(vo.lightning_mixer(), None)] * 2)) == [(0, None), (1, None)]


def test_router_takes_the_largest_logits():
    w = {"p.router": np.eye(5), "p.router.b": np.array([0.0, 0.0, 0.0, 2.0, 0.0])}
    h = np.array([[3.0, 1.0, 2.5, 1.2, -4.0]])
    idx, wt = vo.route(h, w, "p.", {"experts": 5, "top": 3})
    assert list(idx[0]) == [3, 0, 2]  # the bias lifts expert 3 to 3.2
    e = np.exp(np.array([3.2, 3.0, 2.5]) - 3.2)
    assert np.allclose(wt[0], e / e.sum())
    idx, wt = vo.route(h, w, "p.", {"experts": 5, "top": 1})
    assert list(idx[0]) == [3] and np.allclose(wt, 1.0)


def test_oracle_pieces():
    """The restatement's own pieces against closed forms."""
    # a filter of three taps: the last column weighs the current row, zeros before the start
    u = np.array([[1.0], [2.0], [4.0]])
    assert np.allclose(vo.short_conv(u, np.array([[100.0, 10.0, 1.0]]))[:, 0], [1.0, 12.0, 124.0])
    assert np.allclose(vo.short_conv(u, np.array([[1.0]]), np.array([0.5]))[:, 0], [1.5, 2.5, 4.5])
    # rotary positions on neighbouring pairs of the first four coordinates
    v = (np.arange(6, dtype=np.float64) + 1).reshape(1, 1, 6)
    r = vo.rotate_pairs(v, np.array([3.0]), 4, 100.0)[0, 0]
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(r[:4], [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
                               3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)])
    assert np.allclose(r[4:], [5.0, 6.0])
    # the experts' activation: the gate is cut from above only, the up product on both sides
    w = {"e.gate": np.array([[1.0]]), "e.up": np.array([[1.0]]), "e.down": np.array([[1.0]])}
    for x, g, uu in ((5.0, 2.0, 2.0), (-5.0, -5.0, -2.0), (1.0, 1.0, 1.0)):
        want = g / (1.0 + math.exp(-1.702 * g)) * (uu + 1.0)
        assert math.isclose(vo.clamped_expert(np.array([[x]]), w, "e.", 2.0)[0, 0], want)
    assert np.allclose(vo.layer_norm(np.array([[1.0, 3.0]]), np.array([2.0, 2.0]), np.array([0.5, 0.5]), 0.0), [[-1.5, 2.5]])


def test_delta_rule_writes_and_reads_one_association():
    """One head, unit keys: after a token with beta = 1 is written into an empty state, reading with the same key
    returns its value (before the norm and gate), whatever the decay."""
    k = np.array([0.6, 0.8])
    v = np.array([2.0, -1.0, 0.5])
    S = np.zeros((2, 3))
    S = 0.5 * S
    S = S + np.outer(k, 1.0 * (v - S.T @ k))
    assert np.allclose(S.T @ k, v)
    # a second write along the same key with beta = 1 replaces the value
    S = 0.9 * S
    v2 = np.array([0.0, 3.0, 1.0])
    S = S + np.outer(k, v2 - S.T @ k)
    assert np.allclose(S.T @ k, v2)


def test_window_and_kept_tokens_in_the_restatement():
    """Uniform attention (zero queries, sinks far below): the output at position i is the mean of the keys it sees."""
    m = vo.left_mixer(heads=1, kv_heads=1, dim=2, conv=1, window=2, keep_first=1, rot_dims=0, softcap=None)
    W = 2
    w = {"p.q": np.zeros((2, W)), "p.q.b": np.zeros(2), "p.k": np.eye(2), "p.k.b": np.zeros(2),
         "p.q.conv": np.ones((2, 1)), "p.k.conv": np.ones((2, 1)), "p.sink": np.array([-50.0]), "p.o": np.eye(2)}
    h = np.array([[1.0, 0.0], [2.0, 0.0], [4.0, 0.0], [8.0, 0.0], [16.0, 0.0]])
    out = vo.window_attention(h, w, "p.", m, 1e-6)[:, 0]
    assert np.allclose(out, [1.0, 1.5, (1 + 2 + 4) / 3, (1 + 4 + 8) / 3, (1 + 8 + 16) / 3])
