"""Vurazen through the product path (bin/trace_run -> registry -> BatchScheduler -> sequence-batch engine and its
kernels) against the plain float64 restatement in tests/vurazen_oracle.py.  Small random models with bf16-representable
weights; --dtype float32 is compared tightly, bfloat16 loosely."""
import subprocess

import numpy as np
import pytest

import vurazen_oracle as vo
from seq_util import rel_err, run_trace, whole

pytestmark = pytest.mark.gpu
TOL32 = 1e-4   # fp32 kernels against float64: rounding only (a lost key, sink or state costs > 1e-2)
TOL16 = 4e-2   # bf16 products


def toks(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def ref_logits(cfg, w, tokens):
    return vo.forward(cfg, w, tokens)[0]


def single(rid, tokens, end=False):
    """One step per token."""
    steps = [{"entries": [{"id": rid, "tokens": [x], "want": [0]}]} for x in tokens]
    if end and steps:
        steps[-1]["end"] = [rid]
    return steps


def row_errors(got, ref):
    return np.array([rel_err(got[i:i + 1], ref[i:i + 1]) for i in range(len(ref))])


def assert_rows(got, ref, tol=TOL32):
    err = row_errors(got, ref)
    assert err.max() < tol, f"first bad position {int(np.argmax(err >= tol))} of {len(ref)}, worst {err.max():.3g}"


@pytest.fixture(scope="module")
def base(tmp_path_factory):
    """Every mixer and both feed-forwards, a loop of three passes over two layers, sizes that differ wherever they can
    (query and key/value heads, head sizes of the two side-by-side mixers, filters of 4 and 3 taps, a window that is no
    multiple of a key tile or a page, partly rotated heads, an expert limit that differs from the shared expert's)."""
    layers = [(vo.mamba_mixer(inner=40, state=6, dt_rank=3, conv=4), vo.dense_mlp(40)),
              (vo.parallel_mixer(vo.left_mixer(heads=4, kv_heads=2, dim=12, conv=4, window=21, keep_first=3, rot_dims=8),
                                 vo.right_mixer(heads=4, kv_heads=2, dim=10, vdim=6, conv=3)), vo.moe_mlp(6, 2, 16)),
              (vo.lightning_mixer(heads=2, dim=20, vdim=36, decay=[0.97, 0.999]), vo.moe_mlp(8, 3, 12, 0.8, (20, 1.5))),
              (vo.mamba_mixer(inner=24, state=5, dt_rank=2, conv=2), None)]
    cfg = vo.make_config(width=48, vocab=61, layers=layers, loop=(1, 3, 3))
    w = vo.make_weights(cfg, seed=1, sharp=3.0)
    return cfg, w, vo.write_model(tmp_path_factory.mktemp("vura_base"), cfg, w)


# ---- every mechanism on its own -------------------------------------------------------------------------------------
def par(left=None, right=None, **kw):
    return vo.parallel_mixer(vo.left_mixer(**(left or {})), vo.right_mixer(**(right or {})), **kw)


CASES = {
    "scan": [(vo.mamba_mixer(), None)],
    "scan_one_state": [(vo.mamba_mixer(inner=7, state=1, dt_rank=1, conv=2), None)],
    "scan_no_filter": [(vo.mamba_mixer(inner=16, state=3, dt_rank=2, conv=1), None)],
    "scan_long_filter": [(vo.mamba_mixer(inner=16, state=4, dt_rank=5, conv=7), None)],
    "scan_wide": [(vo.mamba_mixer(inner=200, state=40, dt_rank=9, conv=4), None)],      # more states than a warp has lanes
    "scan_many_states": [(vo.mamba_mixer(inner=20, state=100, dt_rank=4, conv=3), None)],  # 4 states on each of 32 lanes
    "lightning": [(vo.lightning_mixer(), None)],
    "lightning_one_decay": [(vo.lightning_mixer(heads=2, dim=8, vdim=8, decay=0.9), None)],
    "pair": [(par(), None)],
    "attention_alone": [(par(right_scale=0.0), None)],
    "delta_alone": [(par(left_scale=0.0), None)],
    "attention_every_head_its_keys": [(par(left=dict(heads=3, kv_heads=3), right_scale=0.0), None)],
    "attention_one_key_head": [(par(left=dict(heads=4, kv_heads=1, dim=16), right_scale=0.0), None)],
    "attention_no_filter": [(par(left=dict(conv=1), right_scale=0.0), None)],
    "attention_unrotated": [(par(left=dict(rot_dims=0), right_scale=0.0), None)],
    "attention_all_rotated": [(par(left=dict(dim=8, rot_dims=8, base=50.0), right_scale=0.0), None)],
    "attention_window_one": [(par(left=dict(window=1, keep_first=0), right_scale=0.0), None)],   # itself and the sink
    "attention_nothing_kept": [(par(left=dict(window=9, keep_first=0), right_scale=0.0), None)],
    "attention_many_kept": [(par(left=dict(window=5, keep_first=70), right_scale=0.0), None)],   # kept tokens past a key tile
    "attention_window_past_the_prompt": [(par(left=dict(window=500), right_scale=0.0), None)],
    "attention_tight_cap": [(par(left=dict(softcap=0.7, scale=1.0), right_scale=0.0), None)],
    "attention_wide": [(par(left=dict(heads=2, kv_heads=1, dim=72, rot_dims=20, window=40), right_scale=0.0), None)],
    "delta_every_head_its_keys": [(par(right=dict(heads=3, kv_heads=3), left_scale=0.0), None)],
    "delta_one_key_head": [(par(right=dict(heads=4, kv_heads=1, dim=5, vdim=9), left_scale=0.0), None)],
    "delta_no_filter": [(par(right=dict(conv=1), left_scale=0.0), None)],
    "delta_wide": [(par(right=dict(heads=2, kv_heads=2, dim=72, vdim=40, conv=4), left_scale=0.0), None)],  # rows of S over 4 lanes
    "delta_wider": [(par(right=dict(heads=2, kv_heads=1, dim=136, vdim=24, conv=2), left_scale=0.0), None)],  # 32 rows of S per thread
    "attention_widest": [(par(left=dict(heads=2, kv_heads=2, dim=136, rot_dims=136, window=33, keep_first=1), right_scale=0.0), None)],
    "dense_only": [(vo.lightning_mixer(), vo.dense_mlp(56))],
    "moe_only": [(vo.lightning_mixer(), vo.moe_mlp(6, 2, 16))],
    "moe_no_shared": [(vo.mamba_mixer(), vo.moe_mlp(5, 2, 16, 1.0, None))],
    "moe_top1": [(vo.mamba_mixer(), vo.moe_mlp(6, 1, 16, 0.5, (8, 2.0)))],
    "moe_many_experts": [(vo.mamba_mixer(), vo.moe_mlp(80, 5, 8))],     # more experts than a warp has lanes
    "moe_all_chosen": [(vo.lightning_mixer(), vo.moe_mlp(4, 4, 16))],
    "moe_beside_the_pair": [(par(), vo.moe_mlp(6, 2, 16))],
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_mechanism_alone(tmp_path, case):
    # a large eps in some cases: it must reach every norm (the layers', the delta rule's, the linear attention's)
    big_eps = case in ("lightning_one_decay", "delta_alone", "dense_only", "scan")
    cfg = vo.make_config(width=40, vocab=50, layers=CASES[case], eps=0.05 if big_eps else 3e-6,
                         logit_softcap=None if case == "scan_no_filter" else 6.0,
                         embed_scale=1.0 if case == "lightning" else 2.5)
    w = vo.make_weights(cfg, seed=3, sharp=3.0)
    if case in ("dense_only", "moe_only"):  # the mixer's output projection is zero: what is left of the layer is the feed-forward
        w["l0.mix.o"] = np.zeros_like(w["l0.mix.o"])
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(75, cfg["vocab"], 5)
    ref, trace = vo.forward(cfg, w, t)
    logits, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    assert np.abs(got - trace).max() < 1e-4 * max(1.0, np.abs(trace).max())
    assert_rows(logits[0], ref)


def test_residual_after_every_layer_run(base):
    cfg, w, d = base
    t = toks(33, cfg["vocab"], 7)
    _, trace = vo.forward(cfg, w, t)
    assert trace.shape[0] == 1 + 2 * 3 + 1
    _, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    for r in range(trace.shape[0]):
        assert np.abs(got[r] - trace[r]).max() < 1e-4 * max(1.0, np.abs(trace[r]).max()), f"layer run {r}"


@pytest.mark.parametrize("loop,runs", [((0, 2, 3), 7), ((1, 2, 1), 3), ((0, 3, 2), 6), ((2, 3, 4), 6), (None, 3)])
def test_loop_shapes(tmp_path, loop, runs):
    """Three passes, one pass (its vector is still added, the embedding output is not), a loop over every layer, a loop
    at the end, no loop: every pass has a cache and a state of its own."""
    layers = [(par(left=dict(window=9)), vo.dense_mlp(24)), (vo.mamba_mixer(), vo.moe_mlp(4, 2, 8)),
              (vo.lightning_mixer(), None)]
    cfg = vo.make_config(width=40, vocab=60, layers=layers, loop=loop)
    w = vo.make_weights(cfg, seed=101, sharp=2.0)
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(45, cfg["vocab"], 102)
    ref, trace = vo.forward(cfg, w, t)
    assert trace.shape[0] == runs
    logits, _ = run_trace(d, [whole("a", t[:30], end=False)] + single("a", t[30:]))
    assert_rows(np.concatenate(logits), ref)


@pytest.mark.parametrize("page", [4, 16, 64])
def test_long_prompt_every_position(base, page):
    cfg, w, d = base
    t = toks(203, cfg["vocab"], 11)  # past three key tiles of 64 and several chunks of the recurrences, no multiple of a page
    logits, _ = run_trace(d, [whole("a", t)], page=page)
    assert_rows(logits[0], ref_logits(cfg, w, t))


# ---- keys at the edges of the window and of the kept first tokens ---------------------------------------------------
def edge_model(window, keep_first, special, vocab=30, width=24, seed=9):
    """Attention alone, made so that ONE token's key wins every softmax it takes part in: every query is the same
    constant vector along the last (unrotated) coordinate of each head -- zero query weights, a bias -- and only the
    special token's key has a large entry there (the key weights read input coordinate 0, which only its embedding
    has).  The values are the keys, so while that key is seen the output is (almost) that key."""
    m = par(left=dict(heads=2, kv_heads=1, dim=8, conv=3, window=window, keep_first=keep_first, rot_dims=4, scale=1.0,
                      softcap=25.0), right_scale=0.0, left_scale=1.0)
    cfg = vo.make_config(width=width, vocab=vocab, layers=[(m, None)], embed_scale=1.0)
    w = vo.make_weights(cfg, seed=seed)
    p = "l0.mix.left."
    w[p + "q"] = np.zeros_like(w[p + "q"])
    w[p + "q.b"] = np.zeros_like(w[p + "q.b"])
    w[p + "q.b"][7::8] = 4.0
    for n in ("q.conv", "k.conv"):          # the filters pass the current token only
        w[p + n] = np.zeros_like(w[p + n])
        w[p + n][:, -1] = 1.0
    w[p + "k"][7] = 0.0
    w[p + "k"][7, 0] = 2.0
    w[p + "k.b"] = np.zeros_like(w[p + "k.b"])
    w["l0.norm1"] = np.ones_like(w["l0.norm1"])
    w["l0.norm1.b"] = np.zeros_like(w["l0.norm1.b"])
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 12.0
    return cfg, w


@pytest.mark.parametrize("window", [2, 17, 64, 65, 100])
def test_the_key_at_the_window_edge_carries_the_output(tmp_path, window):
    """The special key is placed so that it leaves the window inside the prompt, and a second one so that it leaves
    while tokens are decoded one by one (across key tiles and pages): the logits change completely at that position."""
    special = 7
    cfg, w = edge_model(window, 0, special)
    n_prompt, n_all = 150, 150 + window + 20
    t = [x if x != special else special + 1 for x in toks(n_all, cfg["vocab"], 13)]
    t[20] = special            # leaves the window inside the prompt
    t[n_prompt - 5] = special  # leaves it during decoding
    ref = ref_logits(cfg, w, t)
    for p in (20, n_prompt - 5):  # the construction works
        assert rel_err(ref[p + window:p + window + 1], ref[p + window - 1:p + window]) > 0.1
    d = vo.write_model(tmp_path, cfg, w)
    logits, _ = run_trace(d, [whole("a", t[:n_prompt], end=False)] + single("a", t[n_prompt:]), page=16)
    assert_rows(np.concatenate(logits), ref)


@pytest.mark.parametrize("keep,window", [(1, 3), (6, 10), (64, 5), (70, 33)])
def test_the_first_tokens_stay_and_the_next_one_leaves(tmp_path, keep, window):
    """The special token at the last kept position is seen for ever (far outside the window, in prompts and in decoding);
    at the first position that is not kept it leaves with the window."""
    special = 7
    for place, stays in ((keep - 1, True), (keep, False)):
        cfg, w = edge_model(window, keep, special)
        n_prompt, n_all = keep + window + 40, keep + window + 70
        t = [x if x != special else special + 1 for x in toks(n_all, cfg["vocab"], 14)]
        t[place] = special
        ref = ref_logits(cfg, w, t)
        t2 = list(t)
        t2[place] = special + 1
        far = rel_err(ref_logits(cfg, w, t2)[-1:], ref[-1:])
        assert (far > 0.1) == stays  # the construction works: the last logits depend on that token only while it is kept
        d = vo.write_model(tmp_path / f"{place}", cfg, w)
        logits, _ = run_trace(d, [whole("a", t[:n_prompt], end=False)] + single("a", t[n_prompt:]), page=8)
        assert_rows(np.concatenate(logits), ref)


def test_the_sink_takes_its_share(tmp_path):
    """Large sinks: most of the softmax mass goes to them, so leaving one out (or scaling or capping it) multiplies the output."""
    cfg = vo.make_config(width=32, vocab=40, layers=[(par(left=dict(heads=3, kv_heads=1, window=12, softcap=2.0),
                                                          right_scale=0.0), None)])
    w = vo.make_weights(cfg, seed=21)
    w["l0.mix.left.sink"] = np.array([4.0, -3.0, 1.5])
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(40, cfg["vocab"], 22)
    logits, _ = run_trace(d, [whole("a", t[:25], end=False)] + single("a", t[25:]))
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


@pytest.mark.parametrize("mixer", ["scan", "delta"])
def test_far_tokens_stay_in_the_recurrent_state(tmp_path, mixer):
    """Decays next to 1: what the first token wrote is still in the state hundreds of tokens, several chunks, two
    portions and many single steps later, and the last logits depend on it."""
    if mixer == "scan":
        layers = [(vo.mamba_mixer(inner=16, state=4, dt_rank=2, conv=3), None)]
    else:
        layers = [(par(right=dict(heads=2, kv_heads=1, dim=8, vdim=8), left_scale=0.0, right_scale=1.0), None)]
    cfg = vo.make_config(width=32, vocab=40, layers=layers, embed_scale=1.0)
    w = vo.make_weights(cfg, seed=31)
    special = 5
    t = [x if x != special else special + 1 for x in toks(330, cfg["vocab"], 32)]
    t[0] = special
    # only the special token's embedding has coordinate 0, so only its normed row is large there
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 6.0
    w["l0.norm1"][0] = 1.0
    if mixer == "scan":
        w["l0.mix.A_log"] = np.full_like(w["l0.mix.A_log"], vo.bf16_round(np.log(2e-4)))
        w["l0.mix.in"][:16, 0] = 6.0          # every channel's input reads that coordinate: the first token writes most
        w["l0.norm1.b"][0] = 0.0
    else:
        w["l0.mix.right.A_log"] = np.full_like(w["l0.mix.right.A_log"], vo.bf16_round(np.log(2e-4)))
        w["l0.mix.right.b"] = vo.bf16_round(w["l0.mix.right.b"] * 0.1)
        w["l0.mix.right.b"][:, 0] = 4.0       # beta is next to 1 for the first token ...
        w["l0.norm1.b"][0] = -3.0             # ... and next to 0 for every other one
    ref = ref_logits(cfg, w, t)
    t2 = list(t)
    t2[0] = special + 1
    assert rel_err(ref_logits(cfg, w, t2)[-1:], ref[-1:]) > 1e-2  # the construction works
    d = vo.write_model(tmp_path, cfg, w)
    # the second portion is long enough to be cut into segments that are scanned side by side, from a state that is not empty
    steps = [whole("a", t[:10], end=False), whole("a", t[10:300], end=False)] + single("a", t[300:])
    logits, _ = run_trace(d, steps)
    assert_rows(np.concatenate(logits), ref)


def test_long_entries_are_walked_in_segments(tmp_path):
    """Entries of several hundred rows: the recurrences cut them into segments that run side by side and are joined by a
    carry -- from an empty state, from a state that earlier rows left, beside a short entry, and with decoding afterwards."""
    layers = [(vo.mamba_mixer(inner=24, state=6, dt_rank=3, conv=4), None),
              (par(left=dict(window=30), right=dict(heads=4, kv_heads=2, dim=40, vdim=24, conv=3)), vo.dense_mlp(24))]
    cfg = vo.make_config(width=32, vocab=40, layers=layers, loop=(0, 2, 2))
    w = vo.make_weights(cfg, seed=91)
    d = vo.write_model(tmp_path, cfg, w)
    a, b = toks(5 + 600 + 3, cfg["vocab"], 92), toks(390 + 7, cfg["vocab"], 93)
    steps = [{"entries": [{"id": "a", "tokens": a[:5], "want": [4]}]},
             {"entries": [{"id": "a", "tokens": a[5:605], "want": list(range(600))},
                          {"id": "b", "tokens": b[:7], "want": list(range(7))}]},
             {"entries": [{"id": "b", "tokens": b[7:], "want": list(range(390))}]}] + single("a", a[605:])
    logits, _ = run_trace(d, steps, max_tokens=1100)
    ra, rb = ref_logits(cfg, w, a), ref_logits(cfg, w, b)
    assert_rows(np.concatenate([logits[0], logits[1][:600]] + logits[3:]), ra[4:])
    assert_rows(np.concatenate([logits[1][600:], logits[2]]), rb)


# ---- prompt against token-by-token decoding, long decoding ----------------------------------------------------------
def test_prefill_equals_stepwise_decoding(base):
    cfg, w, d = base
    t = toks(90, cfg["vocab"], 17)
    ref = ref_logits(cfg, w, t)
    split = [whole("p", t[:2], end=False)] + single("p", t[2:])
    logits, _ = run_trace(d, single("s", t) + split, page=8)   # "s": from the very first token
    a, b = np.concatenate(logits[:len(t)]), np.concatenate(logits[len(t):])
    assert_rows(a, ref)
    assert_rows(b, ref)
    assert_rows(a, b)


def test_long_decoding(base):
    """Decoding far past every window, key tile, page and chunk size."""
    cfg, w, d = base
    t = toks(40 + 260, cfg["vocab"], 19)
    logits, _ = run_trace(d, [whole("a", t[:40], end=False)] + single("a", t[40:]), page=16)
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


@pytest.mark.parametrize("sizes", [(2, 2, 2, 2), (5, 64, 3, 17), (33, 2, 70), (1, 99, 2), (1, 1, 2, 1, 40, 1, 2)])
def test_prompt_in_portions(base, sizes):
    """A prompt fed in several steps: every portion starts from the cache, the filters' histories and the recurrent
    states the portions before it left -- portions shorter than a filter's history too.  A second request of another
    length rides along."""
    cfg, w, d = base
    t = toks(sum(sizes), cfg["vocab"], 81)
    other = toks(2 * len(sizes) + 1, cfg["vocab"], 82)
    steps, at = [], 0
    for i, n in enumerate(sizes):
        o = other[2 * i:2 * i + 2] if i + 1 < len(sizes) else other[2 * i:]
        steps.append({"entries": [{"id": "o", "tokens": o, "want": list(range(len(o)))},
                                  {"id": "p", "tokens": t[at:at + n], "want": list(range(n))}]})
        at += n
    logits, _ = run_trace(d, steps, page=8, max_tokens=512)
    got_o = np.concatenate([lg[:len(st["entries"][0]["tokens"])] for lg, st in zip(logits, steps)])
    got_p = np.concatenate([lg[len(st["entries"][0]["tokens"]):] for lg, st in zip(logits, steps)])
    assert_rows(got_p, ref_logits(cfg, w, t))
    assert_rows(got_o, ref_logits(cfg, w, other))


# ---- batches ----------------------------------------------------------------------------------------------------------
def test_unequal_batch_equals_each_alone(base):
    cfg, w, d = base
    prompts = {"x": toks(1, cfg["vocab"], 21), "y": toks(67, cfg["vocab"], 22), "z": toks(130, cfg["vocab"], 23)}
    tails = {k: toks(n, cfg["vocab"], 30 + i) for i, (k, n) in enumerate({"x": 3, "y": 30, "z": 7}.items())}
    steps = [{"entries": [{"id": k, "tokens": p, "want": list(range(len(p)))} for k, p in prompts.items()]}]
    for j in range(30):
        live = [k for k in prompts if j < len(tails[k])]
        steps.append({"entries": [{"id": k, "tokens": [tails[k][j]], "want": [0]} for k in live],
                      "end": [k for k in live if j == len(tails[k]) - 1]})
    logits, _ = run_trace(d, steps, page=8, max_tokens=320)
    for k in prompts:
        rows, at = [], 0
        for kk, p in prompts.items():
            if kk == k:
                rows.append(logits[0][at:at + len(p)])
            at += len(p)
        for j in range(len(tails[k])):
            live = [kk for kk in prompts if j < len(tails[kk])]
            rows.append(logits[1 + j][live.index(k)][None])
        assert_rows(np.concatenate(rows), ref_logits(cfg, w, prompts[k] + tails[k]))


def test_pages_slots_and_states_are_reused(base):
    """The pool holds one request at a time: each runs in the pages, the slot and the state memory that the one before
    it gave back, and must see nothing of it."""
    cfg, w, d = base
    reqs = [toks(n, cfg["vocab"], 40 + i) for i, n in enumerate([50, 33, 64, 7, 50])]
    steps = []
    for i, t in enumerate(reqs):
        steps.append(whole(f"r{i}", t[:-3], end=False))
        steps += single(f"r{i}", t[-3:], end=True)
    logits, _ = run_trace(d, steps, page=4, max_tokens=64, extra=["--max-seqs", "1"])
    at = 0
    for t in reqs:
        assert_rows(np.concatenate(logits[at:at + 4]), ref_logits(cfg, w, t))
        at += 4


def test_a_freed_slot_restarts_from_an_empty_state(base):
    """Two slots; requests come and go in an order that hands a slot with a long history to a request that starts by
    decoding from its first token."""
    cfg, w, d = base
    a, b, c = toks(80, cfg["vocab"], 61), toks(12, cfg["vocab"], 62), toks(9, cfg["vocab"], 63)
    steps = [{"entries": [{"id": "a", "tokens": a, "want": [79]}, {"id": "b", "tokens": b[:6], "want": [5]}], "end": ["a"]}]
    for j in range(6):  # c takes a's slot and decodes from its first token beside b
        steps.append({"entries": [{"id": "b", "tokens": [b[6 + j]], "want": [0]}, {"id": "c", "tokens": [c[j]], "want": [0]}]})
    logits, _ = run_trace(d, steps, max_tokens=128, extra=["--max-seqs", "2"])
    got_b = np.concatenate([logits[0][1:2]] + [lg[0:1] for lg in logits[1:]])
    got_c = np.concatenate([lg[1:2] for lg in logits[1:]])
    assert_rows(got_b, ref_logits(cfg, w, b)[5:])
    assert_rows(got_c, ref_logits(cfg, w, c)[:6])
    assert_rows(logits[0][0:1], ref_logits(cfg, w, a)[79:])


def test_first_tokens_and_single_token_requests(base):
    cfg, w, d = base
    ts = [toks(n, cfg["vocab"], 50 + n) for n in (1, 2, 3, 4)]
    logits, _ = run_trace(d, [whole(f"q{i}", t) for i, t in enumerate(ts)])
    for t, lg in zip(ts, logits):
        assert_rows(lg, ref_logits(cfg, w, t))


def test_many_requests_in_one_batch(base):
    """80 prompts of 1..5 tokens in one step, then decoded together."""
    cfg, w, d = base
    reqs = [toks(1 + i % 5, cfg["vocab"], 200 + i) + toks(2, cfg["vocab"], 400 + i) for i in range(80)]
    steps = [{"entries": [{"id": f"r{i}", "tokens": r[:-2], "want": [len(r) - 3]} for i, r in enumerate(reqs)]}]
    for j in (2, 1):
        steps.append({"entries": [{"id": f"r{i}", "tokens": [r[-j]], "want": [0]} for i, r in enumerate(reqs)]})
    logits, _ = run_trace(d, steps, max_tokens=1024)
    for i, r in enumerate(reqs):
        got = np.stack([logits[0][i], logits[1][i], logits[2][i]])
        assert_rows(got, ref_logits(cfg, w, r)[-3:])


# ---- bf16, other sizes, generation ------------------------------------------------------------------------------------
def test_bfloat16_products(tmp_path):
    """bf16 products round the router's input too: every expert is chosen, so that no routing flip drowns the comparison."""
    layers = [(vo.mamba_mixer(inner=48, state=8, dt_rank=4, conv=4), vo.dense_mlp(40)),
              (par(left=dict(window=21)), vo.moe_mlp(4, 4, 16)),
              (vo.lightning_mixer(heads=2, dim=20, vdim=36), None)]
    cfg = vo.make_config(width=72, vocab=101, layers=layers, loop=(0, 2, 2))
    w = vo.make_weights(cfg, seed=5)
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(140, cfg["vocab"], 61)
    logits, _ = run_trace(d, [whole("a", t[:120], end=False)] + single("a", t[120:]), dtype="bfloat16")
    assert rel_err(np.concatenate(logits), ref_logits(cfg, w, t)) < TOL16


@pytest.mark.parametrize("dim,window,keep", [(24, 17, 0), (64, 64, 3), (128, 150, 70), (256, 100, 5)])
def test_bfloat16_prompts_on_the_tensor_cores(tmp_path, dim, window, keep):
    """bf16 prompt steps with head sizes that are multiples of 8 take the tensor-core attention (window, kept first
    tokens, capped scores, sink): against the float64 restatement, and against single-token steps of the same run.
    Heads of 256 are their own values, which is past the tensor-core kernel's value size: they take the split-key kernel."""
    m = par(left=dict(heads=4, kv_heads=2, dim=dim, rot_dims=16, window=window, keep_first=keep, softcap=8.0),
            right_scale=0.0, left_scale=1.0)
    cfg = vo.make_config(width=64, vocab=80, layers=[(m, None)])
    w = vo.make_weights(cfg, seed=41)
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(260, cfg["vocab"], 42)
    ref = ref_logits(cfg, w, t)
    steps = [whole("a", t, end=True), whole("b", t[:200], end=False)] + single("b", t[200:])
    logits, _ = run_trace(d, steps, dtype="bfloat16")
    assert rel_err(logits[0], ref) < TOL16
    assert rel_err(np.concatenate(logits[1:]), ref) < TOL16
    assert rel_err(np.concatenate(logits[2:]), logits[0][200:]) < TOL16


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_sizes_that_fit_no_vector(tmp_path, dtype, tol):
    """Odd sizes everywhere: no 16-byte vector load, no tensor-core tile and no warp-sized loop fits."""
    layers = [(vo.mamba_mixer(inner=13, state=3, dt_rank=1, conv=3), vo.dense_mlp(11)),
              (par(left=dict(heads=3, kv_heads=1, dim=6, rot_dims=2, window=7, keep_first=1, conv=2),
                   right=dict(heads=3, kv_heads=3, dim=5, vdim=7, conv=5)), vo.moe_mlp(3, 3, 7, 1.0, (5, 0.5))),
              (vo.lightning_mixer(heads=1, dim=5, vdim=3, decay=[0.9]), None)]
    cfg = vo.make_config(width=22, vocab=23, layers=layers, loop=(1, 2, 2))
    w = vo.make_weights(cfg, seed=51)
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(77, cfg["vocab"], 52)
    logits, _ = run_trace(d, [whole("a", t[:70], end=False)] + single("a", t[70:]), dtype=dtype)
    assert rel_err(np.concatenate(logits), ref_logits(cfg, w, t)) < tol


def test_larger_shapes_take_the_block_paths(tmp_path):
    """Width and inner sizes past one tile, enough tokens for the grouped expert products and the chunked recurrences."""
    layers = [(vo.mamba_mixer(inner=160, state=16, dt_rank=10, conv=4), vo.dense_mlp(192)),
              (par(left=dict(heads=4, kv_heads=2, dim=32, rot_dims=16, window=100, keep_first=4),
                   right=dict(heads=4, kv_heads=2, dim=64, vdim=32, conv=4)), vo.moe_mlp(8, 2, 64, 1.5, (64, 1.5))),
              (vo.lightning_mixer(heads=2, dim=32, vdim=32), vo.moe_mlp(8, 2, 64))]
    cfg = vo.make_config(width=128, vocab=200, layers=layers)
    w = vo.make_weights(cfg, seed=61)
    d = vo.write_model(tmp_path, cfg, w)
    t = toks(300, cfg["vocab"], 62)
    ref = ref_logits(cfg, w, t)
    logits, _ = run_trace(d, [whole("a", t[:290], end=False)] + single("a", t[290:]))
    assert_rows(np.concatenate(logits), ref)
    lb, _ = run_trace(d, [whole("a", t)], dtype="bfloat16")
    err = row_errors(lb[0], ref)  # a routing flip under bf16 rounding costs single rows
    assert np.median(err) < TOL16 / 2 and (err > TOL16).mean() <= 0.05, np.sort(err)[-5:]


def random_design(seed):
    rng = np.random.default_rng(seed)

    def pick(*xs):
        return xs[int(rng.integers(len(xs)))]

    def mixer():
        kind = pick("scan", "lightning", "pair")
        if kind == "scan":
            return vo.mamba_mixer(inner=pick(8, 24, 40), state=pick(1, 4, 9), dt_rank=pick(1, 3, 6), conv=pick(1, 2, 4))
        if kind == "lightning":
            h = pick(1, 2, 3)
            return vo.lightning_mixer(heads=h, dim=pick(4, 8, 20), vdim=pick(4, 12),
                                      decay=pick(0.95, [float(x) for x in rng.uniform(0.5, 1.0, h)]))
        g = pick(1, 2)
        dim = pick(4, 8, 12)
        left = vo.left_mixer(heads=g * pick(1, 2), kv_heads=g, dim=dim, conv=pick(1, 2, 4), window=pick(1, 5, 30, 66),
                             keep_first=pick(0, 1, 7), rot_dims=pick(0, 2, dim), base=pick(100.0, 10000.0),
                             softcap=pick(None, 3.0, 30.0))
        g = pick(1, 2)
        right = vo.right_mixer(heads=g * pick(1, 3), kv_heads=g, dim=pick(3, 8, 16), vdim=pick(2, 8), conv=pick(1, 3))
        return vo.parallel_mixer(left, right, left_scale=pick(0.3, 1.0), right_scale=pick(0.5, 1.2))

    def mlp():
        kind = pick(None, "dense", "moe")
        if kind == "dense":
            return vo.dense_mlp(pick(8, 30))
        if kind == "moe":
            e = pick(2, 5, 9)
            return vo.moe_mlp(e, pick(1, 2, e), pick(4, 12), pick(0.5, 2.0), pick(None, (6, 1.0)))
        return None

    n = int(rng.integers(1, 5))
    layers = [(mixer(), mlp()) for _ in range(n)]
    start = int(rng.integers(0, n))
    stop = int(rng.integers(start, n + 1))
    loop = (start, stop, int(rng.integers(1, 4))) if stop > start and rng.random() < 0.7 else None
    cfg = vo.make_config(width=pick(16, 24, 40), vocab=pick(17, 50), layers=layers, loop=loop, eps=pick(1e-6, 1e-3),
                         logit_softcap=pick(None, 5.0, 30.0), embed_scale=pick(1.0, 0.5, 4.0))
    return cfg


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_designs(tmp_path, seed):
    """Layer order, sizes and constants drawn at random; a ragged batch that is prefilled together and decoded together,
    in float32 (tight) and bfloat16 (loose; routing flips cost single rows)."""
    cfg = random_design(seed)
    w = vo.make_weights(cfg, seed=100 + seed, sharp=2.0)
    d = vo.write_model(tmp_path, cfg, w)
    reqs = {"a": toks(90, cfg["vocab"], 300 + seed), "b": toks(23, cfg["vocab"], 400 + seed), "c": toks(6, cfg["vocab"], 500 + seed)}
    n_dec = 5
    steps = [{"entries": [{"id": k, "tokens": r[:-n_dec], "want": list(range(len(r) - n_dec))} for k, r in reqs.items()]}]
    for j in range(n_dec):
        steps.append({"entries": [{"id": k, "tokens": [r[len(r) - n_dec + j]], "want": [0]} for k, r in reqs.items()]})
    refs = {k: ref_logits(cfg, w, r) for k, r in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        logits, _ = run_trace(d, steps, dtype=dtype, page=8, max_tokens=256)
        at, loose = 0, []
        for i, (k, r) in enumerate(reqs.items()):
            n = len(r) - n_dec
            got = np.concatenate([logits[0][at:at + n]] + [logits[1 + j][i:i + 1] for j in range(n_dec)])
            at += n
            if dtype == "float32":
                assert_rows(got, refs[k])
            else:
                loose.append(row_errors(got, refs[k]))
        if loose:
            err = np.concatenate(loose)
            assert np.median(err) < TOL16 / 2 and (err > TOL16).mean() <= 0.05, np.sort(err)[-5:]


def test_greedy_generation_through_the_scheduler(base):
    from kuiperllama_b200 import build
    cfg, w, d = base
    tools = build.build_seq_tools()
    prompts = [toks(9, cfg["vocab"], 71), toks(30, cfg["vocab"], 72), toks(2, cfg["vocab"], 73)]
    cmd = [str(tools / "kuiper_generate"), "--model", str(d), "--dtype", "float32", "--new", "12", "--page", "8"]
    for p in prompts:
        cmd += ["--prompt", " ".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(x) for x in ln.split()] for ln in r.stdout.strip().splitlines()]
    for p, g in zip(prompts, got):
        assert g == vo.greedy(cfg, w, p, 12)
