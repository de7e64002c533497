"""Bukuvik through the product path (bin/trace_run -> registry -> BatchScheduler -> sequence-batch engine and its
kernels) against the plain float64 restatement in tests/bukuvik_oracle.py.  Small random models with bf16-representable
weights; --dtype float32 is compared tightly, bfloat16 loosely."""
import subprocess

import numpy as np
import pytest

import bukuvik_oracle as bo
from seq_util import rel_err, run_trace, whole

pytestmark = pytest.mark.gpu
TOL32 = 1e-4   # fp32 kernels against float64: rounding only (a lost key, map or state costs > 1e-2)
TOL16 = 4e-2   # bf16 products


def toks(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def ref_logits(cfg, w, tokens):
    return bo.forward(cfg, w, tokens)[0]


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


def par(left=None, right=None):
    return bo.parallel_mixer(bo.left_mixer(**(left or {})), bo.right_mixer(**(right or {})))


def mute(w, layer, side):
    """A 'parallel' layer with one of its mixers silenced (the weight of that mixer's output norm is zero)."""
    name = f"l{layer}.mix.{side}.out"
    w[name] = np.zeros_like(w[name])


@pytest.fixture(scope="module")
def base(tmp_path_factory):
    """Both kinds of layer twice, with sizes that differ wherever they can: query and key/value heads, key and value
    sizes, state and value sizes, groups and norm parts, filters of 4 and 2 taps, windows that are no multiple of a key
    tile or a page, partly rotated heads, with and without a feed-forward."""
    layers = [(par(left=dict(heads=4, kv_heads=2, dim=12, vdim=8, window=21, keep_first=3, rot_dims=8),
                   right=dict(heads=6, vdim=5, state=7, groups=3, conv=4, norm_groups=2)), 40),
              (bo.diff_mixer(heads=4, kv_heads=2, dim=10, vdim=14, window=19, rot_dims=6), 56),
              (bo.diff_mixer(heads=3, kv_heads=3, dim=8, vdim=6, window=33, rot_dims=8, softcap=None, diff=0.4), None),
              (par(left=dict(heads=2, kv_heads=1, dim=16, vdim=20, window=9, keep_first=0, rot_dims=4, scaling=None),
                   right=dict(heads=2, vdim=12, state=4, groups=1, conv=2, norm_groups=4)), 24)]
    cfg = bo.make_config(width=48, vocab=61, layers=layers)
    w = bo.make_weights(cfg, seed=1, sharp=3.0)
    return cfg, w, bo.write_model(tmp_path_factory.mktemp("buku_base"), cfg, w)


# ---- every mechanism on its own -------------------------------------------------------------------------------------
CASES = {
    "diff": [(bo.diff_mixer(), None)],
    "diff_every_head_its_keys": [(bo.diff_mixer(heads=3, kv_heads=3), None)],
    "diff_one_key_head": [(bo.diff_mixer(heads=4, kv_heads=1, dim=16, vdim=6), None)],
    "diff_unrotated": [(bo.diff_mixer(rot_dims=0), None)],
    "diff_all_rotated": [(bo.diff_mixer(dim=8, rot_dims=8, base=50.0), None)],
    "diff_window_one": [(bo.diff_mixer(window=1), None)],                 # every map sees its own token only
    "diff_window_past_the_prompt": [(bo.diff_mixer(window=500), None)],
    "diff_tight_cap": [(bo.diff_mixer(softcap=0.7, scale=1.0), None)],
    "diff_no_cap": [(bo.diff_mixer(softcap=None), None)],
    "diff_plain_difference": [(bo.diff_mixer(diff=0.0), None)],           # lambda from the vectors alone, output scale 1
    "diff_wide": [(bo.diff_mixer(heads=2, kv_heads=1, dim=72, vdim=40, rot_dims=20, window=40), None)],
    "diff_widest": [(bo.diff_mixer(heads=2, kv_heads=2, dim=136, vdim=24, rot_dims=136, window=33), None)],
    "diff_long_values": [(bo.diff_mixer(heads=2, kv_heads=1, dim=8, vdim=200, window=12), None)],
    "pair": [(par(), None)],
    "left_alone": [(par(), None)],
    "left_every_head_its_keys": [(par(left=dict(heads=3, kv_heads=3)), None)],
    "left_one_key_head": [(par(left=dict(heads=4, kv_heads=1, dim=16, vdim=4)), None)],
    "left_unrotated": [(par(left=dict(rot_dims=0, scaling=None)), None)],
    "left_unscaled_rotation": [(par(left=dict(scaling=None)), None)],
    "left_all_rotated_all_slowed": [(par(left=dict(dim=8, rot_dims=8, base=50.0, scaling=(16.0, 4096, 1e9, 1e8))), None)],
    "left_all_rotated_none_slowed": [(par(left=dict(dim=8, rot_dims=8, base=50.0, scaling=(16.0, 8, 1e-3, 1e-4))), None)],
    "left_window_one": [(par(left=dict(window=1, keep_first=0)), None)],
    "left_nothing_kept": [(par(left=dict(window=9, keep_first=0)), None)],
    "left_many_kept": [(par(left=dict(window=5, keep_first=70)), None)],      # kept tokens past a key tile
    "left_wide": [(par(left=dict(heads=2, kv_heads=1, dim=72, vdim=136, rot_dims=20, window=40)), None)],
    "right_alone": [(par(), None)],
    "right_one_group": [(par(right=dict(heads=3, groups=1)), None)],
    "right_every_head_its_group": [(par(right=dict(heads=3, groups=3, norm_groups=1)), None)],
    "right_one_state": [(par(right=dict(heads=2, vdim=7, state=1, groups=1, norm_groups=7)), None)],
    "right_many_states": [(par(right=dict(heads=2, vdim=3, state=100, groups=2, conv=4, norm_groups=3)), None)],
    "right_states_over_lanes": [(par(right=dict(heads=2, vdim=40, state=40, groups=1, conv=4, norm_groups=5)), None)],
    "right_states_beyond_256": [(par(right=dict(heads=2, vdim=6, state=300, groups=1, conv=2, norm_groups=2)), None)],
    "right_no_filter": [(par(right=dict(conv=1)), None)],
    "right_long_filter": [(par(right=dict(conv=7)), None)],
    "right_one_norm_part": [(par(right=dict(norm_groups=1)), None)],
    "right_a_norm_part_per_value": [(par(right=dict(heads=2, vdim=3, norm_groups=6)), None)],
    "ff_beside_attention": [(bo.diff_mixer(), 56)],
    "ff_only": [(bo.diff_mixer(), 30)],
    "ff_beside_the_pair": [(par(), 17)],
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_mechanism_alone(tmp_path, case):
    # a large eps in some cases: it must reach every norm (the layers', the heads', the maps', the parts')
    big_eps = case in ("diff", "pair", "right_one_norm_part", "ff_only", "left_unrotated")
    cfg = bo.make_config(width=40, vocab=50, layers=CASES[case], eps=0.05 if big_eps else 3e-6,
                         embed_scale=1.0 if case == "diff_no_cap" else 2.5,
                         residual_mult=1.0 if case in ("pair", "diff_unrotated") else 0.6)
    w = bo.make_weights(cfg, seed=3, sharp=3.0)
    if case.startswith("left_"):
        mute(w, 0, "right")
    if case.startswith("right_"):
        mute(w, 0, "left")
    if case == "ff_only":  # the mixer's output projection is zero: what is left of the layer is the feed-forward
        w["l0.mix.o"] = np.zeros_like(w["l0.mix.o"])
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(75, cfg["vocab"], 5)
    ref, trace = bo.forward(cfg, w, t)
    logits, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    assert np.abs(got - trace).max() < 1e-4 * max(1.0, np.abs(trace).max())
    assert_rows(logits[0], ref)


def test_residual_after_every_layer(base):
    cfg, w, d = base
    t = toks(33, cfg["vocab"], 7)
    _, trace = bo.forward(cfg, w, t)
    assert trace.shape[0] == 4
    _, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    for r in range(trace.shape[0]):
        assert np.abs(got[r] - trace[r]).max() < 1e-4 * max(1.0, np.abs(trace[r]).max()), f"layer {r}"


@pytest.mark.parametrize("order", ["AP", "PPA", "APAAP"])
def test_layer_orders(tmp_path, order):
    """Any order of the two kinds of layer; every layer has a cache and a state of its own."""
    layers = [((bo.diff_mixer(window=9) if c == "A" else par(left=dict(window=7))), 24 if i % 2 else None)
              for i, c in enumerate(order)]
    cfg = bo.make_config(width=40, vocab=60, layers=layers)
    w = bo.make_weights(cfg, seed=101, sharp=2.0)
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(45, cfg["vocab"], 102)
    logits, _ = run_trace(d, [whole("a", t[:30], end=False)] + single("a", t[30:]))
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


@pytest.mark.parametrize("page", [4, 16, 64])
def test_long_prompt_every_position(base, page):
    cfg, w, d = base
    t = toks(203, cfg["vocab"], 11)  # past three key tiles of 64 and several chunks of the recurrence, no multiple of a page
    logits, _ = run_trace(d, [whole("a", t)], page=page)
    assert_rows(logits[0], ref_logits(cfg, w, t))


# ---- keys at the edges of the window and of the kept first tokens ---------------------------------------------------
def edge_model(kind, window, keep_first, special, vocab=30, width=24, seed=9):
    """One attention layer, made so that ONE token's key wins every softmax it takes part in.  The sublayers read the
    embeddings as they are.  Input coordinate 1 is the same for every token and feeds the last (unrotated) coordinate
    of every query head (of map 1, when there are two), so every query points along it after its norm; input
    coordinate 0 is zero except for the special token and feeds the same coordinate of the keys, and nothing else
    does.  While the special key is seen, a head's output is (almost) that token's value."""
    if kind == "diff":
        m = bo.diff_mixer(heads=2, kv_heads=1, dim=8, vdim=6, window=window, rot_dims=4, scale=3.0, softcap=40.0)
        layers, p, maps = [(m, None)], "l0.mix.", 2
    else:
        m = par(left=dict(heads=2, kv_heads=1, dim=8, vdim=6, window=window, keep_first=keep_first, rot_dims=4, scale=3.0))
        layers, p, maps = [(m, None)], "l0.mix.left.", 1
    cfg = bo.make_config(width=width, vocab=vocab, layers=layers, embed_scale=1.0)
    w = bo.make_weights(cfg, seed=seed)
    if kind != "diff":
        mute(w, 0, "right")
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 8.0
    w["embed"][:, 1] = 2.0
    last = 7  # of dim = 8
    w[p + "q"] = bo.bf16_round(w[p + "q"] * 0.05)
    w[p + "k"][:, :2] = 0.0
    for head in range(2):
        w[p + "q"][head * maps * 8 + last] = 0.0
        w[p + "q"][head * maps * 8 + last, 1] = 4.0
    w[p + "k"][last] = 0.0
    w[p + "k"][last, 0] = 2.0
    return cfg, w


@pytest.mark.parametrize("kind", ["diff", "left"])
@pytest.mark.parametrize("window", [2, 17, 64, 65, 100])
def test_the_key_at_the_window_edge_carries_the_output(tmp_path, kind, window):
    """The special key is placed so that it leaves the window inside the prompt, and a second one so that it leaves
    while tokens are decoded one by one (across key tiles and pages).  The last position that still sees it depends on
    it heavily; the next one does not depend on it at all."""
    special = 7
    cfg, w = edge_model(kind, window, 0, special)
    n_prompt, n_all = 150, 150 + window + 20
    t = [x if x != special else special + 1 for x in toks(n_all, cfg["vocab"], 13)]
    places = (20, n_prompt - 5)  # leaves the window inside the prompt / during decoding
    for p in places:
        t[p] = special
    ref = ref_logits(cfg, w, t)
    for p in places:  # the construction works
        t2 = list(t)
        t2[p] = special + 1
        other = ref_logits(cfg, w, t2)
        if window > 1:
            assert rel_err(other[p + window - 1:p + window], ref[p + window - 1:p + window]) > 0.1
        assert rel_err(other[p + window:p + window + 1], ref[p + window:p + window + 1]) < 1e-9
    d = bo.write_model(tmp_path, cfg, w)
    logits, _ = run_trace(d, [whole("a", t[:n_prompt], end=False)] + single("a", t[n_prompt:]), page=16)
    assert_rows(np.concatenate(logits), ref)


@pytest.mark.parametrize("keep,window", [(1, 3), (6, 10), (64, 5), (70, 33)])
def test_the_first_tokens_stay_and_the_next_one_leaves(tmp_path, keep, window):
    """The special token at the last kept position is seen for ever (far outside the window, in prompts and in decoding);
    at the first position that is not kept it leaves with the window."""
    special = 7
    for place, stays in ((keep - 1, True), (keep, False)):
        cfg, w = edge_model("left", window, keep, special)
        n_prompt, n_all = keep + window + 40, keep + window + 70
        t = [x if x != special else special + 1 for x in toks(n_all, cfg["vocab"], 14)]
        t[place] = special
        ref = ref_logits(cfg, w, t)
        t2 = list(t)
        t2[place] = special + 1
        far = rel_err(ref_logits(cfg, w, t2)[-1:], ref[-1:])
        assert (far > 0.1) == stays  # the construction works: the last logits depend on that token only while it is kept
        d = bo.write_model(tmp_path / f"{place}", cfg, w)
        logits, _ = run_trace(d, [whole("a", t[:n_prompt], end=False)] + single("a", t[n_prompt:]), page=8)
        assert_rows(np.concatenate(logits), ref)


def test_the_second_map_is_subtracted(tmp_path):
    """The special key wins map 2 instead of map 1 and lambda is large: dropping the map, its lambda or the norm after
    the difference changes the output completely."""
    special = 7
    cfg, w = edge_model("diff", 12, 0, special)
    p = "l0.mix."
    for head in range(2):  # the queries of map 2 point along the special coordinate, those of map 1 anywhere
        w[p + "q"][head * 16 + 15] = w[p + "q"][head * 16 + 7]
        w[p + "q"][head * 16 + 7] = bo.bf16_round(0.05 * np.random.default_rng(head).standard_normal(24))
    w[p + "k"][15] = w[p + "k"][7]
    w[p + "k"][7] = 0.0
    w[p + "lq1"] = bo.bf16_round(np.full(8, 0.5))
    w[p + "lk1"] = bo.bf16_round(np.full(8, 0.25))   # exp(1) - exp(small) + diff
    assert bo.differential_lambda(w, p, cfg["layers"][0]["mixer"]["diff"]) > 1.5
    t = [x if x != special else special + 1 for x in toks(60, cfg["vocab"], 15)]
    t[30] = special
    ref = ref_logits(cfg, w, t)
    t2 = list(t)
    t2[30] = special + 1
    assert rel_err(ref_logits(cfg, w, t2)[35:36], ref[35:36]) > 0.1
    d = bo.write_model(tmp_path, cfg, w)
    logits, _ = run_trace(d, [whole("a", t[:33], end=False)] + single("a", t[33:]))
    assert_rows(np.concatenate(logits), ref)


# ---- the recurrent state ----------------------------------------------------------------------------------------------
def test_far_tokens_stay_in_the_recurrent_state(tmp_path):
    """Decays next to 1: what the first token wrote is still in the state hundreds of tokens, several chunks, two
    portions and many single steps later, and the last logits depend on it."""
    cfg = bo.make_config(width=32, vocab=40, layers=[(par(right=dict(heads=2, vdim=8, state=6, groups=1, conv=3)), None)],
                         embed_scale=1.0)
    w = bo.make_weights(cfg, seed=31)
    mute(w, 0, "left")
    special, r = 5, "l0.mix.right."
    t = [x if x != special else special + 1 for x in toks(330, cfg["vocab"], 32)]
    t[0] = special
    # only the special token's embedding has coordinate 0; every value channel and every step size reads it
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 6.0
    w[r + "in"][:, 0] = 0.0
    w[r + "in"][16:32, 0] = 3.0      # x rows
    w[r + "in"][-2:, 0] = 1.0        # dt rows: a large step for the special token ...
    w[r + "dt_bias"] = np.full_like(w[r + "dt_bias"], -3.0)   # ... and small ones for every other
    w[r + "A_log"] = np.full_like(w[r + "A_log"], bo.bf16_round(np.log(2e-3)))
    ref = ref_logits(cfg, w, t)
    t2 = list(t)
    t2[0] = special + 1
    assert rel_err(ref_logits(cfg, w, t2)[-1:], ref[-1:]) > 1e-2  # the construction works
    d = bo.write_model(tmp_path, cfg, w)
    # the second portion is long enough to be cut into segments that are scanned side by side, from a state that is not empty
    steps = [whole("a", t[:10], end=False), whole("a", t[10:300], end=False)] + single("a", t[300:])
    logits, _ = run_trace(d, steps)
    assert_rows(np.concatenate(logits), ref)


def test_long_entries_are_walked_in_segments(tmp_path):
    """Entries of several hundred rows: the recurrence cuts them into segments that run side by side and are joined by a
    carry -- from an empty state, from a state that earlier rows left, beside a short entry, and with decoding afterwards."""
    layers = [(par(left=dict(window=30), right=dict(heads=4, vdim=10, state=24, groups=2, conv=4)), 24),
              (bo.diff_mixer(window=40), None),
              (par(left=dict(window=11, keep_first=0), right=dict(heads=3, vdim=5, state=3, groups=3, conv=2, norm_groups=1)), None)]
    cfg = bo.make_config(width=32, vocab=40, layers=layers)
    w = bo.make_weights(cfg, seed=91)
    d = bo.write_model(tmp_path, cfg, w)
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
    """A prompt fed in several steps: every portion starts from the cache, the filter's history and the recurrent
    state the portions before it left -- portions shorter than the filter's history too.  A second request of another
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
    """bf16 products against float64, on a model whose softmaxes are not sharpened (a peaky map amplifies the rounding of
    its scores)."""
    layers = [(par(left=dict(window=21), right=dict(heads=4, vdim=12, state=8, groups=2, conv=4)), 40),
              (bo.diff_mixer(heads=4, kv_heads=2, dim=20, vdim=36, window=19, rot_dims=6), 56),
              (par(left=dict(heads=2, kv_heads=1, dim=16, vdim=20, window=9, keep_first=0, rot_dims=4, scaling=None)), None)]
    cfg = bo.make_config(width=72, vocab=101, layers=layers)
    w = bo.make_weights(cfg, seed=5)
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(140, cfg["vocab"], 61)
    logits, _ = run_trace(d, [whole("a", t[:120], end=False)] + single("a", t[120:]), dtype="bfloat16")
    assert rel_err(np.concatenate(logits), ref_logits(cfg, w, t)) < TOL16


@pytest.mark.parametrize("kind,dim,vdim,window,keep", [("diff", 24, 40, 17, 0), ("diff", 64, 128, 64, 0), ("diff", 128, 64, 150, 0),
                                                       ("left", 24, 24, 17, 0), ("left", 64, 128, 64, 3), ("left", 128, 64, 150, 70),
                                                       ("left", 256, 128, 100, 5), ("diff", 64, 200, 40, 0)])
def test_bfloat16_prompts_on_the_tensor_cores(tmp_path, kind, dim, vdim, window, keep):
    """bf16 prompt steps with head sizes that are multiples of 8 take the tensor-core attention (both maps of a
    differential head, the window, the kept first tokens, the cap): against the float64 restatement, and against
    single-token steps of the same run.  Values of 200 are past the tensor-core kernel: they take the split-key kernel."""
    if kind == "diff":
        layers = [(bo.diff_mixer(heads=4, kv_heads=2, dim=dim, vdim=vdim, rot_dims=16, window=window, softcap=8.0), None)]
    else:
        layers = [(par(left=dict(heads=4, kv_heads=2, dim=dim, vdim=vdim, rot_dims=16, window=window, keep_first=keep)), None)]
    cfg = bo.make_config(width=64, vocab=80, layers=layers)
    w = bo.make_weights(cfg, seed=41, sharp=2.0)
    if kind == "left":
        mute(w, 0, "right")
    d = bo.write_model(tmp_path, cfg, w)
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
    layers = [(par(left=dict(heads=3, kv_heads=1, dim=6, vdim=5, rot_dims=2, window=7, keep_first=1),
                   right=dict(heads=3, vdim=7, state=5, groups=3, conv=3, norm_groups=3)), 11),
              (bo.diff_mixer(heads=3, kv_heads=3, dim=5, vdim=7, rot_dims=2, window=13), 9),
              (par(left=dict(heads=1, kv_heads=1, dim=10, vdim=3, rot_dims=6, window=3, keep_first=2),
                   right=dict(heads=1, vdim=13, state=3, groups=1, conv=5, norm_groups=13)), None)]
    cfg = bo.make_config(width=22, vocab=23, layers=layers)
    w = bo.make_weights(cfg, seed=51)
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(77, cfg["vocab"], 52)
    logits, _ = run_trace(d, [whole("a", t[:70], end=False)] + single("a", t[70:]), dtype=dtype)
    err = row_errors(np.concatenate(logits), ref_logits(cfg, w, t))
    if dtype == "float32":
        assert err.max() < tol
    else:  # a sublayer whose output is nearly zero is normed up together with its rounding: that costs single rows
        assert np.median(err) < tol / 2 and (err > tol).mean() <= 0.05, np.sort(err)[-5:]


def test_larger_shapes_take_the_block_paths(tmp_path):
    """Width and inner sizes past one tile, heads of tensor-core sizes, a state of 128 over 8 lanes, enough tokens for
    the token-block products and the segmented recurrence."""
    layers = [(par(left=dict(heads=4, kv_heads=2, dim=32, vdim=64, rot_dims=16, window=100, keep_first=4),
                   right=dict(heads=4, vdim=32, state=128, groups=2, conv=4, norm_groups=2)), 192),
              (bo.diff_mixer(heads=4, kv_heads=2, dim=32, vdim=64, rot_dims=16, window=80), 160)]
    cfg = bo.make_config(width=128, vocab=200, layers=layers)
    w = bo.make_weights(cfg, seed=61)
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(300, cfg["vocab"], 62)
    ref = ref_logits(cfg, w, t)
    logits, _ = run_trace(d, [whole("a", t[:290], end=False)] + single("a", t[290:]))
    assert_rows(np.concatenate(logits), ref)
    lb, _ = run_trace(d, [whole("a", t[:290], end=False)] + single("a", t[290:]), dtype="bfloat16")
    assert rel_err(np.concatenate(lb), ref) < TOL16


def random_design(seed):
    rng = np.random.default_rng(seed)

    def pick(*xs):
        return xs[int(rng.integers(len(xs)))]

    def mixer():
        g = pick(1, 2, 3)
        if pick("diff", "pair") == "diff":
            dim = pick(4, 8, 12)
            return bo.diff_mixer(heads=g * pick(1, 2), kv_heads=g, dim=dim, vdim=pick(3, 8, 16), window=pick(1, 5, 30, 66),
                                 rot_dims=pick(0, 2, dim), base=pick(100.0, 10000.0), softcap=pick(None, 3.0, 30.0),
                                 diff=pick(0.0, 0.2, 0.5))
        dim = pick(4, 8, 12)
        left = dict(heads=g * pick(1, 2), kv_heads=g, dim=dim, vdim=pick(3, 8, 16), window=pick(1, 5, 30, 66),
                    keep_first=pick(0, 1, 7), rot_dims=pick(0, 2, dim), base=pick(100.0, 10000.0),
                    scaling=pick(None, (4.0, 64, 16.0, 1.0), (2.0, 32, 4.0, 2.0)))
        sg = pick(1, 2)
        heads, vdim = sg * pick(1, 3), pick(2, 4, 8)
        right = dict(heads=heads, vdim=vdim, state=pick(1, 3, 8, 20), groups=sg, conv=pick(1, 2, 4),
                     norm_groups=pick(1, heads, vdim))
        return par(left=left, right=right)

    layers = [(mixer(), pick(None, 8, 30)) for _ in range(int(rng.integers(1, 5)))]
    return bo.make_config(width=pick(16, 24, 40), vocab=pick(17, 50), layers=layers, eps=pick(1e-6, 1e-3),
                          embed_scale=pick(1.0, 0.5, 4.0), residual_mult=pick(1.0, 0.5, 0.8))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_designs(tmp_path, seed):
    """Layer order, sizes and constants drawn at random; a ragged batch that is prefilled together and decoded together,
    in float32 (tight) and bfloat16 (loose)."""
    cfg = random_design(seed)
    w = bo.make_weights(cfg, seed=100 + seed, sharp=2.0)
    d = bo.write_model(tmp_path, cfg, w)
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
            assert np.median(err) < TOL16 / 2 and (err > 2 * TOL16).mean() <= 0.02, np.sort(err)[-5:]


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
        assert g == bo.greedy(cfg, w, p, 12)


def test_a_tensor_of_the_wrong_shape_is_reported(base, tmp_path):
    from kuiperllama_b200 import build
    cfg, w, _ = base
    w2 = dict(w)
    w2["l1.mix.q"] = w["l1.mix.q"][:-1]  # one query row short of heads * 2 * dim
    d = bo.write_model(tmp_path / "m", cfg, w2)
    r = subprocess.run([str(build.build_seq_tools() / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype",
                        "float32"], capture_output=True, text=True)
    assert r.returncode == 2 and "l1.mix." in r.stderr


def test_many_heads_in_single_token_steps(tmp_path):
    """More query and key maps than a CTA has warps for: the preparation of single-token steps walks them in turns."""
    layers = [(bo.diff_mixer(heads=20, kv_heads=5, dim=8, vdim=6, window=12, rot_dims=4), None),
              (par(left=dict(heads=36, kv_heads=4, dim=4, vdim=4, window=9, rot_dims=2)), None)]
    cfg = bo.make_config(width=32, vocab=40, layers=layers)
    w = bo.make_weights(cfg, seed=77, sharp=2.0)
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(30, cfg["vocab"], 78)
    logits, _ = run_trace(d, [whole("a", t[:10], end=False)] + single("a", t[10:]))
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


@pytest.mark.parametrize("kind,heads,kv_heads", [("diff", 6, 2), ("diff", 5, 5), ("diff", 8, 1), ("left", 6, 2), ("left", 5, 1)])
def test_bfloat16_prompts_with_other_head_counts(tmp_path, kind, heads, kv_heads):
    """Three, one and eight query heads per key head on the tensor-core prompt path (a row tile then mixes the rows of
    several heads), beside a second request and followed by single-token steps."""
    if kind == "diff":
        layers = [(bo.diff_mixer(heads=heads, kv_heads=kv_heads, dim=40, vdim=72, rot_dims=24, window=50), 48)]
    else:
        layers = [(par(left=dict(heads=heads, kv_heads=kv_heads, dim=40, vdim=24, rot_dims=24, window=50, keep_first=9)), 48)]
    cfg = bo.make_config(width=64, vocab=80, layers=layers)
    w = bo.make_weights(cfg, seed=43, sharp=2.0)
    d = bo.write_model(tmp_path, cfg, w)
    a, b = toks(150, cfg["vocab"], 44), toks(37, cfg["vocab"], 45)
    steps = [{"entries": [{"id": "a", "tokens": a[:140], "want": list(range(140))},
                          {"id": "b", "tokens": b[:27], "want": list(range(27))}]}]
    for j in range(10):
        steps.append({"entries": [{"id": "a", "tokens": [a[140 + j]], "want": [0]}, {"id": "b", "tokens": [b[27 + j]], "want": [0]}]})
    for dtype, tol in (("float32", TOL32), ("bfloat16", TOL16)):
        logits, _ = run_trace(d, steps, dtype=dtype)
        got_a = np.concatenate([logits[0][:140]] + [lg[0:1] for lg in logits[1:]])
        got_b = np.concatenate([logits[0][140:]] + [lg[1:2] for lg in logits[1:]])
        assert rel_err(got_a, ref_logits(cfg, w, a)) < tol
        assert rel_err(got_b, ref_logits(cfg, w, b)) < tol


def test_wide_states_in_segments(tmp_path):
    """More than 256 state coordinates (16 per lane, two columns a thread) in an entry long enough to be cut into segments,
    then single-token steps."""
    cfg = bo.make_config(width=32, vocab=40, layers=[(par(right=dict(heads=2, vdim=5, state=270, groups=2, conv=3, norm_groups=1)), None)])
    w = bo.make_weights(cfg, seed=95)
    mute(w, 0, "left")
    d = bo.write_model(tmp_path, cfg, w)
    t = toks(3 + 290 + 4, cfg["vocab"], 96)
    steps = [whole("a", t[:3], end=False), whole("a", t[3:293], end=False)] + single("a", t[293:])
    logits, _ = run_trace(d, steps, max_tokens=512)
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


def test_a_mid_sized_model(tmp_path):
    """Five layers at sizes between the toy models above and a real one: every product past one tile, heads on the
    tensor-core sizes, a prompt long enough for segments, a ragged batch decoded together -- float32 tight, bfloat16 loose."""
    layers = [(bo.diff_mixer(heads=6, kv_heads=3, dim=32, vdim=64, rot_dims=16, window=100, softcap=30.0), 768),
              (par(left=dict(heads=6, kv_heads=2, dim=48, vdim=32, rot_dims=16, window=64, keep_first=5, scaling=(6.0, 256, 16.0, 2.0)),
                   right=dict(heads=8, vdim=32, state=64, groups=4, conv=4, norm_groups=4)), 512),
              (bo.diff_mixer(heads=4, kv_heads=4, dim=64, vdim=64, rot_dims=64, window=300, softcap=None, diff=0.1), None),
              (par(left=dict(heads=4, kv_heads=1, dim=64, vdim=96, rot_dims=32, window=200, keep_first=0, scaling=None),
                   right=dict(heads=12, vdim=16, state=32, groups=1, conv=3, norm_groups=1)), 768)]
    layers.append(layers[1])
    cfg = bo.make_config(width=384, vocab=500, layers=layers, eps=2e-5, embed_scale=12.0, residual_mult=0.6)
    w = bo.make_weights(cfg, seed=123)
    d = bo.write_model(tmp_path, cfg, w)
    reqs = {"a": toks(330, cfg["vocab"], 124), "b": toks(70, cfg["vocab"], 125), "c": toks(9, cfg["vocab"], 126)}
    n_dec = 6
    steps = [{"entries": [{"id": k, "tokens": r[:-n_dec], "want": list(range(len(r) - n_dec))} for k, r in reqs.items()]}]
    for j in range(n_dec):
        steps.append({"entries": [{"id": k, "tokens": [r[len(r) - n_dec + j]], "want": [0]} for k, r in reqs.items()]})
    refs = {k: ref_logits(cfg, w, r) for k, r in reqs.items()}
    for dtype, tol in (("float32", TOL32), ("bfloat16", TOL16)):
        logits, _ = run_trace(d, steps, dtype=dtype, max_tokens=1024)
        at = 0
        for i, (k, r) in enumerate(reqs.items()):
            n = len(r) - n_dec
            got = np.concatenate([logits[0][at:at + n]] + [logits[1 + j][i:i + 1] for j in range(n_dec)])
            at += n
            err = row_errors(got, refs[k])
            if dtype == "float32":
                assert err.max() < tol, (k, int(err.argmax()), err.max())
            else:
                assert np.median(err) < tol / 2 and (err > tol).mean() <= 0.05, (k, np.sort(err)[-5:])
