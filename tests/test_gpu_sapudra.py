"""Sapudra (layer-list family) on the GPU against the float64 oracle of tests/ref_sapudra.py: every mechanism alone, prompts against
token-by-token decoding, prompt portions, ragged batches, slot reuse, a far key, keys just inside and just outside the window (in
prompts and decoded, also across the ring cache's wrap), the edges of the kernels' tiles, the first tokens, long decoding, odd sizes,
greedy generation through the scheduler, the directory loader and the command-line replay.  Small configurations made here; weights
are random but exactly representable in bf16, so the float32 engine and the oracle see the same numbers and the comparison is sharp."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import ref_sapudra as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4     # relative rms error of a logits row, float32 engine vs float64 oracle
BF16_TOL = 6e-2


def dense_ff(ff=88):
    return {"kind": "dense", "ff": ff}


def moe_ff(experts=8, top=3, ff=40, count=4, keep=3, scale=1.75, shared=56):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def att_layer(heads=4, kv_heads=2, dim=24, vdim=40, window=29, scale=0.3, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}, "mlp": mlp}


def config(layers, width=72, vocab=149, max_positions=512, mult=0.6, cap=9.0, eps=1e-5):
    c = {"architecture": "Sapudra", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps}, "residual_mult": mult,
         "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


def mixed_config():
    return config([att_layer(mlp=dense_ff()), att_layer(heads=6, kv_heads=1, dim=16, vdim=16, window=11, mlp=moe_ff()),
                   att_layer(heads=3, kv_heads=3, dim=20, vdim=12, window=64, mlp=None),
                   att_layer(heads=2, kv_heads=1, dim=32, vdim=24, window=37, mlp=moe_ff(experts=5, top=2, ff=32, count=1, keep=1, shared=None))])


def load(pkg, cfg, bits, dtype="float32", n_ctx=512, n_seq=8):
    m = pkg.Model.from_config(cfg, dtype=dtype, n_ctx=n_ctx, n_seq=n_seq)
    for name, b in bits.items():
        m.set_tensor(name, pkg.TYPES["bf16"], b)
    m.finalize()
    return m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run_whole(m, toks, want=None):
    s = m.seq_alloc()
    lg, _ = m.batch_step([(s, toks, list(range(len(toks))) if want is None else want)])
    m.seq_free(s)
    return lg


def run_decoded(m, toks, first):
    """The first `first` tokens as a prompt, the rest one by one; logits of every position."""
    s = m.seq_alloc()
    rows = [m.batch_step([(s, toks[:first], list(range(first)))])[0]]
    for t in toks[first:]:
        rows.append(m.batch_step([(s, [t], [0])])[0])
    m.seq_free(s)
    return np.concatenate(rows)


def check(got, want, tol, sure=None):
    """sure: rows to compare (True) and rows left out (False)."""
    e = R.rel_err(np.asarray(got, dtype=np.float64), want)
    if sure is not None:
        assert sure.mean() > 0.5
        e = np.where(sure, e, 0.0)
    assert e.max() < tol, f"worst row {int(e.argmax())}: {e.max():.3e} (tolerance {tol})"


def oracle(cfg, W, toks, dtype="float32"):
    """The oracle's logits, and for bfloat16 runs the rows whose tokens are routed without a close call: a choice score that wins by less
    than bf16 rounding moves it may send the token to another expert, which is no fault of the engine.  float32 runs compare every row."""
    margins = []
    want, taps = R.forward(cfg, W, toks, margins)
    sure = None
    if dtype == "bfloat16" and margins:
        sure = np.min(np.stack(margins), axis=0) > 0.02
    return want, taps, sure


def negative_choice_case():
    # every choice score below zero: an expert outside the kept groups would win if "not eligible" were written as 0
    cfg = config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff(experts=9, top=2, ff=24, count=3, keep=1))])
    return cfg, {"l0.mlp.correction": lambda a: a - 4.0}


MECHANISMS = {
    "attention_grouped_heads": lambda: (config([att_layer()]), {}),
    "attention_one_key_head": lambda: (config([att_layer(heads=5, kv_heads=1, dim=12, vdim=12, window=500)]), {}),
    "attention_every_head_its_own": lambda: (config([att_layer(heads=3, kv_heads=3, dim=16, vdim=8, window=7)]), {}),
    "dense_ff": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=dense_ff(136))]), {}),
    "moe_groups": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff())]), {}),
    "moe_groups_of_one": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff(experts=6, top=2, count=6, keep=3))]), {}),
    "moe_negative_choice_scores": negative_choice_case,
    "moe_no_shared_expert": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff(shared=None))]), {}),
    "strong_soft_cap": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8)], cap=1.5), {"head": lambda a: 4.0 * a}),
    "no_soft_cap_multiplier_one": lambda: (config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=dense_ff(24))], cap=None, mult=1.0), {}),
    "four_layers": lambda: (mixed_config(), {}),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(MECHANISMS))
def test_each_mechanism_alone(pkg, cuda, which, dtype, tol):
    cfg, edits = MECHANISMS[which]()
    bits, W = R.random_weights(cfg, seed=3)
    for name, f in edits.items():
        R.set_weight(bits, W, name, f(W[name]))
    toks = tokens_for(cfg, 41, 1)
    want, taps, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    m.tap_layers(True)
    got = run_whole(m, toks)
    got_taps = m.debug_read("layers", taps.size).reshape(taps.shape)
    m.close()
    check(got, want, tol, sure)
    scale = np.abs(taps).max()
    rows = slice(None) if sure is None else sure
    assert np.abs(got_taps - taps)[:, rows].max() < (1e-4 if dtype == "float32" else 8e-2) * scale


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_and_decoding_agree_with_the_oracle(pkg, cuda, dtype, tol):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=5)
    toks = tokens_for(cfg, 90, 2)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_whole(m, toks), want, tol, sure)
    check(run_decoded(m, toks, 1), want, tol, sure)    # everything after the first token through the decode path
    check(run_decoded(m, toks, 41), want, tol, sure)
    m.close()


def test_prompt_portions_of_several_sizes(pkg, cuda):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=6)
    toks = tokens_for(cfg, 61, 3)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    for cuts in ([2, 2, 2, 55], [17, 16, 1, 27], [33, 2, 26], [60, 1]):
        s = m.seq_alloc()
        rows, at = [], 0
        for n in cuts:
            rows.append(m.batch_step([(s, toks[at:at + n], list(range(n)))])[0])
            at += n
        m.seq_free(s)
        check(np.concatenate(rows), want, F32_TOL)
    m.close()


def test_ragged_batch_equals_each_request_alone(pkg, cuda):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=7)
    m = load(pkg, cfg, bits, n_seq=6)
    lens = [1, 70, 9, 33, 18]
    reqs = [tokens_for(cfg, n + 6, 10 + i) for i, n in enumerate(lens)]
    alone = [run_decoded(m, r, n) for r, n in zip(reqs, lens)]
    slots = [m.seq_alloc() for _ in reqs]
    lg, _ = m.batch_step([(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, lens)])
    got = [[] for _ in reqs]
    at = 0
    for i, n in enumerate(lens):
        got[i].append(lg[at:at + n])
        at += n
    live = list(range(len(reqs)))
    for k in range(6):
        if k == 3:
            live = live[:3]                                    # two requests end earlier
        lg, _ = m.batch_step([(slots[i], [reqs[i][lens[i] + k]], [0]) for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
    for i, r in enumerate(reqs):
        g = np.concatenate(got[i])
        assert np.abs(g - alone[i][:len(g)]).max() < 5e-5 * np.abs(alone[i]).max()
        want, _ = R.forward(cfg, W, r[:len(g)])
        check(g, want, F32_TOL)
    m.close()


def test_slots_are_clean_when_handed_out_again(pkg, cuda):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=8)
    m = load(pkg, cfg, bits, n_seq=2)
    a, b = tokens_for(cfg, 80, 20), tokens_for(cfg, 23, 21)     # the longer one wraps the ring of every window; the shorter must not see its rows
    wa, _ = R.forward(cfg, W, a)
    wb, _ = R.forward(cfg, W, b)
    for _ in range(3):                                          # the same two slots over and over, in changing roles
        s0, s1 = m.seq_alloc(), m.seq_alloc()
        lg, _ = m.batch_step([(s0, a, list(range(len(a)))), (s1, b, list(range(len(b))))])
        check(lg[:len(a)], wa, F32_TOL)
        check(lg[len(a):], wb, F32_TOL)
        m.seq_free(s0)
        s2 = m.seq_alloc()
        assert s2 == s0
        check(run_rest(m, s2, b, 5), wb, F32_TOL)
        m.seq_free(s1)
        m.seq_free(s2)
        a, b, wa, wb = b, a, wb, wa
    m.close()


def run_rest(m, s, toks, first):
    rows = [m.batch_step([(s, toks[:first], list(range(first)))])[0]]
    for t in toks[first:]:
        rows.append(m.batch_step([(s, [t], [0])])[0])
    return np.concatenate(rows)


def one_key_case(window, heads=2, T=300, where=5):
    """One attention layer whose last query puts nearly all its weight on position `where`: the position table is zero and every query
    head is the negated key of its own token (so a token never looks at itself or its like); the last token A and the token B at
    `where` are the pair of the vocabulary with the largest score; the other positions hold tokens that score far below it against A."""
    cfg = config([att_layer(heads=heads, kv_heads=1, dim=24, vdim=16, window=window, scale=2.0)], width=48, vocab=97, max_positions=T + 8)
    bits, W = R.random_weights(cfg, seed=11)
    R.set_weight(bits, W, "pos", np.zeros_like(W["pos"]))
    R.set_weight(bits, W, "l0.mix.q", -np.tile(W["l0.mix.k"], (heads, 1)))
    R.set_weight(bits, W, "l0.mix.q.norm", W["l0.mix.k.norm"])
    k = R.head_norm((W["embed"] @ W["l0.mix.k"].T).reshape(97, 1, 24), W["l0.mix.k.norm"], cfg["norm"]["eps"])[:, 0]   # every token of the vocabulary
    score = -(k @ k.T) * 2.0
    np.fill_diagonal(score, -np.inf)
    A, B = np.unravel_index(np.argmax(score), score.shape)
    quiet = [t for t in range(97) if t not in (A, B) and score[A, t] < score[A, B] - 14.0]
    assert len(quiet) >= 20
    rng = np.random.default_rng(4)
    toks = [quiet[i] for i in rng.integers(0, len(quiet), T)]
    toks[where], toks[-1] = int(B), int(A)
    return cfg, bits, W, toks


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window", [1000, 295, 294])
def test_one_key_far_back_or_at_the_window_edge_decides_the_output(pkg, cuda, window, decoded):
    # the last query sits at position 299 and the key that matters at position 5: far inside a window of 1000, the oldest key a window
    # of 295 keeps, the newest key a window of 294 has dropped.  Decoded: the last 20 tokens one by one, the ring cache has wrapped.
    cfg, bits, W, toks = one_key_case(window)
    want, _ = R.forward(cfg, W, toks)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["mask"]["size"] = 294 if window != 294 else 295
    moved, _ = R.forward(other, W, toks)
    assert R.rel_err(moved[-1:], want[-1:])[0] > 0.05           # the test is blind unless one position of window decides the answer
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 280) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_the_window_passes_over_decoded_tokens_many_times(pkg, cuda, dtype, tol):
    # windows of 1, 2, 5 and 17 rows: every decoded token overwrites the oldest row of each ring; 150 steps wrap them many times
    cfg = config([att_layer(window=17, mlp=dense_ff(40)), att_layer(heads=2, kv_heads=2, dim=8, vdim=8, window=1),
                  att_layer(heads=2, kv_heads=1, dim=12, vdim=20, window=2, mlp=moe_ff()), att_layer(heads=3, kv_heads=1, dim=8, vdim=8, window=5)])
    bits, W = R.random_weights(cfg, seed=12)
    toks = tokens_for(cfg, 170, 5)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_decoded(m, toks, 20), want, tol, sure)
    check(run_decoded(m, toks, 3), want, tol, sure)             # the prompt is shorter than a window
    m.close()


@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130, 200])
def test_lengths_and_windows_around_the_edges_of_tiles(pkg, cuda, n):
    # prompt attention walks 32 or 64 keys per tile and 4 or 64 queries per CTA, decode attention 128 cache rows per pass: a prompt that
    # ends just before, at and just after an edge, windows that end there too, then two decoded tokens
    cfg = config([att_layer(heads=2, kv_heads=1, dim=8, vdim=16, window=64), att_layer(heads=2, kv_heads=2, dim=8, vdim=12, window=33),
                  att_layer(heads=2, kv_heads=1, dim=8, vdim=8, window=max(n - 1, 1))], width=32, vocab=53)
    bits, W = R.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, n + 2, n)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    check(run_decoded(m, toks, n), want, F32_TOL)
    m.close()


def test_first_tokens_of_a_sequence(pkg, cuda):
    # position 0 sees only itself and takes the first row of the position table
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=14)
    m = load(pkg, cfg, bits)
    for tok in (0, 7, cfg["vocab"] - 1):
        want, _ = R.forward(cfg, W, [tok])
        check(run_whole(m, [tok]), want, F32_TOL)
    toks = tokens_for(cfg, 3, 9)
    want, _ = R.forward(cfg, W, toks)
    check(run_decoded(m, toks, 1), want, F32_TOL)
    m.close()


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_long_decoding(pkg, cuda, dtype, tol):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=15)
    toks = tokens_for(cfg, 260, 6)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_decoded(m, toks, 4), want, tol, sure)
    m.close()


def test_the_position_table_ends_the_sequence(pkg, cuda):
    cfg = config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8)], max_positions=12)
    bits, W = R.random_weights(cfg, seed=22)
    toks = tokens_for(cfg, 13, 3)
    want, _ = R.forward(cfg, W, toks[:12])
    m = load(pkg, cfg, bits)
    s = m.seq_alloc()
    with pytest.raises(Exception):
        m.batch_step([(s, toks, [12])])                         # position 12 has no vector
    check(m.batch_step([(s, toks[:11], list(range(11)))])[0], want[:11], F32_TOL)
    check(m.batch_step([(s, toks[11:12], [0])])[0], want[11:], F32_TOL)
    with pytest.raises(Exception):
        m.batch_step([(s, toks[12:], [0])])
    m.close()


ODD = {
    "one_of_everything": lambda: config([att_layer(heads=1, kv_heads=1, dim=4, vdim=4, window=1, mlp=moe_ff(experts=1, top=1, ff=8, count=1, keep=1, shared=8))],
                                        width=16, vocab=11),
    "every_expert_chosen": lambda: config([att_layer(mlp=moe_ff(experts=4, top=4, ff=24, count=2, keep=2, shared=None))]),
    "odd_sizes": lambda: config([att_layer(heads=3, kv_heads=1, dim=10, vdim=13, window=6, mlp=dense_ff(50)),
                                 att_layer(heads=10, kv_heads=5, dim=6, vdim=9, window=21, mlp=moe_ff(experts=15, top=4, ff=18, count=5, keep=2, shared=10)),
                                 att_layer(heads=2, kv_heads=2, dim=9, vdim=35, window=400)], width=30, vocab=67),
    "wide_heads": lambda: config([att_layer(heads=2, kv_heads=1, dim=136, vdim=72, window=30), att_layer(heads=2, kv_heads=2, dim=40, vdim=264, window=19)],
                                 width=64, vocab=31),
    "no_feed_forward_anywhere": lambda: config([att_layer(), att_layer(window=3), att_layer(heads=2, kv_heads=1)]),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(ODD))
def test_other_sizes(pkg, cuda, which, dtype, tol):
    cfg = ODD[which]()
    bits, W = R.random_weights(cfg, seed=16)
    toks = tokens_for(cfg, 45, 7)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_whole(m, toks), want, tol, sure)
    check(run_decoded(m, toks, 20), want, tol, sure)
    m.close()


def test_many_tokens_take_the_sorted_expert_path(pkg, cuda):
    # a prompt long enough for the per-expert products, against the same tokens decoded one by one (the per-pair path)
    cfg = config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff(experts=9, top=3, ff=48, count=3, keep=2))])
    bits, W = R.random_weights(cfg, seed=17)
    toks = tokens_for(cfg, 150, 8)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    whole = run_whole(m, toks)
    check(whole, want, F32_TOL)
    dec = run_decoded(m, toks, 1)
    assert np.abs(whole - dec).max() < 5e-5 * np.abs(whole).max()
    m.close()


@pytest.mark.parametrize("experts,count", [(3, 1), (12, 4)])
def test_expert_products_over_wide_token_tiles(pkg, cuda, experts, count):
    # 1200 (token, choice) pairs: 400 or 100 rows per expert on average, so the grouped tensor-core product runs its 256- and 128-token
    # tiles, with experts whose rows end inside a tile
    cfg = config([att_layer(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe_ff(experts=experts, top=2, ff=48, count=count, keep=max(count - 1, 1), shared=32))],
                 width=64, vocab=97, max_positions=640)
    bits, W = R.random_weights(cfg, seed=21)
    toks = tokens_for(cfg, 600, 9)
    want, _, sure = oracle(cfg, W, toks, "bfloat16")
    m = load(pkg, cfg, bits, "bfloat16", n_ctx=640, n_seq=2)
    check(run_whole(m, toks), want, BF16_TOL, sure)
    m.close()


def test_greedy_generation_through_the_scheduler(pkg, cuda):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=18, gain=1.5)
    m = load(pkg, cfg, bits, n_seq=2)                           # fewer slots than requests: two batches
    prompts = [tokens_for(cfg, n, 30 + n) for n in (5, 19, 11)]
    outs = pkg.BatchScheduler(m).generate(prompts, 6)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        seq = list(p)
        for tok in o:
            lg, _ = R.forward(cfg, W, seq)
            top2 = np.sort(lg[-1])[-2:]
            if top2[1] - top2[0] > 1e-3 * np.abs(lg[-1]).max():   # a clear winner must be the engine's choice
                assert int(np.argmax(lg[-1])) == tok
            seq.append(tok)
    m.close()


def test_directory_loader_and_trace_replay(pkg, cuda, tmp_path):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=19)
    d = tmp_path / "model"
    R.write_model_dir(str(d), cfg, bits)
    toks = tokens_for(cfg, 30, 4)
    want, _ = R.forward(cfg, W, toks)
    m = pkg.Model.from_dir(str(d), dtype="float32", n_ctx=64, n_seq=2)
    check(run_whole(m, toks), want, F32_TOL)
    m.close()
    for gone in ("l1.mlp.e3.up", "l1.mlp.correction", "l0.norm2.b", "pos"):
        part = {k: v for k, v in bits.items() if k != gone}
        R.write_model_dir(str(d), cfg, part)
        with pytest.raises(Exception):
            pkg.Model.from_dir(str(d), dtype="float32", n_ctx=64, n_seq=2)
    # the command-line replay: a prompt of two requests, then one decoded token each
    R.write_model_dir(str(d), cfg, bits)
    a, b = toks[:20], tokens_for(cfg, 8, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:19], "want": [0, 18]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[19:], "want": [0]}, {"id": "b", "tokens": b[7:], "want": [0]}], "end": ["a", "b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert "done 0" in p.stdout and "done 1" in p.stdout
        wa, _, sa = oracle(cfg, W, a, dtype)
        wb, _, sb = oracle(cfg, W, b, dtype)
        g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
        g1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1)
        if sa is not None:                                      # bfloat16: the replay must run; rows routed by a close call are not compared
            g0, g1 = g0[[sa[0], sa[18], sb[6]]], g1[[sa[19], sb[7]]]
            w0, w1 = np.stack([wa[0], wa[18], wb[6]])[[sa[0], sa[18], sb[6]]], np.stack([wa[19], wb[7]])[[sa[19], sb[7]]]
        else:
            w0, w1 = np.stack([wa[0], wa[18], wb[6]]), np.stack([wa[19], wb[7]])
        if len(g0):
            check(g0, w0, tol)
        if len(g1):
            check(g1, w1, tol)
