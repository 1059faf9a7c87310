"""Zevedra (layer-list family) on the GPU against the float64 oracle of tests/ref_zevedra.py: every mechanism alone, prompts against
token-by-token decoding, prompt portions, ragged batches, slot reuse, one position that decides the output far back and just inside /
outside a window (in prompts and decoded, also after the ring cache has wrapped), a token felt hundreds of steps later through a
recurrent state, the edges of the kernels' tiles, the first tokens, long decoding, odd sizes, greedy generation through the scheduler,
the directory loader and the command-line replay.  Small configurations made here; weights are random but exactly representable in
bf16, so the float32 engine and the oracle see the same numbers and the comparison is sharp."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import ref_zevedra as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4     # relative rms error of a logits row, float32 engine vs float64 oracle
BF16_TOL = 6e-2


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def par(heads=4, kv_heads=2, dim=16, vdim=12, window=29, rot=12, base=5000.0, conv=4, scale=0.4, r_heads=4, r_kv=2, r_dim=8, r_vdim=12, r_conv=3,
        ls=0.55, rs=0.85, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "mask": {"size": window},
            "rot": {"base": base, "dims": rot}}
    right = {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": r_conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def par2(heads=4, kv_heads=2, dim=16, vdim=12, rot=8, base=20000.0, scale=0.3, r_heads=3, r_dim=8, r_vdim=20, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot}}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}
    return {"type": "parallel_2", "mixer": {"left": left, "right": right}, "mlp": mlp}


def config(layers, width=64, vocab=131, loop=None, mult=0.65, scale=6.0, bigram=(61, 37, 11), eps=1e-5):
    c = {"architecture": "Zevedra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult, "embedding": {"scale": scale},
         "layers": layers}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def every_expert(cfg):
    """The same model with at most three experts per layer, all of them chosen by every token: no score's rounding can send a token
    elsewhere.  For bfloat16 runs through several layers, where a routing flip early on would move every later row."""
    c = copy.deepcopy(cfg)
    for layer in c["layers"]:
        if layer.get("mlp"):
            n = min(layer["mlp"]["router"]["experts"], 3)
            layer["mlp"]["router"] = {"experts": n, "top": n}
    return c


def for_dtype(cfg, dtype):
    deep = len(R.layer_runs(cfg)) > 1
    return every_expert(cfg) if dtype == "bfloat16" and deep else cfg


def mixed_config():
    # five layers, the middle three run three times
    return config([par(mlp=moe()), par2(mlp=moe(experts=5, top=1, ff=32)), par(heads=6, kv_heads=1, dim=12, vdim=8, window=11, rot=4, conv=2, r_heads=2, r_kv=1,
                                                                                r_dim=16, r_vdim=8, r_conv=4),
                   par2(heads=2, kv_heads=2, dim=24, vdim=8, rot=24, r_heads=2, r_dim=12, r_vdim=12, mlp=moe(experts=4, top=3, ff=16)),
                   par(heads=2, kv_heads=2, dim=8, vdim=16, window=64, rot=8, mlp=moe())], loop=(1, 4, 3))


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


def run_rest(m, s, toks, first):
    rows = [m.batch_step([(s, toks[:first], list(range(first)))])[0]]
    for t in toks[first:]:
        rows.append(m.batch_step([(s, [t], [0])])[0])
    return np.concatenate(rows)


def run_decoded(m, toks, first):
    """The first `first` tokens as a prompt, the rest one by one; logits of every position."""
    s = m.seq_alloc()
    out = run_rest(m, s, toks, first)
    m.seq_free(s)
    return out


def check(got, want, tol, sure=None):
    """sure: rows to compare (True) and rows left out (False)."""
    e = R.rel_err(np.asarray(got, dtype=np.float64), want)
    if sure is not None:
        assert sure.mean() > 0.4
        e = np.where(sure, e, 0.0)
    assert e.max() < tol, f"worst row {int(e.argmax())}: {e.max():.3e} (tolerance {tol})"


def oracle(cfg, W, toks, dtype="float32"):
    """The oracle's logits, and for bfloat16 runs the rows up to the first token that is routed by a close call: a score that wins by
    less than bf16 rounding moves it may send the token to another expert, and the recurrent states carry that on to every later row.
    float32 runs compare every row."""
    margins = []
    want, taps = R.forward(cfg, W, toks, margins)
    sure = None
    if dtype == "bfloat16" and margins:
        close = np.min(np.stack(margins), axis=0) < 0.02
        sure = np.cumsum(close) == 0
        if sure.mean() <= 0.4:
            sure = None     # too few rows would be left: compare all, a routing flip then shows and the seed is to be changed
    return want, taps, sure


def scaled(name, f):
    return {name: lambda a: a * f}


MECHANISMS = {
    "window_attention_beside_delta_rule": lambda: (config([par()]), {}),
    "sink_attention_beside_hgrn2": lambda: (config([par2()]), {}),
    "one_key_head": lambda: (config([par(heads=5, kv_heads=1, dim=12, vdim=12, window=500, rot=12), par2(heads=3, kv_heads=1)]), {}),
    "every_head_its_own": lambda: (config([par(heads=3, kv_heads=3, dim=16, vdim=8, window=7, r_heads=3, r_kv=3), par2(heads=2, kv_heads=2)]), {}),
    "part_of_a_head_rotates": lambda: (config([par(dim=16, rot=4), par2(dim=16, rot=2)]), {}),
    "nothing_rotates": lambda: (config([par(rot=0), par2(rot=0)]), {}),
    "taps_differ_between_branches": lambda: (config([par(conv=5, r_conv=2), par(conv=1, r_conv=6)]), {}),
    "one_tap": lambda: (config([par(conv=1, r_conv=1)]), {}),
    "strong_sink": lambda: (config([par2(scale=0.05)]), {}),                 # scores near zero: the sink takes a large share
    "weak_sink": lambda: (config([par2(scale=3.0)]), {}),
    "fast_and_slow_decays": lambda: (config([par()]), {"l0.mix.right.A_log": lambda a: np.linspace(-6.0, 1.5, a.size).reshape(a.shape)}),
    "lower_bounds_near_one": lambda: (config([par2()]), {"l0.mix.right.lower": lambda a: 0.97 + 0.03 * a}),
    "moe_top_one": lambda: (config([par2(mlp=moe(experts=7, top=1))]), {}),
    "moe_every_expert_chosen": lambda: (config([par(mlp=moe(experts=3, top=3))]), {}),
    "block_runs_three_times": lambda: (config([par(mlp=moe()), par2()], loop=(0, 2, 3)), {}),
    "block_in_the_middle": lambda: (config([par2(), par(), par2(mlp=moe())], loop=(1, 2, 2)), {}),
    "block_runs_once": lambda: (config([par(), par2()], loop=(0, 1, 1)), {}),
    "no_block": lambda: (config([par(), par2(mlp=moe())]), {}),
    "no_bigram": lambda: (config([par(), par2()], bigram=None), {}),
    "bigram_of_one_bucket": lambda: (config([par2()], bigram=(1, 3, 5)), {}),
    "five_layers_looped": lambda: (mixed_config(), {}),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(MECHANISMS))
def test_each_mechanism_alone(pkg, cuda, which, dtype, tol):
    cfg, edits = MECHANISMS[which]()
    cfg = for_dtype(cfg, dtype)
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
    cfg = for_dtype(mixed_config(), dtype)
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
    for cuts in ([2, 2, 2, 55], [17, 16, 1, 27], [33, 2, 26], [60, 1], [1, 3, 57]):
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
    # caches, convolution inputs, recurrent states and the token before the next one must all start empty in a slot that is used again
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


def loud_value_case(layer, T, where, vocab=97, width=48):
    """One layer whose attention branch carries one loud position: token B (only at `where`) has an embedding along a direction that no
    other token has, and the value projection answers that direction fifty times louder than any other; so whoever sees position `where`
    gets a result far from whoever does not.  The recurrent branch is silenced (its output projection is zero)."""
    cfg = config([layer], width=width, vocab=vocab, bigram=None)
    bits, W = R.random_weights(cfg, seed=11)
    B = 5
    emb = W["embed"].copy()
    emb[:, 0] = 0.0
    emb[B, :] = 0.0
    emb[B, 0] = 4.0
    R.set_weight(bits, W, "embed", emb)
    wv = W["l0.mix.left.v"].copy()
    wv[:, 0] = 50.0 * np.sign(wv[:, 1] + 1e-9)
    R.set_weight(bits, W, "l0.mix.left.v", wv)
    R.set_weight(bits, W, "l0.mix.right.o", np.zeros_like(W["l0.mix.right.o"]))
    toks = [t if t != B else B + 1 for t in tokens_for(cfg, T, 4)]
    toks[where] = B
    return cfg, bits, W, toks


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window", [1000, 295, 294])
def test_one_position_far_back_or_at_the_window_edge_decides_the_output(pkg, cuda, window, decoded):
    # the last query sits at position 299 and the loud position at 5: far inside a window of 1000, the oldest one a window of 295 keeps,
    # the newest one a window of 294 has dropped.  Decoded: the last 20 tokens one by one, the ring cache has wrapped.  One tap, so the
    # loud value is not smeared over the following positions.
    cfg, bits, W, toks = loud_value_case(par(heads=2, kv_heads=1, dim=16, vdim=16, window=window, rot=16, conv=1, r_conv=1, scale=0.05), 300, 5)
    want, _ = R.forward(cfg, W, toks)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["left"]["mask"]["size"] = 294 if window != 294 else 295
    moved, _ = R.forward(other, W, toks)
    assert R.rel_err(moved[-1:], want[-1:])[0] > 0.05           # the test is blind unless that one position decides the answer
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 280) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("decoded", [False, True])
def test_taps_carry_a_position_across_the_window_edge(pkg, cuda, decoded):
    # four taps: the loud token at position 5 also sounds in the values of positions 6, 7, 8; a window that has dropped 5 still hears those
    cfg, bits, W, toks = loud_value_case(par(heads=2, kv_heads=1, dim=16, vdim=16, window=293, rot=16, conv=4, r_conv=2, scale=0.05), 300, 5)
    want, _ = R.forward(cfg, W, toks)
    for size in (290, 297):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        moved, _ = R.forward(other, W, toks)
        assert R.rel_err(moved[-1:], want[-1:])[0] > 0.05
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 281) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("decoded", [False, True])
def test_one_position_far_back_under_causal_attention_with_a_sink(pkg, cuda, decoded):
    # no window: position 3 of 400 must still be seen by the last query; the same model with a window that has dropped it answers otherwise
    cfg, bits, W, toks = loud_value_case(par2(heads=2, kv_heads=1, dim=16, vdim=16, rot=8, scale=0.05), 400, 3)
    want, _ = R.forward(cfg, W, toks)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["left"]["mask"] = {"size": 396}
    moved, _ = R.forward(other, W, toks)
    assert R.rel_err(moved[-1:], want[-1:])[0] > 0.05
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 370) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("which", ["delta", "hgrn2"])
def test_a_token_is_felt_hundreds_of_steps_later_through_the_state(pkg, cuda, which):
    # attention is silenced; with slow decays the first token still moves the last logits 350 positions later, in a prompt and decoded
    if which == "delta":
        cfg = config([par(window=4, r_dim=64, mlp=moe())], bigram=None)   # wide keys: a write erases little of what the state holds
        edits = {"l0.mix.left.o": lambda a: 0 * a, "l0.mix.right.A_log": lambda a: 0 * a - 7.0}
    else:
        cfg = config([par2(mlp=moe())], bigram=None)
        edits = {"l0.mix.left.o": lambda a: 0 * a, "l0.mix.right.lower": lambda a: 0 * a + 0.996}
    bits, W = R.random_weights(cfg, seed=12)
    for name, f in edits.items():
        R.set_weight(bits, W, name, f(W[name]))
    toks = tokens_for(cfg, 350, 6)
    want, _ = R.forward(cfg, W, toks)
    changed = list(toks)
    changed[0] = (toks[0] + 1) % cfg["vocab"]
    moved, _ = R.forward(cfg, W, changed)
    assert R.rel_err(moved[-1:], want[-1:])[0] > 10 * F32_TOL
    m = load(pkg, cfg, bits)
    check(run_whole(m, toks), want, F32_TOL)
    check(run_decoded(m, toks, 300), want, F32_TOL)
    m.close()


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_the_window_passes_over_decoded_tokens_many_times(pkg, cuda, dtype, tol):
    # windows of 1, 2, 5 and 17 rows: every decoded token overwrites the oldest row of each ring; 150 steps wrap them many times
    cfg = config([par(window=17, mlp=moe()), par(heads=2, kv_heads=2, dim=8, vdim=8, window=1, rot=8), par(heads=2, kv_heads=1, dim=12, vdim=20, window=2, rot=6),
                  par(heads=3, kv_heads=1, dim=8, vdim=8, window=5, rot=8)])
    cfg = for_dtype(cfg, dtype)
    bits, W = R.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, 170, 5)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_decoded(m, toks, 20), want, tol, sure)
    check(run_decoded(m, toks, 3), want, tol, sure)             # the prompt is shorter than a window
    m.close()


@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130, 200])
def test_lengths_and_windows_around_the_edges_of_tiles(pkg, cuda, n):
    # prompt attention walks 32 or 64 keys per tile and 4 or 64 queries per CTA, decode attention 128 cache rows per pass, the recurrences
    # 16 tokens per chunk: a prompt that ends just before, at and just after an edge, windows that end there too, then two decoded tokens
    cfg = config([par(heads=2, kv_heads=1, dim=8, vdim=16, window=64, rot=8), par2(heads=2, kv_heads=2, dim=8, vdim=12, rot=4),
                  par(heads=2, kv_heads=1, dim=8, vdim=8, window=max(n - 1, 1), rot=8)], width=32, vocab=53)
    bits, W = R.random_weights(cfg, seed=14)
    toks = tokens_for(cfg, n + 2, n)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    check(run_decoded(m, toks, n), want, F32_TOL)
    m.close()


def test_first_tokens_of_a_sequence(pkg, cuda):
    # the first token takes the bigram table's last row, convolutions see zeros before it, the states start at zero, position 0 turns nothing
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=15)
    m = load(pkg, cfg, bits)
    for tok in (0, 7, cfg["vocab"] - 1):
        want, _ = R.forward(cfg, W, [tok])
        check(run_whole(m, [tok]), want, F32_TOL)
    toks = tokens_for(cfg, 6, 9)
    want, _ = R.forward(cfg, W, toks)
    check(run_decoded(m, toks, 1), want, F32_TOL)
    check(run_decoded(m, toks, 2), want, F32_TOL)
    m.close()


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_long_decoding(pkg, cuda, dtype, tol):
    cfg = for_dtype(mixed_config(), dtype)
    bits, W = R.random_weights(cfg, seed=16)
    toks = tokens_for(cfg, 260, 6)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_decoded(m, toks, 4), want, tol, sure)
    m.close()


ODD = {
    "one_of_everything": lambda: config([par(heads=1, kv_heads=1, dim=4, vdim=2, window=1, rot=2, conv=1, r_heads=1, r_kv=1, r_dim=1, r_vdim=1, r_conv=1, ls=1.0,
                                             rs=1.0, mlp=moe(experts=1, top=1, ff=8)),
                                         par2(heads=1, kv_heads=1, dim=2, vdim=1, rot=2, r_heads=1, r_dim=1, r_vdim=1)], width=16, vocab=11, mult=1.0, scale=1.0,
                                        bigram=(1, 1, 1)),
    "odd_sizes": lambda: config([par(heads=3, kv_heads=1, dim=10, vdim=14, window=6, rot=6, conv=3, r_heads=6, r_kv=2, r_dim=9, r_vdim=13, r_conv=5,
                                     mlp=moe(experts=15, top=4, ff=18)),
                                 par2(heads=10, kv_heads=5, dim=6, vdim=9, rot=2, r_heads=5, r_dim=7, r_vdim=3, mlp=moe(experts=3, top=2, ff=50)),
                                 par2(heads=2, kv_heads=2, dim=9, vdim=35, rot=8, r_heads=1, r_dim=33, r_vdim=17)], width=30, vocab=67, bigram=(509, 1000003, 999983)),
    "wide_heads": lambda: config([par(heads=2, kv_heads=1, dim=136, vdim=72, window=30, rot=64, r_heads=2, r_kv=1, r_dim=136, r_vdim=40),
                                  par2(heads=2, kv_heads=2, dim=40, vdim=264, rot=40, r_heads=2, r_dim=72, r_vdim=136)], width=64, vocab=31),
    "state_in_shared_memory": lambda: config([par(heads=1, kv_heads=1, dim=8, vdim=8, rot=8, r_heads=2, r_kv=1, r_dim=264, r_vdim=24),
                                              par2(heads=1, kv_heads=1, dim=8, vdim=8, rot=8, r_heads=1, r_dim=260, r_vdim=70)], width=64, vocab=31),
    "window_longer_than_the_context": lambda: config([par(window=100000)]),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(ODD))
def test_other_sizes(pkg, cuda, which, dtype, tol):
    cfg = for_dtype(ODD[which](), dtype)
    bits, W = R.random_weights(cfg, seed=17)
    toks = tokens_for(cfg, 45, 7)
    want, _, sure = oracle(cfg, W, toks, dtype)
    m = load(pkg, cfg, bits, dtype)
    check(run_whole(m, toks), want, tol, sure)
    check(run_decoded(m, toks, 20), want, tol, sure)
    m.close()


def test_many_tokens_take_the_sorted_expert_path(pkg, cuda):
    # a prompt long enough for the per-expert products, against the same tokens decoded one by one (the per-pair path)
    cfg = config([par2(heads=1, kv_heads=1, dim=8, vdim=8, rot=8, mlp=moe(experts=9, top=3, ff=48))])
    bits, W = R.random_weights(cfg, seed=18)
    toks = tokens_for(cfg, 150, 8)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    whole = run_whole(m, toks)
    check(whole, want, F32_TOL)
    dec = run_decoded(m, toks, 1)
    assert np.abs(whole - dec).max() < 5e-5 * np.abs(whole).max()
    m.close()


def test_expert_products_over_wide_token_tiles(pkg, cuda):
    # 1200 (token, choice) pairs in bfloat16: the grouped tensor-core product with the weight applied to its gate / up results
    cfg = config([par2(heads=1, kv_heads=1, dim=8, vdim=8, rot=8, mlp=moe(experts=3, top=2, ff=48))], width=64, vocab=97)
    bits, W = R.random_weights(cfg, seed=19)
    toks = tokens_for(cfg, 600, 9)
    want, _, sure = oracle(cfg, W, toks, "bfloat16")
    m = load(pkg, cfg, bits, "bfloat16", n_ctx=640, n_seq=2)
    check(run_whole(m, toks), want, BF16_TOL, sure)
    m.close()


def test_greedy_generation_through_the_scheduler(pkg, cuda):
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=20, gain=1.5)
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
    bits, W = R.random_weights(cfg, seed=21)
    d = tmp_path / "model"
    R.write_model_dir(str(d), cfg, bits)
    toks = tokens_for(cfg, 30, 4)
    want, _ = R.forward(cfg, W, toks)
    m = pkg.Model.from_dir(str(d), dtype="float32", n_ctx=64, n_seq=2)
    check(run_whole(m, toks), want, F32_TOL)
    m.close()
    for gone in ("l1.mlp.e3.up", "l0.mix.right.k.conv", "l2.mix.left.g", "l3.mix.right.lower", "l1.mix.left.out", "l0.norm2", "bigram", "loop.step"):
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
    wa, _ = R.forward(cfg, W, a)
    wb, _ = R.forward(cfg, W, b)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "done 0" in p.stdout and "done 1" in p.stdout
    g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
    g1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1)
    check(g0, np.stack([wa[0], wa[18], wb[6]]), F32_TOL)
    check(g1, np.stack([wa[19], wb[7]]), F32_TOL)


def test_fused_and_single_step_kernels_agree(pkg, cuda, tmp_path):
    # the mixer's fused launches (preparation of both branches, both results into the output product's operand) against the same steps as
    # single kernels, one launch each (PB200_DUAL_UNFUSED), through the command-line replay: a prompt of two requests, then decoded tokens
    cfg = mixed_config()
    bits, W = R.random_weights(cfg, seed=22)
    d = tmp_path / "model"
    R.write_model_dir(str(d), cfg, bits)
    a, b = tokens_for(cfg, 40, 6), tokens_for(cfg, 9, 7)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:36], "want": list(range(36))}, {"id": "b", "tokens": b[:5], "want": [0, 4]}], "end": []}]
    for k in range(4):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[36 + k]], "want": [0]}, {"id": "b", "tokens": [b[5 + k]], "want": [0]}], "end": ["a", "b"] if k == 3 else []})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rows = {}
    for mode in ("fused", "single"):
        env = dict(os.environ)
        env.pop("PB200_DUAL_UNFUSED", None)
        if mode == "single":
            env["PB200_DUAL_UNFUSED"] = "1"
        out = tmp_path / mode
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600, env=env)
        assert p.returncode == 0, p.stderr[-2000:]
        rows[mode] = np.concatenate([np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for k in range(5)])
    wa, _ = R.forward(cfg, W, a)
    wb, _ = R.forward(cfg, W, b)
    want = np.concatenate([wa[:36], wb[[0, 4]]] + [np.stack([wa[36 + k], wb[5 + k]]) for k in range(4)])
    check(rows["fused"], want, F32_TOL)
    check(rows["single"], want, F32_TOL)
    assert np.abs(rows["fused"] - rows["single"]).max() < 2e-5 * np.abs(want).max()
