"""CPU-side tests of the Zevedra design: its place in the architecture table, configurations the reader refuses, and the float64
oracle's own invariants (the GPU tests compare the engine with that oracle)."""
import json

import numpy as np

import ref_zevedra as R


def moe(experts=4, top=2, ff=8):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def par(heads=2, kv_heads=1, dim=4, vdim=4, window=5, rot=4, conv=3, r_heads=2, r_kv=1, r_dim=4, r_vdim=4, r_conv=2, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.5, "conv": conv, "mask": {"size": window}, "rot": {"base": 100.0, "dims": rot}}
    right = {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": r_conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.5, "right_scale": 1.5}, "mlp": mlp}


def par2(heads=2, kv_heads=1, dim=4, vdim=4, rot=2, r_heads=2, r_dim=4, r_vdim=4, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.5, "rot": {"base": 100.0, "dims": rot}}
    return {"type": "parallel_2", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}}, "mlp": mlp}


def tiny(layers, width=16, vocab=8, loop=None, bigram=(5, 3, 2)):
    c = {"architecture": "Zevedra", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "embedding": {"scale": 2.0}, "layers": layers}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def test_architecture_table(lib):
    names = [lib.c.pb200_arch_name(i).decode() for i in range(lib.c.pb200_arch_count())]
    assert "Zevedra" in names
    assert lib.c.pb200_arch_family(b"Zevedra") == 1


def test_bad_configurations_are_refused_before_any_device_work(lib):
    mk = lib.c.pb200_model_create_from_config

    def refused(cfg):
        return not mk(json.dumps(cfg).encode(), 30, 0, 64, 1)
    assert refused(tiny([]))
    assert refused(tiny([{"type": "attention", "mixer": {"heads": 2, "dim": 4}}]))                      # another design's layer
    assert refused(tiny([{"type": "parallel", "mixer": {"left": par()["mixer"]["left"]}}]))             # one branch only
    assert refused(tiny([par(heads=3, kv_heads=2)]))                                                    # query heads per key head
    assert refused(tiny([par(r_heads=3, r_kv=2)]))
    assert refused(tiny([par(rot=6)]))                                                                  # more rotated entries than a head has
    assert refused(tiny([par(rot=3)]))                                                                  # pairs need an even count
    assert refused(tiny([par(vdim=5)]))                                                                 # values turn in pairs
    assert refused(tiny([par(conv=0)]))                                                                 # the delta rule's inputs pass a convolution
    assert refused(tiny([par2(mlp=moe(experts=4, top=5))]))                                             # more choices than experts
    assert refused(tiny([par2(mlp={"kind": "dense", "ff": 8})]))                                        # unknown feed-forward
    assert refused(tiny([par(), par2()], loop=(1, 3, 2)))                                               # block beyond the last layer
    assert refused(tiny([par2()], bigram=(0, 1, 1)))                                                    # a table without buckets


def test_norms():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 12)) * 3 + 2
    y = R.rms_unit(x, 0.0)
    assert np.allclose((y ** 2).mean(-1), 1.0)
    assert np.allclose(R.scalar_norm(x, 1.75, 0.0), 1.75 * y)
    assert np.allclose(R.rms_unit(np.zeros((1, 4)), 1e-3), 0.0)                 # eps sits inside the root: no division by zero
    assert np.allclose(R.rms_unit(np.full((1, 4), 2.0), 12.0), 0.5)             # 2 / sqrt(4 + 12)


def test_causal_convolution():
    rng = np.random.default_rng(1)
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = R.causal_conv(u, w)
    for t in range(9):
        for c in range(3):
            want = sum(w[c, j] * u[t - 3 + j, c] for j in range(4) if t - 3 + j >= 0)
            assert abs(y[t, c] - want) < 1e-12
    assert np.allclose(R.causal_conv(u, np.ones((3, 1)) * 2.0), 2.0 * u)       # one tap: the current token only
    # causal: a later input changes no earlier output
    u2 = u.copy()
    u2[6] += 1.0
    assert np.allclose(R.causal_conv(u2, w)[:6], y[:6]) and not np.allclose(R.causal_conv(u2, w)[6], y[6])


def test_rotation():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((7, 2, 8))
    pos = np.arange(7) + 3
    for layout in ("interleaved", "half"):
        y = R.rotate(x, pos, 6, 50.0, layout)
        assert np.allclose(y[..., 6:], x[..., 6:])                              # the rest of a head passes unchanged
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
        assert np.allclose(R.rotate(y, pos, 6, 50.0, layout, sign=-1.0), x)
        assert np.allclose(R.rotate(x, np.zeros(7), 6, 50.0, layout), x)        # position 0 turns nothing
    # the two layouts are the same rotation under a permutation of the entries
    perm = [0, 2, 4, 1, 3, 5, 6, 7]
    assert np.allclose(R.rotate(x, pos, 6, 50.0, "interleaved")[..., perm], R.rotate(x[..., perm], pos, 6, 50.0, "half"))
    # pair i turns by position * base^(-2i/dims)
    e = np.zeros((1, 1, 4))
    e[0, 0, 2] = 1.0
    y = R.rotate(e, [5], 4, 100.0, "interleaved")
    a = 5 * 100.0 ** (-2.0 / 4)
    assert np.allclose(y[0, 0], [0, 0, np.cos(a), np.sin(a)])
    # a score between turned vectors depends on the distance only
    q, k = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    s1 = (R.rotate(q, [9], 8, 50.0, "half") * R.rotate(k, [4], 8, 50.0, "half")).sum()
    s2 = (R.rotate(q, [105], 8, 50.0, "half") * R.rotate(k, [100], 8, 50.0, "half")).sum()
    assert abs(s1 - s2) < 1e-9


def test_window_and_sink():
    T = 40
    see = R.visible(np.arange(T)[:, None], np.arange(T)[None, :], 7)
    assert see[10, 10] and see[10, 4] and not see[10, 3] and not see[10, 11]
    assert (see[:, 5].sum() == 7) and see[:, T - 1].sum() == 1                   # a position is seen by itself and the window - 1 after it
    assert R.visible(39, 0, None) and not R.visible(0, 1, None)
    rng = np.random.default_rng(3)
    q, k, v = rng.standard_normal((T, 4, 6)), rng.standard_normal((T, 2, 6)), rng.standard_normal((T, 2, 5))
    plain = R.softmax_attention(q, k, v, 0.4, None, sink=False)
    sunk = R.softmax_attention(q, k, v, 0.4, None, sink=True)
    assert np.allclose(plain[0], v[0][[0, 0, 1, 1]])                             # the first position sees itself only; heads 0, 1 -> key head 0
    assert np.allclose(sunk[0, 0], v[0, 0] * np.exp(0.4 * q[0, 0] @ k[0, 0]) / (1 + np.exp(0.4 * q[0, 0] @ k[0, 0])))
    # the sink is a key of score 0 with a zero value: add such a key before everything and the plain softmax gives the same
    for i in (3, 17):
        s = 0.4 * (q[i, 2] @ k[:i + 1, 1].T)
        e = np.exp(np.concatenate([[0.0], s]))
        want = (e[1:] / e.sum()) @ v[:i + 1, 1]
        assert np.allclose(sunk[i, 2], want)
    # grouped heads equal repeated heads
    rep = R.softmax_attention(q, np.repeat(k, 2, axis=1), np.repeat(v, 2, axis=1), 0.4, 9, sink=True)
    assert np.allclose(rep, R.softmax_attention(q, k, v, 0.4, 9, sink=True))


def test_values_turned_by_position_make_the_result_relative():
    # sum_j p_j R(j) v_j turned back by i is sum_j p_j R(j - i) v_j
    rng = np.random.default_rng(4)
    v = rng.standard_normal((6, 1, 4))
    p = rng.random(6)
    p /= p.sum()
    i = 5
    turned = R.rotate(v, np.arange(6), 4, 30.0, "interleaved")
    back = R.rotate((p[:, None, None] * turned).sum(0, keepdims=True), [i], 4, 30.0, "interleaved", sign=-1.0)
    want = sum(p[j] * R.rotate(v[j:j + 1], [j - i], 4, 30.0, "interleaved") for j in range(6))
    assert np.allclose(back, want)


def test_gated_delta_rule():
    rng = np.random.default_rng(5)
    T, H, d, dv = 12, 2, 5, 3
    k = rng.standard_normal((T, H, d))
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    q, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    one = np.ones((T, H))
    # beta = 1, no decay: right after a write the state answers the key with the value it was given
    o, S = R.gated_delta_rule(k, k, v, one, one)
    assert np.allclose(o, v)
    # beta = 0 writes nothing
    o0, S0 = R.gated_delta_rule(q, k, v, 0 * one, one)
    assert np.allclose(o0, 0) and np.allclose(S0, 0)
    # the state carries over: two halves equal the whole
    beta, g = rng.random((T, H)), rng.random((T, H))
    whole, Sw = R.gated_delta_rule(q, k, v, beta, g)
    a, Sa = R.gated_delta_rule(q[:7], k[:7], v[:7], beta[:7], g[:7])
    b, Sb = R.gated_delta_rule(q[7:], k[7:], v[7:], beta[7:], g[7:], Sa)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(Sb, Sw)
    # one step by hand: the decay comes first, the read-out sees the write
    S1 = np.zeros((1, d, dv))
    S1[0] = rng.standard_normal((d, dv))
    o1, S2 = R.gated_delta_rule(q[:1, :1], k[:1, :1], v[:1, :1], np.array([[0.3]]), np.array([[0.5]]), S1)
    Sd = 0.5 * S1[0]
    u = 0.3 * (v[0, 0] - Sd.T @ k[0, 0])
    assert np.allclose(S2[0], Sd + np.outer(k[0, 0], u)) and np.allclose(o1[0, 0], S2[0].T @ q[0, 0])


def test_hgrn2_equals_the_unrolled_sum():
    rng = np.random.default_rng(6)
    T, H, d, dv = 9, 2, 4, 3
    q, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    f = rng.uniform(0.2, 0.95, (T, H, d))
    o, _ = R.hgrn2(q, f, v)
    for t in (0, 4, 8):
        for h in range(H):
            S = np.zeros((d, dv))
            for j in range(t + 1):
                S += (np.prod(f[j + 1:t + 1, h], axis=0) * (1 - f[j, h]))[:, None] * v[j, h][None, :]
            assert np.allclose(o[t, h], S.T @ q[t, h])
    # a forget gate of one keeps the state and writes nothing
    o1, S1 = R.hgrn2(q, np.ones_like(f), v)
    assert np.allclose(o1, 0) and np.allclose(S1, 0)


def test_router_and_experts():
    cfg = tiny([par2(mlp=moe(experts=5, top=2, ff=6))])
    bits, W = R.random_weights(cfg, seed=7)
    rng = np.random.default_rng(8)
    h = rng.standard_normal((6, 16))
    idx, s, margin = R.route(cfg["layers"][0]["mlp"], W, "l0.mlp.", h)
    assert np.all((s > 0) & (s < 1)) and idx.shape == (6, 2)
    for t in range(6):
        assert set(idx[t]) == set(np.argsort(-s[t])[:2]) and margin[t] >= 0
    out = R.moe(cfg["layers"][0]["mlp"], W, "l0.mlp.", h)
    # the weight sits on the expert's input: not the same as a weight on its output, and not renormalised
    t = 0
    on_out = sum(s[t, e] * (W[f"l0.mlp.e{e}.down"] @ (R.silu(W[f"l0.mlp.e{e}.gate"] @ h[t]) * (W[f"l0.mlp.e{e}.up"] @ h[t]))) for e in idx[t])
    on_in = sum(W[f"l0.mlp.e{e}.down"] @ (R.silu(W[f"l0.mlp.e{e}.gate"] @ (s[t, e] * h[t])) * (W[f"l0.mlp.e{e}.up"] @ (s[t, e] * h[t]))) for e in idx[t])
    assert np.allclose(out[t], on_in) and not np.allclose(out[t], on_out, rtol=1e-3)


def test_embedding_and_order_of_runs():
    cfg = tiny([par(), par2(), par()], loop=(1, 3, 2), bigram=(5, 3, 2))
    bits, W = R.random_weights(cfg, seed=9)
    toks = [3, 7, 7, 0]
    x = R.embedding(cfg, W, toks)
    assert np.allclose(x[0], W["embed"][3] * 2.0 + W["bigram"][5])               # the first token takes the table's last row
    assert np.allclose(x[1], W["embed"][7] * 2.0 + W["bigram"][(3 * 3 + 7 * 2) % 5])
    assert np.allclose(x[3], W["embed"][0] * 2.0 + W["bigram"][(7 * 3 + 0) % 5])
    assert R.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    assert R.layer_runs(tiny([par(), par2()])) == [(0, None), (1, None)]
    lg, taps = R.forward(cfg, W, toks)
    assert taps.shape == (5, 4, 16) and lg.shape == (4, 8)
    # causal: a later token changes no earlier logits
    lg2, _ = R.forward(cfg, W, toks[:3] + [5])
    assert np.allclose(lg[:3], lg2[:3]) and not np.allclose(lg[3], lg2[3])
    assert set(R.tensor_shapes(cfg)) == set(bits)
