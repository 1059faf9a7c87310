"""CPU-side tests of the Sapudra design: its place in the architecture table, configurations the reader refuses, and the float64
oracle's own invariants (the GPU tests compare the engine with that oracle)."""
import json

import numpy as np

import ref_sapudra as R


def att(heads=2, kv_heads=1, dim=4, vdim=4, window=5, scale=0.5, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}, "mlp": mlp}


def moe(experts=6, top=2, ff=8, count=3, keep=2, scale=1.5, shared=4):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def tiny(layers, width=16, vocab=8, max_positions=32, mult=0.7, cap=12.0):
    return {"architecture": "Sapudra", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": 1e-5}, "residual_mult": mult,
            "logit_softcap": cap, "layers": layers}


def test_architecture_table(lib):
    names = [lib.c.pb200_arch_name(i).decode() for i in range(lib.c.pb200_arch_count())]
    assert "Sapudra" in names
    assert lib.c.pb200_arch_family(b"Sapudra") == 1


def test_bad_configurations_are_refused_before_any_device_work(lib):
    mk = lib.c.pb200_model_create_from_config

    def refused(cfg):
        return not mk(json.dumps(cfg).encode(), 30, 0, 64, 1)
    assert refused(tiny([]))
    assert refused(tiny([att()], max_positions=0))                                                      # no position table
    assert refused(tiny([{"type": "mamba2", "mixer": {"heads": 2, "vdim": 4, "state": 4}}]))            # another design's mixer
    assert refused(tiny([att(heads=3, kv_heads=2)]))                                                    # query heads per key head
    assert refused(tiny([att(mlp=moe(experts=6, top=7))]))                                              # more choices than experts
    assert refused(tiny([att(mlp=moe(experts=6, count=4))]))                                            # groups must be equal
    assert refused(tiny([att(mlp=moe(experts=6, count=3, keep=4))]))                                    # more groups kept than there are
    assert refused(tiny([att(mlp=moe(experts=6, top=3, count=3, keep=1))]))                             # the kept groups hold too few experts
    assert refused(tiny([att(mlp={"kind": "gated", "ff": 8})]))                                         # unknown feed-forward


def test_layer_norm_and_head_norm():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 12)) * 3 + 2
    y = R.layer_norm(x, np.ones(12), np.zeros(12), 0.0)
    assert np.allclose(y.mean(-1), 0.0) and np.allclose((y ** 2).mean(-1), 1.0)
    w, b = rng.standard_normal(12), rng.standard_normal(12)
    assert np.allclose(R.layer_norm(x, w, b, 0.0), y * w + b)
    # eps sits inside the root
    assert np.allclose(R.layer_norm(np.zeros((1, 4)), np.ones(4), np.full(4, 0.5), 1e-3), 0.5)
    q = rng.standard_normal((3, 2, 6))
    n = R.head_norm(q, np.full(6, 2.0), 0.0)
    assert np.allclose((n ** 2).mean(-1), 4.0)                                  # every head by itself, the weight shared
    assert np.allclose(R.head_norm(5 * q, np.full(6, 2.0), 0.0), n)


def test_window_visibility():
    assert R.visible(7, 7, 1) and not R.visible(7, 6, 1)
    assert R.visible(9, 5, 5) and not R.visible(9, 4, 5)
    assert not R.visible(3, 4, 100)
    cfg = tiny([att(window=3)])
    _, W = R.random_weights(cfg, seed=1)
    c = cfg["layers"][0]["mixer"]
    rng = np.random.default_rng(2)
    h = rng.standard_normal((9, 16))
    base = R.window_attention(h, W, "l0.mix.", c, 1e-5)
    h2 = h.copy()
    h2[4] += 1.0                                                                # position 4 is seen by 4, 5, 6 and nobody else
    moved = np.abs(R.window_attention(h2, W, "l0.mix.", c, 1e-5) - base).max(-1)
    assert np.all(moved[[4, 5, 6]] > 1e-6) and np.all(moved[[0, 1, 2, 3, 7, 8]] == 0.0)


def test_grouped_heads_share_keys_and_values():
    cfg = tiny([att(heads=4, kv_heads=2, dim=4, vdim=3, window=50)])
    _, W = R.random_weights(cfg, seed=3)
    c = cfg["layers"][0]["mixer"]
    h = np.random.default_rng(4).standard_normal((6, 16))
    base = R.window_attention(h, W, "l0.mix.", c, 1e-5)
    # the same result from four key / value heads that repeat the two
    c4 = dict(c, kv_heads=4)
    W4 = dict(W)
    W4["l0.mix.k"] = np.repeat(W["l0.mix.k"].reshape(2, 4, 16), 2, axis=0).reshape(16, 16)
    W4["l0.mix.v"] = np.repeat(W["l0.mix.v"].reshape(2, 3, 16), 2, axis=0).reshape(12, 16)
    assert np.allclose(R.window_attention(h, W4, "l0.mix.", c4, 1e-5), base)


def test_router():
    rng = np.random.default_rng(5)
    E, Wd = 12, 10
    W = {"r.router": rng.standard_normal((E, Wd)), "r.correction": 0.4 * rng.standard_normal(E)}
    h = rng.standard_normal((64, Wd))
    r = {"experts": E, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}
    idx, wts = R.route(h, W, "r.", r)
    s = R.sigmoid(h @ W["r.router"].T)
    choice = s + W["r.correction"]
    free_idx, _ = R.route(h, W, "r.", dict(r, groups={"count": 1, "keep": 1}))
    plain_idx, _ = R.route(h, {"r.router": W["r.router"], "r.correction": np.zeros(E)}, "r.", r)
    assert np.allclose(wts.sum(-1), 2.5)
    for t in range(64):
        assert len(set(idx[t] // 3)) <= 2                                       # the chosen experts live in two groups
        assert np.all(np.diff(choice[t, idx[t]]) <= 1e-12)                      # in the order of the choice score
        assert np.allclose(wts[t], s[t, idx[t]] / s[t, idx[t]].sum() * 2.5)     # weights from the scores without the correction
    assert any(set(idx[t]) != set(free_idx[t]) for t in range(64))              # the groups change the choice for some token
    assert any(set(idx[t]) != set(plain_idx[t]) for t in range(64))             # and so does the correction
    # choice scores below zero: an expert outside the kept groups must not win because "not eligible" was written as 0
    Wn = {"r.router": W["r.router"], "r.correction": W["r.correction"] - 3.0}
    nidx, _ = R.route(h, Wn, "r.", r)
    assert np.array_equal(nidx, idx)
    # a group of one expert scores with that expert alone
    one, _ = R.route(h, W, "r.", dict(r, top=2, groups={"count": 12, "keep": 2}))
    for t in range(64):
        assert set(one[t]) == set(np.argsort(-choice[t])[:2])


def test_feed_forward_forms():
    G = {"f.up": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), "f.down": np.array([[1.0, 0.0, 0.0], [0.0, 1.0, 2.0]])}
    y = R.relu2_unit(np.array([[2.0, -3.0]]), G, "f.")[0]
    assert np.allclose(y, [4.0, 0.0])                                           # relu(2)^2, relu(-3)^2 = 0, relu(-1)^2 = 0
    cfg = tiny([att(mlp=moe())])
    _, W = R.random_weights(cfg, seed=6)
    h = np.random.default_rng(7).standard_normal((5, 16))
    ml = cfg["layers"][0]["mlp"]
    full = R.mixture(h, W, "l0.mlp.", ml)
    bare = R.mixture(h, W, "l0.mlp.", {k: v for k, v in ml.items() if k != "shared"})
    gate = R.sigmoid(h @ W["l0.mlp.shared.sg"].T)
    assert gate.shape == (5, 1)
    assert np.allclose(full - bare, R.relu2_unit(h, W, "l0.mlp.shared.") * gate)


def test_soft_cap_positions_and_causality():
    assert np.allclose(R.soft_cap(np.array([0.0, 1e6, -1e6]), 30.0), [0.0, 30.0, -30.0])
    assert np.allclose(R.soft_cap(np.array([0.3]), 30.0), 30.0 * np.tanh(0.01))
    cfg = tiny([att(window=4, mlp={"kind": "dense", "ff": 12}), att(heads=2, kv_heads=2, window=2, mlp=moe()), att(window=9)])
    _, W = R.random_weights(cfg, seed=8)
    toks = [1, 5, 2, 7, 7, 0, 3, 3, 3]
    full, taps = R.forward(cfg, W, toks)
    part, _ = R.forward(cfg, W, toks[:4])
    assert np.allclose(full[:4], part)                                          # later tokens do not change earlier logits
    assert taps.shape == (3, 9, 16)
    assert np.abs(full).max() <= 12.0
    # equal tokens at different positions differ through the position table alone
    assert not np.allclose(R.embed(W, [3, 3])[0], R.embed(W, [3, 3])[1])
    assert np.allclose(R.embed(W, [3, 3])[1] - R.embed(W, [3, 3])[0], W["pos"][1] - W["pos"][0])
    assert np.allclose(R.embed(W, [4], pos0=6)[0], W["embed"][4] + W["pos"][6])
