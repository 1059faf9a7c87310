"""Plain, slow float64 oracle of the Sapudra design (layer-list family), one function per mechanism, written from the equations; it
shares no code with the product.  Whole sequences at once.

Notation: h [T, width] is a sublayer's input, W a dict name -> float64 array (matrices stored [out, in]), c a mixer's configuration.

The design: the stream starts as  embed[token] + pos[position];  every layer is  x <- x + m LN(mixer(x)),  x <- x + m LN(ff(x))  where LN
is a layer norm with weight and bias on the SUBLAYER'S RESULT (the sublayers read x itself) and m one number for the whole model.  The
mixer is softmax attention over a sliding window with grouped key / value heads and an RMS norm with a shared weight on every query and
key head; positions enter nowhere else.  The feed-forward is  down(relu(up h)^2),  dense or as a mixture of experts whose router takes
sigmoid scores, chooses with an added per-expert correction among the experts of the best groups, weighs with the uncorrected scores,
and adds a shared expert behind a per-token sigmoid gate.  The logits pass a final layer norm, the head and a tanh soft-cap.
"""
import json
import os
import struct

import numpy as np


# ---- element-wise / norms ----
def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def rms_unit(x, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def soft_cap(z, cap):
    return cap * np.tanh(z / cap) if cap else z


# ---- embedding ----
def embed(W, tokens, pos0=0):
    T = len(tokens)
    return W["embed"][np.asarray(tokens)] + W["pos"][pos0:pos0 + T]


# ---- attention over a sliding window ----
def head_norm(x, w, eps):
    """x [T, heads, dim]: every head divided by its own root mean square, then the weight all heads share."""
    return rms_unit(x, eps) * w


def visible(i, j, window):
    """Query position i sees key position j: itself and the window - 1 positions before it."""
    return 0 <= i - j < window


def window_attention(h, W, pre, c, eps):
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    window = c["mask"]["size"]
    q = head_norm((h @ W[pre + "q"].T).reshape(T, H, D), W[pre + "q.norm"], eps)
    k = head_norm((h @ W[pre + "k"].T).reshape(T, G, D), W[pre + "k.norm"], eps)
    v = (h @ W[pre + "v"].T).reshape(T, G, Dv)
    out = np.zeros((T, H, Dv))
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            js = [j for j in range(T) if visible(i, j, window)]
            s = (k[js, g] @ q[i, hh]) * c["scale"]
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hh] = p @ v[js, g]
    return out.reshape(T, H * Dv) @ W[pre + "o"].T


# ---- feed-forward ----
def relu2_unit(h, W, pre):
    return np.maximum(h @ W[pre + "up"].T, 0.0) ** 2 @ W[pre + "down"].T


def route(h, W, pre, r):
    """Per token: the chosen experts (in the order of the choice) and their weights.
    s = sigmoid(router logits); choice score = s + correction; a group's score is the sum of its two largest choice scores (of its only
    one in a group of one); experts outside the `keep` best groups cannot be chosen; the `top` largest choice scores win (ties: the lower
    index); weight = s of the chosen / (their sum + 1e-20) * scale."""
    E, top = r["experts"], r["top"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    ng, keep = gr["count"], gr["keep"]
    s = sigmoid(h @ W[pre + "router"].T)
    choice = s + W[pre + "correction"]
    T = h.shape[0]
    per = E // ng
    idx = np.zeros((T, top), dtype=np.int64)
    wts = np.zeros((T, top))
    for t in range(T):
        cg = choice[t].reshape(ng, per)
        gscore = np.sort(cg, axis=-1)[:, -2:].sum(-1)
        best = np.argsort(-gscore, kind="stable")[:keep]
        allowed = np.full(E, -np.inf)
        for g in best:
            allowed[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        idx[t] = np.argsort(-allowed, kind="stable")[:top]
        st = s[t, idx[t]]
        wts[t] = st / (st.sum() + 1e-20) * r.get("scale", 1.0)
    return idx, wts


def route_margin(h, W, pre, r):
    """Per token: the smallest gap that decides the choice, i.e. between the last chosen and the best not chosen eligible choice score, and
    between the last kept and the best dropped group score.  A token with a small margin may be routed differently after rounding."""
    E, top = r["experts"], r["top"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    ng, keep = gr["count"], gr["keep"]
    choice = sigmoid(h @ W[pre + "router"].T) + W[pre + "correction"]
    per = E // ng
    out = np.full(h.shape[0], np.inf)
    for t in range(h.shape[0]):
        cg = choice[t].reshape(ng, per)
        gscore = np.sort(np.sort(cg, axis=-1)[:, -2:].sum(-1))[::-1]
        if keep < ng:
            out[t] = min(out[t], gscore[keep - 1] - gscore[keep])
        best = np.argsort(-np.sort(cg, axis=-1)[:, -2:].sum(-1), kind="stable")[:keep]
        elig = np.sort(np.concatenate([cg[g] for g in best]))[::-1]
        if top < len(elig):
            out[t] = min(out[t], elig[top - 1] - elig[top])
    return out


def mixture(h, W, pre, mlp):
    idx, wts = route(h, W, pre, mlp["router"])
    y = np.zeros((h.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t], wts[t]):
            y[t] += wt * relu2_unit(h[t:t + 1], W, pre + "e%d." % e)[0]
    if mlp.get("shared"):
        y += relu2_unit(h, W, pre + "shared.") * sigmoid(h @ W[pre + "shared.sg"].T)
    return y


def feed_forward(h, W, pre, mlp):
    if mlp["kind"] == "dense":
        return relu2_unit(h, W, pre)
    return mixture(h, W, pre, mlp)


# ---- the model ----
def forward(cfg, W, tokens, margins=None):
    """logits [T, vocab] and the stream that leaves every layer [layers, T, width], for one sequence from position 0.  margins: a list
    that receives one array [T] per mixture layer, the routing margin of every token there (route_margin)."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = embed(W, tokens)
    taps = []
    for i, l in enumerate(cfg["layers"]):
        p = "l%d." % i
        assert l["type"] == "attention"
        x = x + m * layer_norm(window_attention(x, W, p + "mix.", l["mixer"], eps), W[p + "norm1"], W[p + "norm1.b"], eps)
        if l.get("mlp"):
            if margins is not None and l["mlp"]["kind"] == "moe":
                margins.append(route_margin(x, W, p + "mlp.", l["mlp"]["router"]))
            x = x + m * layer_norm(feed_forward(x, W, p + "mlp.", l["mlp"]), W[p + "norm2"], W[p + "norm2.b"], eps)
        taps.append(x)
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return soft_cap(x @ W["head"].T, cfg.get("logit_softcap", 0.0)), np.stack(taps)


# ---- test models: shapes from a configuration, random bf16-representable weights ----
def tensor_shapes(cfg):
    Wd = cfg["width"]
    sh = {"embed": (cfg["vocab"], Wd), "pos": (cfg["max_positions"], Wd), "head": (cfg["vocab"], Wd), "final.norm": (Wd,), "final.norm.b": (Wd,)}
    for i, l in enumerate(cfg["layers"]):
        p, c = "l%d." % i, l["mixer"]
        sh[p + "norm1"] = sh[p + "norm1.b"] = (Wd,)
        H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        sh[p + "mix.q"] = (H * D, Wd)
        sh[p + "mix.k"] = (G * D, Wd)
        sh[p + "mix.v"] = (G * Dv, Wd)
        sh[p + "mix.q.norm"] = sh[p + "mix.k.norm"] = (D,)
        sh[p + "mix.o"] = (Wd, H * Dv)
        ml = l.get("mlp")
        if ml:
            sh[p + "norm2"] = sh[p + "norm2.b"] = (Wd,)
            if ml["kind"] == "dense":
                sh[p + "mlp.up"], sh[p + "mlp.down"] = (ml["ff"], Wd), (Wd, ml["ff"])
            else:
                for e in range(ml["router"]["experts"]):
                    sh[p + "mlp.e%d.up" % e], sh[p + "mlp.e%d.down" % e] = (ml["expert"]["ff"], Wd), (Wd, ml["expert"]["ff"])
                sh[p + "mlp.router"] = (ml["router"]["experts"], Wd)
                sh[p + "mlp.correction"] = (ml["router"]["experts"],)
                if ml.get("shared"):
                    sh[p + "mlp.shared.up"], sh[p + "mlp.shared.down"] = (ml["shared"]["ff"], Wd), (Wd, ml["shared"]["ff"])
                    sh[p + "mlp.shared.sg"] = (1, Wd)
    return sh


def to_bf16_bits(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bit pattern uint16 array, float64 value array); values are exactly representable in bf16."""
    rng = np.random.default_rng(seed)
    bits, vals = {}, {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif leaf.startswith("norm"):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif name == "pos":
            a = 0.5 * rng.standard_normal(shape)
        elif leaf == "router":
            a = 6.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])      # spread scores: the choice of experts is no close call
        elif leaf == "correction":
            a = 0.2 * rng.standard_normal(shape)
        else:
            a = gain * rng.standard_normal(shape) / np.sqrt(shape[-1])
        bits[name] = to_bf16_bits(a)
        vals[name] = from_bf16_bits(bits[name])
    return bits, vals


def set_weight(bits, vals, name, a):
    bits[name] = to_bf16_bits(a)
    vals[name] = from_bf16_bits(bits[name])


def write_model_dir(path, cfg, bits):
    """config.json + model.safetensors (bf16) as a loader expects them."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, off, blobs = {}, 0, []
    for name, b in bits.items():
        raw = np.ascontiguousarray(b).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(b.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def rel_err(got, want):
    """Per row: rms of the difference (mean taken off) over the rms of the wanted row (mean taken off)."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.maximum(np.sqrt((w ** 2).mean(-1)), 1e-30)
