"""Float64 oracle of the Zevedra design (layer-list family), written from its equations, one function per mechanism.  It shares no code
with the engine.  Shapes: a sequence is [T, width]; weights are stored [out, in] and applied as W x.

The design: the stream starts as embed[token] * scale + bigram[hash(previous token, token)]; every layer is
x <- x + m * mixer(norm(x)), x <- x + m * ff(norm(x)) with an RMS norm that has ONE learned number; a block of consecutive layers may run
several times with the same weights (before every pass but the first the embedding output is added, before every pass a step vector).
Two mixers, each two branches side by side over the same input:
  "parallel"    windowed softmax attention (short convolution on q, k, v; interleaved partial rotation; per-head unit RMS after the
                rotation; values rotated by their position and the head's result rotated back; a sigmoid gate per head)
                + the gated delta rule; result = a * left + b * right
  "parallel_2"  causal softmax attention with a zero-score sink in the denominator (RMS norm with weight over the whole q / k projection
                before a rotate-half partial rotation; a sigmoid gate per output element) + an HGRN2 recurrence;
                result = (rmsnorm(left) * w_l + rmsnorm(right) * w_r) / 2
Feed-forward: mixture of SiLU-gated experts, sigmoid router, the chosen scores multiply the experts' INPUT."""
import json
import os
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------------------------- small pieces
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    return rms_unit(x, eps) * float(g)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j); zeros before the start; the last column meets the current token."""
    T, C = u.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += pad[j:j + T] * w[:, j][None, :]
    return y


def rotate(x, pos, dims, base, layout, sign=1.0):
    """x [T, heads, d]: the first `dims` entries of every head turn by pos * base^(-2i/dims); layout "interleaved" pairs (2i, 2i+1),
    "half" pairs (i, i + dims/2).  sign -1 turns back."""
    if dims <= 0:
        return x.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = sign * np.asarray(pos, dtype=np.float64)[:, None, None] * f[None, None, :]
    c, s = np.cos(a), np.sin(a)
    y = x.copy()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2] = u * c - v * s
        y[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        y[..., :half] = u * c - v * s
        y[..., half:dims] = v * c + u * s
    return y


def visible(i, j, window):
    """Does position i see position j?  window None: every earlier position and itself.  Works on arrays."""
    d = np.asarray(i) - np.asarray(j)
    return (d >= 0) & (True if window is None else d < window)


def softmax_attention(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key / value head h // (H / G).  sink: one is added to the denominator
    (a key of score 0 without a value).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    see = visible(np.arange(T)[:, None], np.arange(T)[None, :], window)
    for h in range(H):
        g = h // (H // G)
        s = np.where(see, (q[:, h, :] @ k[:, g, :].T) * scale, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), 0.0) if sink else s.max(axis=1, keepdims=True)
        e = np.exp(s - top)
        den = e.sum(axis=1, keepdims=True) + (np.exp(-top) if sink else 0.0)
        out[:, h] = (e / den) @ v[:, g, :]
    return out


def gated_delta_rule(q, k, v, beta, g, S=None):
    """q, k [T, H, d] (already unit vectors, q scaled), v [T, H, dv], beta, g [T, H].  Per head: S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = np.zeros((H, d, dv)) if S is None else S.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            S[h] *= g[t, h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] += np.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def hgrn2(q, f, v, S=None):
    """q, f [T, H, d], v [T, H, dv]: S <- diag(f) S + (1 - f) v^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = np.zeros((H, d, dv)) if S is None else S.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            S[h] = f[t, h][:, None] * S[h] + np.outer(1.0 - f[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


# ---------------------------------------------------------------------------------------------------------------- branches
def window_attention_branch(cfg, c, W, p, h, pos):
    """Left branch of "parallel"."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    eps = cfg["norm"]["eps"]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if c.get("conv"):
        q, k, v = causal_conv(q, W[p + "q.conv"]), causal_conv(k, W[p + "k.conv"]), causal_conv(v, W[p + "v.conv"])
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    rot = c.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], "interleaved")
        k = rotate(k, pos, rot["dims"], rot["base"], "interleaved")
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    base = rot["base"] if rot else 10000.0
    v = rotate(v, pos, dv, base, "interleaved")
    window = c["mask"]["size"] if c.get("mask") else None
    o = softmax_attention(q, k, v, c["scale"], window, sink=False)
    o = rotate(o, pos, dv, base, "interleaved", sign=-1.0)
    gate = sigmoid(h @ W[p + "g"].T)                       # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def delta_branch(cfg, c, W, p, h):
    """Right branch of "parallel"."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if c.get("conv"):
        q, k, v = causal_conv(q, W[p + "q.conv"]), causal_conv(k, W[p + "k.conv"]), causal_conv(v, W[p + "v.conv"])
    q, k, v = silu(q).reshape(T, G, d), silu(k).reshape(T, G, d), silu(v).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ W[p + "b"].T)
    g = np.exp(-np.exp(W[p + "A_log"])[None, :] * softplus(h @ W[p + "a"].T + W[p + "dt_bias"][None, :]))
    o, _ = gated_delta_rule(q, k, v, beta, g)
    o = rms_unit(o, cfg["norm"]["eps"]) * W[p + "norm"][None, None, :]
    o = o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def sink_attention_branch(cfg, c, W, p, h, pos):
    """Left branch of "parallel_2"."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    eps = cfg["norm"]["eps"]
    q = rms_unit(h @ W[p + "q"].T, eps) * W[p + "q.norm"][None, :]
    k = rms_unit(h @ W[p + "k"].T, eps) * W[p + "k.norm"][None, :]
    v = h @ W[p + "v"].T
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    rot = c.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], "half")
        k = rotate(k, pos, rot["dims"], rot["base"], "half")
    window = c["mask"]["size"] if c.get("mask") else None
    o = softmax_attention(q, k, v, c["scale"], window, sink=True)
    o = o.reshape(T, H * dv) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def hgrn2_branch(cfg, c, W, p, h):
    """Right branch of "parallel_2"."""
    T = h.shape[0]
    H, d, dv = c["heads"], c["dim"], c.get("vdim", c["dim"])
    q = silu(h @ W[p + "q"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    low = W[p + "lower"][None, :]
    f = (low + (1.0 - low) * sigmoid(h @ W[p + "f"].T + W[p + "f.b"][None, :])).reshape(T, H, d)
    o, _ = hgrn2(q, f, v)
    o = rms_unit(o, cfg["norm"]["eps"]) * W[p + "norm"][None, None, :]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def mixer(cfg, layer, W, p, h, pos):
    c = layer["mixer"]
    if layer["type"] == "parallel":
        left = window_attention_branch(cfg, c["left"], W, p + "left.", h, pos)
        right = delta_branch(cfg, c["right"], W, p + "right.", h)
        return c.get("left_scale", 1.0) * left + c.get("right_scale", 1.0) * right
    if layer["type"] == "parallel_2":
        eps = cfg["norm"]["eps"]
        left = sink_attention_branch(cfg, c["left"], W, p + "left.", h, pos)
        right = hgrn2_branch(cfg, c["right"], W, p + "right.", h)
        return 0.5 * (rms_unit(left, eps) * W[p + "left.out"][None, :] + rms_unit(right, eps) * W[p + "right.out"][None, :])
    raise ValueError(layer["type"])


# ---------------------------------------------------------------------------------------------------------------- feed-forward
def route(mlp, W, p, h):
    """Scores s = sigmoid(W_r h); the `top` largest (ties: the lower index).  Returns (idx [T, top], s [T, experts], margin [T])."""
    s = sigmoid(h @ W[p + "router"].T)
    top = mlp["router"]["top"]
    order = np.argsort(-s, axis=1, kind="stable")
    idx = order[:, :top]
    srt = np.take_along_axis(s, order, axis=1)
    margin = srt[:, top - 1] - srt[:, top] if s.shape[1] > top else np.full(s.shape[0], np.inf)
    return idx, s, margin


def moe(mlp, W, p, h, margins=None):
    idx, s, margin = route(mlp, W, p, h)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in idx[t]:
            xin = s[t, e] * h[t]
            a = silu(W[f"{p}e{e}.gate"] @ xin) * (W[f"{p}e{e}.up"] @ xin)
            out[t] += W[f"{p}e{e}.down"] @ a
    return out


# ---------------------------------------------------------------------------------------------------------------- the model
def embedding(cfg, W, toks):
    e = cfg["embedding"]
    toks = np.asarray(toks)
    x = W["embed"][toks] * e.get("scale", 1.0)
    bg = e.get("bigram")
    if bg:
        rows = [bg["buckets"]] + [int((int(toks[i - 1]) * bg["mul_prev"] + int(toks[i]) * bg["mul_cur"]) % bg["buckets"]) for i in range(1, len(toks))]
        x = x + W["bigram"][rows]
    return x


def layer_runs(cfg):
    """(layer index, pass number or None): a pass number marks the first layer of a pass of the repeated block."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    runs = []
    i = 0
    while i < n:
        if lp and i == lp["start"]:
            for t in range(lp["times"]):
                for k in range(lp["start"], lp["stop"]):
                    runs.append((k, t if k == lp["start"] else None))
            i = lp["stop"]
        else:
            runs.append((i, None))
            i += 1
    return runs


def forward(cfg, W, toks, margins=None):
    """Logits [T, vocab] and the stream after every layer run [runs, T, width]."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    T = len(toks)
    pos = np.arange(T)
    x0 = embedding(cfg, W, toks)
    x = x0.copy()
    taps = []
    for il, t in layer_runs(cfg):
        layer = cfg["layers"][il]
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t][None, :]
        p = f"l{il}."
        x = x + m * mixer(cfg, layer, W, p + "mix.", scalar_norm(x, W[p + "norm1"], eps), pos)
        if layer.get("mlp"):
            x = x + m * moe(layer["mlp"], W, p + "mlp.", scalar_norm(x, W[p + "norm2"], eps), margins)
        taps.append(x.copy())
    logits = scalar_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, np.stack(taps)


# ---------------------------------------------------------------------------------------------------------------- weights for tests
def tensor_shapes(cfg):
    """name -> shape of every tensor of a configuration."""
    Wd, V = cfg["width"], cfg["vocab"]
    sh = {"embed": (V, Wd), "head": (V, Wd), "final.norm": ()}
    bg = cfg["embedding"].get("bigram")
    if bg:
        sh["bigram"] = (bg["buckets"] + 1, Wd)
    if cfg.get("loop"):
        sh["loop.step"] = (cfg["loop"]["times"], Wd)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        sh[p + "norm1"] = ()
        L, R = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, d, dv = L["heads"], L.get("kv_heads", L["heads"]), L["dim"], L.get("vdim", L["dim"])
        a = p + "mix.left."
        sh[a + "q"], sh[a + "k"], sh[a + "v"], sh[a + "o"] = (H * d, Wd), (G * d, Wd), (G * dv, Wd), (Wd, H * dv)
        if layer["type"] == "parallel":
            sh[a + "g"] = (H, Wd)
            if L.get("conv"):
                sh[a + "q.conv"], sh[a + "k.conv"], sh[a + "v.conv"] = (H * d, L["conv"]), (G * d, L["conv"]), (G * dv, L["conv"])
            H, G, d, dv = R["heads"], R.get("kv_heads", R["heads"]), R["dim"], R.get("vdim", R["dim"])
            b = p + "mix.right."
            sh[b + "q"], sh[b + "k"], sh[b + "v"] = (G * d, Wd), (G * d, Wd), (H * dv, Wd)
            if R.get("conv"):
                sh[b + "q.conv"], sh[b + "k.conv"], sh[b + "v.conv"] = (G * d, R["conv"]), (G * d, R["conv"]), (H * dv, R["conv"])
            sh[b + "b"], sh[b + "a"], sh[b + "A_log"], sh[b + "dt_bias"] = (H, Wd), (H, Wd), (H,), (H,)
            sh[b + "norm"], sh[b + "g"], sh[b + "o"] = (dv,), (H * dv, Wd), (Wd, H * dv)
        else:
            sh[a + "g"] = (H * dv, Wd)
            sh[a + "q.norm"], sh[a + "k.norm"] = (H * d,), (G * d,)
            H, d, dv = R["heads"], R["dim"], R.get("vdim", R["dim"])
            b = p + "mix.right."
            sh[b + "q"], sh[b + "f"], sh[b + "f.b"], sh[b + "lower"] = (H * d, Wd), (H * d, Wd), (H * d,), (H * d,)
            sh[b + "v"], sh[b + "norm"], sh[b + "o"] = (H * dv, Wd), (dv,), (Wd, H * dv)
            sh[p + "mix.left.out"], sh[p + "mix.right.out"] = (Wd,), (Wd,)
        mlp = layer.get("mlp")
        if mlp:
            sh[p + "norm2"] = ()
            ff = mlp["expert"]["ff"]
            sh[p + "mlp.router"] = (mlp["router"]["experts"], Wd)
            for e in range(mlp["router"]["experts"]):
                sh[f"{p}mlp.e{e}.gate"], sh[f"{p}mlp.e{e}.up"], sh[f"{p}mlp.e{e}.down"] = (ff, Wd), (ff, Wd), (Wd, ff)
    return sh


def to_bf16_bits(a):
    """Round-to-nearest-even bfloat16 bit patterns (uint16) of a float array."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def random_weights(cfg, seed=0, gain=1.0):
    """Random weights that bfloat16 holds exactly: (bits for the engine, float64 values for the oracle)."""
    rng = np.random.default_rng(seed)
    bits, W = {}, {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        n_in = shape[-1] if len(shape) == 2 else 1
        if name in ("embed", "bigram"):
            a = rng.normal(0, 0.5 if name == "bigram" else 1.0 / cfg["embedding"].get("scale", 1.0), shape)
        elif name == "loop.step":
            a = rng.normal(0, 0.3, shape)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            a = np.asarray(rng.uniform(0.7, 1.4))
        elif leaf == "conv":
            a = rng.normal(0, 0.5, shape)
        elif leaf in ("norm", "out"):
            a = rng.uniform(0.6, 1.5, shape)
        elif leaf == "A_log":
            a = rng.uniform(-2.0, 0.5, shape)
        elif leaf == "dt_bias":
            a = rng.uniform(-1.5, 1.0, shape)
        elif leaf == "lower":
            a = rng.uniform(0.0, 0.95, shape)
        elif name.endswith("f.b"):
            a = rng.normal(0, 1.0, shape)
        elif leaf == "router":
            a = rng.normal(0, 2.0 / np.sqrt(n_in), shape)
        else:
            a = rng.normal(0, (gain if name == "head" else 1.0) / np.sqrt(n_in), shape)
        b = to_bf16_bits(np.asarray(a))
        bits[name] = b
        W[name] = from_bf16_bits(b).reshape(shape)
    return bits, W


def set_weight(bits, W, name, value):
    b = to_bf16_bits(np.asarray(value))
    bits[name] = b
    W[name] = from_bf16_bits(b).reshape(np.shape(value))


def write_model_dir(path, cfg, bits, shapes=None):
    """config.json and model.safetensors (an 8-byte header length, a JSON table, then the bfloat16 data)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    shapes = shapes or tensor_shapes(cfg)
    table, blobs, at = {}, [], 0
    for name, b in bits.items():
        raw = np.ascontiguousarray(b).tobytes()
        table[name] = {"dtype": "BF16", "shape": list(shapes[name]), "data_offsets": [at, at + len(raw)]}
        at += len(raw)
        blobs.append(raw)
    head = json.dumps(table).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        f.write(b"".join(blobs))


def rel_err(got, want):
    """Per row: rms of the difference (mean removed) over the rms spread of the wanted row."""
    d = got - want
    d = d - d.mean(axis=-1, keepdims=True)
    s = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((d * d).mean(axis=-1)) / np.maximum(np.sqrt((s * s).mean(axis=-1)), 1e-30)
