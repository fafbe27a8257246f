"""Plain Begupel: a slow float64 numpy restatement of the design, one function per mechanism, whole sequences from
position 0, no cache and no state carried between calls.  The tests compare the framework against this; it shares no
code with the product.

Notation: x [T, W] residual stream; weights are dicts of float64 arrays named as in the weight file; linear weights
are [out, in] and applied as x @ w.T."""
import numpy as np


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def group_norm(x, w, groups, eps):
    """the last axis in `groups` equal consecutive parts, each divided by its own root mean square; then times w"""
    T, W = x.shape
    return rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * w


def causal_conv(h, w):
    """y_t = sum_j w[:, j] h_(t - taps + 1 + j): the last column weighs the current token, zeros before the start"""
    T, C = h.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), h], 0)
    y = np.zeros_like(h)
    for j in range(taps):
        y += pad[j:j + T] * w[:, j]
    return y


def embed(tokens, table, bigram, buckets, mul_prev, mul_cur):
    tokens = np.asarray(tokens, dtype=np.int64)
    rows = np.empty(len(tokens), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (tokens[:-1] * mul_prev + tokens[1:] * mul_cur) % buckets
    return table[tokens] + bigram[rows]


def rotate_pairs(x, pos, freqs, sign=1.0):
    """x [T, n >= 2 len(freqs)]: coordinates (2i, 2i+1) turned by sign * pos * freqs[i]; the rest untouched"""
    y = x.copy()
    n = len(freqs)
    a = sign * np.asarray(pos, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(a), np.sin(a)
    u, v = x[:, 0:2 * n:2], x[:, 1:2 * n:2]
    y[:, 0:2 * n:2] = u * c - v * s
    y[:, 1:2 * n:2] = v * c + u * s
    return y


def rot_freqs(base, dims, factor=1.0):
    return base ** (-2.0 * np.arange(dims // 2) / dims) / factor


def window_core(q, k, v, H, G, window, scale, fk, fv, pos=None):
    """q [T, H D], k [T, G D], v [T, G Dv] (normed already): rotary positions, scores of head h against key head
    h // (H / G), the keys j with 0 <= i - j < window (window None: all j <= i), soft-max, values rotated by their own
    position and the sum turned back by the reader's.  fk / fv None: no rotation.  Returns [T, H Dv]."""
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    pos = np.arange(T) if pos is None else np.asarray(pos)
    out = np.zeros((T, H * Dv))
    for hd in range(H):
        g = hd // (H // G)
        qh, kh, vh = q[:, hd * D:(hd + 1) * D], k[:, g * D:(g + 1) * D], v[:, g * Dv:(g + 1) * Dv]
        if fk is not None:
            qh, kh = rotate_pairs(qh, pos, fk), rotate_pairs(kh, pos, fk)
        if fv is not None:
            vh = rotate_pairs(vh, pos, fv)
        s = (qh @ kh.T) * scale
        d = pos[:, None] - pos[None, :]
        s = np.where((d >= 0) & ((d < window) if window else True), s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        o = p @ vh
        out[:, hd * Dv:(hd + 1) * Dv] = rotate_pairs(o, pos, fv, -1.0) if fv is not None else o
    return out


def window_attention(h, w, m, eps, pre):
    """soft-max attention over a sliding window with grouped heads, a norm over the whole q / k projection, rotary
    positions on q and k, and rotated values"""
    rot = m.get("rot")
    q = rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    k = rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = h @ w[pre + "v"].T
    fk = fv = None
    if rot:
        fk = rot_freqs(rot["base"], rot.get("dims", m["dim"]), (rot.get("scaling") or {}).get("factor", 1.0))
        fv = rot_freqs(rot["base"], m["vdim"])
    window = (m.get("mask") or {}).get("size")
    return window_core(q, k, v, m["heads"], m["kv_heads"], window, m["scale"], fk, fv) @ w[pre + "o"].T


def delta_core(q, k, v, beta, g, H, G, S0=None):
    """q, k [T, G D] (any length; made unit vectors here, q times D^-1/2), v [T, H Dv], beta, g [T, H].
    Returns (o [T, H Dv], S [H, D, Dv])."""
    T = q.shape[0]
    D, Dv = q.shape[1] // G, v.shape[1] // H
    out = np.zeros((T, H * Dv))
    S = np.zeros((H, D, Dv)) if S0 is None else S0.copy()
    for hd in range(H):
        kv = hd // (H // G)
        qh, kh = q[:, kv * D:(kv + 1) * D], k[:, kv * D:(kv + 1) * D]
        qh = qh / np.sqrt((qh * qh).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
        kh = kh / np.sqrt((kh * kh).sum(-1, keepdims=True) + 1e-6)
        for t in range(T):
            S[hd] = g[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd * Dv:(hd + 1) * Dv] - S[hd].T @ kh[t])
            S[hd] = S[hd] + np.outer(kh[t], u)
            out[t, hd * Dv:(hd + 1) * Dv] = S[hd].T @ qh[t]
    return out, S


def lightning_core(q, k, v, decay, S0=None):
    """q, k [T, H D], v [T, H Dv] (activated already): S <- decay S + k v^T, o = S^T q.  Returns (o, S [H, D, Dv])."""
    T, H = q.shape[0], len(decay)
    D, Dv = q.shape[1] // H, v.shape[1] // H
    out = np.zeros((T, H * Dv))
    S = np.zeros((H, D, Dv)) if S0 is None else S0.copy()
    for hd in range(H):
        for t in range(T):
            S[hd] = decay[hd] * S[hd] + np.outer(k[t, hd * D:(hd + 1) * D], v[t, hd * Dv:(hd + 1) * Dv])
            out[t, hd * Dv:(hd + 1) * Dv] = S[hd].T @ q[t, hd * D:(hd + 1) * D]
    return out, S


def delta_rule(h, w, m, eps, pre):
    """gated delta rule: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q"""
    T = h.shape[0]
    H, G, Dv = m["heads"], m["kv_heads"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"]))
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"]))
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"]))
    beta = sigmoid(h @ w[pre + "b"].T)
    g = np.exp(-np.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o, _ = delta_core(q, k, v, beta, g, H, G)
    o = (rms(o.reshape(T, H, Dv), eps) * w[pre + "norm"]).reshape(T, H * Dv)
    return (o * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def parallel_mixer(h, w, m, eps, pre):
    return m["left_scale"] * window_attention(h, w, m["left"], eps, pre + "left.") + \
        m["right_scale"] * delta_rule(h, w, m["right"], eps, pre + "right.")


def lightning(h, w, m, eps, pre):
    """per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; heads normed together, gated, projected"""
    o, _ = lightning_core(silu(h @ w[pre + "q"].T), silu(h @ w[pre + "k"].T), silu(h @ w[pre + "v"].T), m["decay"])
    return (rms(o, eps) * w[pre + "norm"] * sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def dense_ff(x, w, pre):
    gate = np.maximum(x @ w[pre + "gate"].T + w[pre + "gate.b"], 0.0)
    up = x @ w[pre + "up"].T + w[pre + "up.b"]
    return (gate * up) @ w[pre + "down"].T + w[pre + "down.b"]


def layer(x, w, cfg, li):
    L = cfg["layers"][li]
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    pre = "l%d." % li
    h = x + causal_conv(x, w[pre + "canon1"]) if cfg.get("canon") else x
    if L["type"] == "lightning":
        y = lightning(h, w, L["mixer"], eps, pre + "mix.")
    elif L["type"] == "parallel":
        y = parallel_mixer(h, w, L["mixer"], eps, pre + "mix.")
    else:
        raise ValueError(L["type"])
    x = x + group_norm(y, w[pre + "norm1"], groups, eps)
    if L.get("mlp"):
        x = x + group_norm(dense_ff(x, w, pre + "mlp."), w[pre + "norm2"], groups, eps)
    return x


def forward(tokens, w, cfg, layers_out=None):
    """logits [T, vocab] of a whole sequence; layers_out (a list) receives the residual stream after every layer"""
    b = (cfg.get("embedding") or {}).get("bigram")
    x = embed(tokens, w["embed"], w["bigram"], b["buckets"], b["mul_prev"], b["mul_cur"]) if b else w["embed"][np.asarray(tokens)]
    for li in range(len(cfg["layers"])):
        x = layer(x, w, cfg, li)
        if layers_out is not None:
            layers_out.append(x.copy())
    z = group_norm(x, w["final.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z


def random_weights(cfg, seed=0):
    """float64 weights of every tensor the configuration names"""
    r = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    lin = lambda o, i: r.standard_normal((o, i)) / np.sqrt(i)
    near1 = lambda n: 1.0 + 0.1 * r.standard_normal(n)
    w = {"embed": r.standard_normal((V, W)), "head": lin(V, W), "final.norm": near1(W)}
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        w["bigram"] = 0.7 * r.standard_normal((b["buckets"] + 1, W))
    for li, L in enumerate(cfg["layers"]):
        p, m = "l%d." % li, L["mixer"]
        w[p + "norm1"] = near1(W)
        if cfg.get("canon"):
            w[p + "canon1"] = 0.4 * r.standard_normal((W, cfg["canon"]["taps"]))
        if L["type"] == "lightning":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": lin(H * D, W), p + "mix.k": lin(H * D, W), p + "mix.v": lin(H * Dv, W), p + "mix.g": lin(H * Dv, W),
                      p + "mix.o": lin(W, H * Dv), p + "mix.norm": near1(H * Dv)})
        else:
            a, d = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w.update({p + "mix.left.q": lin(H * D, W), p + "mix.left.k": lin(G * D, W), p + "mix.left.v": lin(G * Dv, W),
                      p + "mix.left.q.norm": near1(H * D), p + "mix.left.k.norm": near1(G * D), p + "mix.left.o": lin(W, H * Dv)})
            H, G, D, Dv, c = d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]
            w.update({p + "mix.right.q": lin(G * D, W), p + "mix.right.k": lin(G * D, W), p + "mix.right.v": lin(H * Dv, W),
                      p + "mix.right.q.conv": 0.5 * r.standard_normal((G * D, c)), p + "mix.right.k.conv": 0.5 * r.standard_normal((G * D, c)),
                      p + "mix.right.v.conv": 0.5 * r.standard_normal((H * Dv, c)), p + "mix.right.b": lin(H, W), p + "mix.right.a": lin(H, W),
                      p + "mix.right.A_log": r.uniform(-2.0, 0.5, H), p + "mix.right.dt_bias": r.uniform(-1.0, 1.0, H),
                      p + "mix.right.norm": near1(Dv), p + "mix.right.g": lin(H * Dv, W), p + "mix.right.o": lin(W, H * Dv)})
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            w.update({p + "norm2": near1(W), p + "mlp.gate": lin(F, W), p + "mlp.gate.b": 0.2 * r.standard_normal(F), p + "mlp.up": lin(F, W),
                      p + "mlp.up.b": 0.2 * r.standard_normal(F), p + "mlp.down": lin(W, F), p + "mlp.down.b": 0.2 * r.standard_normal(W)})
    return w
