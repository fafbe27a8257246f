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


def window_attention(h, w, m, eps, pre):
    """soft-max attention over a sliding window with grouped heads, a norm over the whole q / k projection, rotary
    positions on q and k, and values that are rotated by their own position and turned back at the reader's"""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    nd = rot["dims"]
    pos = np.arange(T)
    q = rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    k = rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = h @ w[pre + "v"].T
    fk = rot["base"] ** (-2.0 * np.arange(nd // 2) / nd)
    if rot.get("scaling"):
        fk = fk / rot["scaling"]["factor"]
    fv = rot["base"] ** (-2.0 * np.arange(Dv // 2) / Dv)
    out = np.zeros((T, H * Dv))
    for hd in range(H):
        g = hd // (H // G)
        qh = rotate_pairs(q[:, hd * D:(hd + 1) * D], pos, fk)
        kh = rotate_pairs(k[:, g * D:(g + 1) * D], pos, fk)
        vh = rotate_pairs(v[:, g * Dv:(g + 1) * Dv], pos, fv)
        s = (qh @ kh.T) * m["scale"]
        d = pos[:, None] - pos[None, :]
        s = np.where((d >= 0) & (d < m["mask"]["size"]), s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, hd * Dv:(hd + 1) * Dv] = rotate_pairs(p @ vh, pos, fv, -1.0)
    return out @ w[pre + "o"].T


def delta_rule(h, w, m, eps, pre):
    """gated delta rule: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q"""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"]))
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"]))
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"]))
    beta = sigmoid(h @ w[pre + "b"].T)
    g = np.exp(-np.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    gate = silu(h @ w[pre + "g"].T)
    out = np.zeros((T, H * Dv))
    for hd in range(H):
        kv = hd // (H // G)
        qh = q[:, kv * D:(kv + 1) * D]
        kh = k[:, kv * D:(kv + 1) * D]
        qh = qh / np.sqrt((qh * qh).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
        kh = kh / np.sqrt((kh * kh).sum(-1, keepdims=True) + 1e-6)
        vh = v[:, hd * Dv:(hd + 1) * Dv]
        S = np.zeros((D, Dv))
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (vh[t] - S.T @ kh[t])
            S = S + np.outer(kh[t], u)
            out[t, hd * Dv:(hd + 1) * Dv] = S.T @ qh[t]
        o = out[:, hd * Dv:(hd + 1) * Dv]
        out[:, hd * Dv:(hd + 1) * Dv] = rms(o, eps) * w[pre + "norm"]
    return (out * gate) @ w[pre + "o"].T


def parallel_mixer(h, w, m, eps, pre):
    return m["left_scale"] * window_attention(h, w, m["left"], eps, pre + "left.") + \
        m["right_scale"] * delta_rule(h, w, m["right"], eps, pre + "right.")


def lightning(h, w, m, eps, pre):
    """per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; heads normed together, gated, projected"""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T)
    k = silu(h @ w[pre + "k"].T)
    v = silu(h @ w[pre + "v"].T)
    out = np.zeros((T, H * Dv))
    for hd in range(H):
        S = np.zeros((D, Dv))
        for t in range(T):
            S = m["decay"][hd] * S + np.outer(k[t, hd * D:(hd + 1) * D], v[t, hd * Dv:(hd + 1) * Dv])
            out[t, hd * Dv:(hd + 1) * Dv] = S.T @ q[t, hd * D:(hd + 1) * D]
    out = rms(out, eps) * w[pre + "norm"] * sigmoid(h @ w[pre + "g"].T)
    return out @ w[pre + "o"].T


def dense_ff(x, w, pre):
    gate = np.maximum(x @ w[pre + "gate"].T + w[pre + "gate.b"], 0.0)
    up = x @ w[pre + "up"].T + w[pre + "up.b"]
    return (gate * up) @ w[pre + "down"].T + w[pre + "down.b"]


def layer(x, w, cfg, li):
    L = cfg["layers"][li]
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    pre = "l%d." % li
    h = x + causal_conv(x, w[pre + "canon1"])
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
    b = cfg["embedding"]["bigram"]
    x = embed(tokens, w["embed"], w["bigram"], b["buckets"], b["mul_prev"], b["mul_cur"])
    for li in range(len(cfg["layers"])):
        x = layer(x, w, cfg, li)
        if layers_out is not None:
            layers_out.append(x.copy())
    z = group_norm(x, w["final.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"]) @ w["head"].T
    cap = cfg["logit_softcap"]
    return cap * np.tanh(z / cap)
