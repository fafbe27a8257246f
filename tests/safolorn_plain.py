"""A plain, slow Safolorn forward pass in numpy float64: the oracle of the Safolorn tests.

One function per mechanism, written from the design's equations; nothing here is shared with the product
path (no ctypes, no CUDA, no code of the host library).  Weights come as a dict name -> float64 array,
the configuration as the dict that config.json holds.

Notation: x residual stream [T, W]; h a layer's normed input; p positions; c latent [T, R]; kr the rotated
key part shared by the heads [T, Dr].
"""
import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_number(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return rms(x, eps) * float(np.asarray(g).reshape(-1)[0])


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """f_i of the rotation, with the YaRN blend when rot['scaling'] is there, and the factor on cos / sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, orig = float(s["factor"]), float(s["original"])

    def corr(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(corr(float(s["fast"]))), 0)
    hi = min(math.ceil(corr(float(s["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v, p, rot):
    """v [..., T, D]: the first rot['dims'] coordinates are rotated pairwise (2i with 2i+1), the rest pass."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    a = p[:, None].astype(np.float64) * f[None, :]
    cs, sn = np.cos(a) * m, np.sin(a) * m
    out = v.copy()
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * cs - w * sn
    out[..., 1:dims:2] = w * cs + u * sn
    return out


def latent_kv(h, p, mx, W, pre, eps):
    """What a layer with a down-projection of its own puts into its cache: (c, kr)."""
    R = int(mx["kv_rank"])
    d = h @ W[pre + "mix.dkv"].T
    c = norm_plain(d[:, :R], W[pre + "mix.dkv.norm"], eps)
    kr = rotate_pairs(d[:, R:], p, mx["rot"])
    return c, kr


def latent_attention(h, p, mx, W, pre, c, kr, pk):
    """h [T, W] queries at positions p [T]; c [S, R], kr [S, Dr] the cached latents at positions pk [S]."""
    H, D, Dr, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    T, S = h.shape[0], c.shape[0]
    q = (h @ W[pre + "mix.q"].T).reshape(T, H, D + Dr)
    qn, qr = q[:, :, :D], q[:, :, D:]
    qr = rotate_pairs(qr.transpose(1, 0, 2), p, mx["rot"]).transpose(1, 0, 2)
    kn = (c @ W[pre + "mix.uk"].T).reshape(S, H, D)
    v = (c @ W[pre + "mix.uv"].T).reshape(S, H, Dv)
    s = (np.einsum("thd,shd->hts", qn, kn) + np.einsum("thd,sd->hts", qr, kr)) * float(mx["scale"])
    s = np.where(pk[None, None, :] <= p[None, :, None], s, -np.inf)
    sink = W[pre + "mix.sink"]
    m = np.maximum(s.max(axis=-1), sink[:, None])
    e = np.exp(s - m[..., None])
    w = e / (e.sum(axis=-1) + np.exp(sink[:, None] - m))[..., None]
    o = np.einsum("hts,shd->thd", w, v).reshape(T, H * Dv)
    return o @ W[pre + "mix.o"].T


def ff_dense(h, ml, W, pre):
    lim = float(ml["limit"])
    g = np.minimum(h @ W[pre + "mlp.gate"].T, lim)
    u = np.clip(h @ W[pre + "mlp.up"].T, -lim, lim)
    y = g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)
    return y @ W[pre + "mlp.down"].T


def route(h, ml, W, pre):
    """Chosen experts [T, top] and their weights: softmax over the chosen logits only."""
    top = int(ml["router"]["top"])
    z = h @ W[pre + "mlp.router"].T + W[pre + "mlp.router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zs = np.take_along_axis(z, idx, axis=-1)
    e = np.exp(zs - zs.max(axis=-1, keepdims=True))
    return idx, e / e.sum(axis=-1, keepdims=True)


def ff_moe(h, ml, W, pre):
    idx, wt = route(h, ml, W, pre)
    out = np.zeros((h.shape[0], W[pre + "mlp.e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t]):
            a = np.maximum(h[t] @ W[pre + "mlp.e%d.up" % e].T, 0.0) ** 2
            out[t] += wt[t, j] * (a @ W[pre + "mlp.e%d.down" % e].T)
    return out


def side_input(x, tokens, li, cfg, W, pre):
    dim = int(cfg["token_side"]["dim"])
    e = W["side.embed"][tokens][:, li * dim:(li + 1) * dim]
    g = gelu_tanh(x @ W[pre + "side.gate"].T) * e
    y = g @ W[pre + "side.proj"].T
    return x + norm_plain(y, W[pre + "side.norm"], float(cfg["norm"]["eps"]))


class Plain:
    """Holds the latents of one sequence, so that a prompt can be fed whole, in portions or token by token."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
        self.n = 0
        self.lat = {}

    def forward(self, tokens, layers_out=None):
        cfg, W = self.cfg, self.W
        eps = float(cfg["norm"]["eps"])
        tokens = np.asarray(tokens, dtype=np.int64)
        p = np.arange(self.n, self.n + len(tokens))
        x = W["embed"][tokens]
        for li, L in enumerate(cfg["layers"]):
            pre = "l%d." % li
            mx = L["mixer"]
            h1 = norm_one_number(x, W[pre + "norm1"], eps)
            src = mx.get("kv_from")
            if src is None:
                c, kr = latent_kv(h1, p, mx, W, pre, eps)
                if li in self.lat:
                    c, kr = np.concatenate([self.lat[li][0], c]), np.concatenate([self.lat[li][1], kr])
                self.lat[li] = (c, kr)
                src = li
            c, kr = self.lat[int(src)]
            y = latent_attention(h1, p, mx, W, pre, c, kr, np.arange(c.shape[0]))
            if L.get("mlp"):
                h2 = norm_one_number(x, W[pre + "norm2"], eps)
                y = y + (ff_dense if L["mlp"]["kind"] == "dense" else ff_moe)(h2, L["mlp"], W, pre)
            x = x + y
            if cfg.get("token_side"):
                x = side_input(x, tokens, li, cfg, W, pre)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.n += len(tokens)
        return norm_one_number(x, W["final.norm"], eps) @ W["head"].T


def random_weights(cfg, seed, scale=1.0):
    """Random weights of every tensor a configuration names (float64; the caller rounds them as it likes)."""
    r = np.random.default_rng(seed)
    Wd, V = int(cfg["width"]), int(cfg["vocab"])
    W = {"embed": r.standard_normal((V, Wd)), "head": r.standard_normal((V, Wd)) / math.sqrt(Wd),
         "final.norm": np.array(1.0 + 0.1 * r.standard_normal())}
    side = cfg.get("token_side")
    if side:
        W["side.embed"] = r.standard_normal((V, len(cfg["layers"]) * int(side["dim"])))
    for li, L in enumerate(cfg["layers"]):
        pre, mx = "l%d." % li, L["mixer"]
        H, D, Dr, Dv, R = (int(mx[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))

        def lin(o, i):
            return r.standard_normal((o, i)) * scale / math.sqrt(i)
        W[pre + "norm1"] = np.array(1.0 + 0.1 * r.standard_normal())
        W[pre + "mix.q"] = lin(H * (D + Dr), Wd)
        if mx.get("kv_from") is None:
            W[pre + "mix.dkv"] = lin(R + Dr, Wd)
            W[pre + "mix.dkv.norm"] = 1.0 + 0.1 * r.standard_normal(R)
        W[pre + "mix.uk"] = lin(H * D, R)
        W[pre + "mix.uv"] = lin(H * Dv, R)
        W[pre + "mix.sink"] = r.standard_normal(H)
        W[pre + "mix.o"] = lin(Wd, H * Dv)
        ml = L.get("mlp")
        if ml:
            W[pre + "norm2"] = np.array(1.0 + 0.1 * r.standard_normal())
            if ml["kind"] == "dense":
                F = int(ml["ff"])
                W[pre + "mlp.gate"], W[pre + "mlp.up"], W[pre + "mlp.down"] = lin(F, Wd), lin(F, Wd), lin(Wd, F)
            else:
                F, E = int(ml["expert"]["ff"]), int(ml["router"]["experts"])
                for e in range(E):
                    W[pre + "mlp.e%d.up" % e], W[pre + "mlp.e%d.down" % e] = lin(F, Wd), lin(Wd, F)
                W[pre + "mlp.router"] = lin(E, Wd) * 2.0
                W[pre + "mlp.router.b"] = 0.5 * r.standard_normal(E)
        if side:
            sd = int(side["dim"])
            W[pre + "side.gate"], W[pre + "side.proj"] = lin(sd, Wd), lin(Wd, sd)
            W[pre + "side.norm"] = 0.2 * (1.0 + 0.1 * r.standard_normal(Wd))
    return W
