"""Model folders for the Begupel tests: small configurations of their own, random weights rounded to bfloat16, written as
config.json + model.safetensors."""
import json
import os

import numpy as np

import begupel_plain as BP
from safolorn_fixture import bf16_round, close_enough, rel_err, write_safetensors  # noqa: F401  (file format helpers)


def left(heads=4, kv_heads=2, dim=8, vdim=6, window=11, scale=0.4, base=50.0, dims=4, factor=2.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if base:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def right(heads=4, kv_heads=2, dim=12, vdim=5, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(lft=None, rgt=None, mlp=40, left_scale=0.8, right_scale=1.3):
    return {"type": "parallel", "mixer": {"left": lft or left(), "right": rgt or right(), "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def lightning(heads=3, dim=10, vdim=7, decay=None, mlp=None):
    decay = decay or [float(np.exp(-1.0 / (1.5 * 3.0 ** i))) for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def config(layers, vocab=53, width=36, groups=3, taps=4, eps=1e-5, buckets=29, softcap=9.0):
    c = {"architecture": "Begupel", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if taps:
        c["canon"] = {"taps": taps}
    if buckets:
        c["embedding"] = {"bigram": {"buckets": buckets, "mul_prev": 31, "mul_cur": 7}}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def small_config(**kw):
    """A lightning layer with a feed-forward first, two parallel layers (one without feed-forward), a bare lightning layer."""
    return config([lightning(mlp=24), parallel(), lightning(heads=2, dim=16, vdim=4),
                   parallel(left(heads=3, kv_heads=3, dim=6, vdim=10, window=5, dims=None, factor=None), right(heads=2, kv_heads=1, dim=7, vdim=9, conv=2), mlp=None)],
                  **kw)


def make_model(tmp, cfg, seed=0, edit=None):
    """Writes the folder; returns (folder, weights as float64 of the bfloat16 values)."""
    W = BP.random_weights(cfg, seed)
    if edit:
        edit(W)
    out, vals = {}, {}
    for k, v in W.items():
        vals[k], codes = bf16_round(v)
        out[k] = (codes, np.shape(v))
    os.makedirs(tmp, exist_ok=True)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp, "model.safetensors"), out, misalign=True)
    return tmp, vals
