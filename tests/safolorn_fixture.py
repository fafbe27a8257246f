"""Model folders for the Safolorn tests: small configurations of their own, random weights rounded to bfloat16,
written as config.json + model.safetensors (8-byte header length, JSON header, data)."""
import json
import os
import struct

import numpy as np

import safolorn_plain as SP


def bf16_round(a):
    """float64 / float32 array -> the nearest bfloat16 values (ties to even), as float64, and their 16-bit codes."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    codes = u.astype(np.uint16)
    return (codes.astype(np.uint32) << 16).view(np.float32).astype(np.float64), codes


def write_safetensors(path, tensors, misalign=False):
    """tensors: name -> (codes uint16, shape).  misalign: start the data at an odd byte, as files in the wild may."""
    header, blobs, off = {}, [], 0
    for name, (codes, shape) in tensors.items():
        raw = np.ascontiguousarray(codes, dtype="<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header).encode()
    if misalign and (len(text) + 8) % 2 == 0:
        text += b" "
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def mixer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=12, scale=0.3, base=100.0, scaling=True, kv_from=None, dims=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=40, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=24, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mx, mlp):
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def config(layers, vocab=61, width=48, side=5, eps=1e-5):
    c = {"architecture": "Safolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


def small_config(**kw):
    """Two caching layers, two borrowing ones, both kinds of feed-forward and a layer without one."""
    return config([layer(mixer(), dense()), layer(mixer(heads=2, dim=6, rot_dim=6, vdim=10, kv_rank=20, scaling=False), moe()),
                   layer(mixer(heads=5, dim=4, kv_from=0), None), layer(mixer(heads=2, dim=6, rot_dim=6, vdim=3, kv_rank=20, scaling=False, kv_from=1), moe(top=1)),
                   layer(mixer(kv_from=0), dense(ff=17, limit=0.5))], **kw)


def make_model(tmp, cfg, seed=0, scale=1.0, edit=None):
    """Writes the folder and returns (folder, weights as float64 of the bfloat16 values).  edit(W) may change weights
    before they are rounded (tests that make one key or the sink stand out)."""
    W = SP.random_weights(cfg, seed, scale)
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


def rel_err(got, want):
    """Root mean square of the difference over the root mean square of the wanted values."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.sqrt(np.mean((got - want) ** 2)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


def close_enough(got, want, dtype, loose=1.0):
    """float32: every row of logits within rounding of the oracle.  bfloat16: rounding may flip a close call of a router
    (another expert for one token), which moves that token's row a lot and says nothing about the mechanism: nine rows
    in ten must be within the bfloat16 tolerance and the typical row well inside it."""
    got, want = np.atleast_2d(np.asarray(got, dtype=np.float64)), np.atleast_2d(np.asarray(want, dtype=np.float64))
    assert got.shape == want.shape, (got.shape, want.shape)
    e = np.sqrt(((got - want) ** 2).mean(-1)) / (np.sqrt((want ** 2).mean()) + 1e-30)
    if dtype == "float32":
        return bool(e.max() < 3e-5 * loose)
    return bool(np.quantile(e, 0.9) < 5e-2 * loose and np.median(e) < 2.5e-2 * loose)
