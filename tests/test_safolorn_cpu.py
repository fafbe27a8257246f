"""Host-side pieces of the Safolorn path that need no GPU: configuration reader, safetensors reader, registry, and the
plain oracle's own consistency (whole prompt = portions = token by token)."""
import ctypes as C
import json

import numpy as np
import pytest

import safolorn_fixture as F
import safolorn_plain as SP


def probe(G, cfg):
    out = (C.c_int64 * 5)()
    rc = G.host_lib().sf_config_probe(json.dumps(cfg).encode(), out)
    return rc, list(out), G.host_lib().gm_last_error().decode()


def test_registry_knows_the_architecture(G):
    assert "Safolorn" in G.architectures()


def test_config_reader_takes_every_size_from_the_file(G):
    rc, out, _ = probe(G, F.small_config())
    assert rc == 0 and out == [5, 2, 61, 48, 5]
    rc, out, _ = probe(G, F.config([F.layer(F.mixer(), None)], vocab=7, width=16, side=0))
    assert rc == 0 and out == [1, 1, 7, 16, 0]


@pytest.mark.parametrize("breaker, word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=99), "same kv_rank"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "own cache"),
    (lambda c: c["layers"][0].update(type="other_mixer"), "unknown mixer"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="odd"), "unknown mlp"),
    (lambda c: c.update(width=0), "positive"),
])
def test_config_reader_refuses_what_the_design_does_not_have(G, breaker, word):
    cfg = F.small_config()
    breaker(cfg)
    rc, _, msg = probe(G, cfg)
    assert rc != 0 and word in msg, msg


def test_safetensors_reader_with_data_at_an_odd_byte(G, tmp_path):
    d, vals = F.make_model(str(tmp_path / "m"), F.small_config(), seed=3)
    shape, nbytes, n = (C.c_int64 * 8)(), C.c_int64(), C.c_int64()
    dt = C.create_string_buffer(16)
    nd = G.host_lib().st_probe((d + "/model.safetensors").encode(), b"l1.mlp.e3.up", shape, C.byref(nbytes), dt, 16, C.byref(n))
    assert nd == 2 and list(shape)[:2] == [24, 48] and nbytes.value == 24 * 48 * 2 and dt.value == b"BF16"
    assert n.value == len(vals)
    assert G.host_lib().st_probe((d + "/model.safetensors").encode(), b"l0.norm1", shape, None, None, 0, None) == 0
    assert G.host_lib().st_probe((d + "/model.safetensors").encode(), b"nope", shape, None, None, 0, None) == -2
    (tmp_path / "bad.safetensors").write_bytes(b"\xff" * 12)
    assert G.host_lib().st_probe(str(tmp_path / "bad.safetensors").encode(), b"x", shape, None, None, 0, None) == -1


def test_plain_oracle_portions_equal_the_whole_prompt():
    cfg = F.small_config()
    W = SP.random_weights(cfg, 5)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 23)
    whole = SP.Plain(cfg, W).forward(toks)
    m, parts = SP.Plain(cfg, W), []
    for lo, hi in ((0, 5), (5, 7), (7, 8), (8, 20), (20, 23)):
        parts.append(m.forward(toks[lo:hi]))
    assert np.allclose(np.concatenate(parts), whole, rtol=0, atol=1e-9)


def test_plain_oracle_mechanisms():
    # sink: with no key visible but itself, the weight on the own value is exp(s) / (exp(s) + exp(sink))
    cfg = F.config([F.layer(F.mixer(heads=1, scaling=False), None)], side=0)
    W = SP.random_weights(cfg, 2)
    h = np.random.default_rng(0).standard_normal((1, cfg["width"]))
    p = np.zeros(1, dtype=np.int64)
    mx = cfg["layers"][0]["mixer"]
    c, kr = SP.latent_kv(h, p, mx, W, "l0.", 1e-5)
    W["l0.mix.sink"] = np.array([-1e9])
    no_sink = SP.latent_attention(h, p, mx, W, "l0.", c, kr, p)
    W["l0.mix.sink"] = np.array([1e9])
    all_sink = SP.latent_attention(h, p, mx, W, "l0.", c, kr, p)
    assert np.abs(all_sink).max() < 1e-12 and np.abs(no_sink).max() > 1e-3
    # rotation: position 0 leaves a vector alone up to the magnitude factor; pairs are (2i, 2i + 1)
    rot = F.mixer()["rot"]
    v = np.arange(1.0, 5.0)[None, :]
    f, mag = SP.rotary_frequencies(rot)
    assert np.allclose(SP.rotate_pairs(v, np.zeros(1, dtype=np.int64), rot), v * mag)
    r = SP.rotate_pairs(v, np.array([3]), rot)[0]
    a = 3 * f[0]
    assert np.allclose(r[:2], mag * np.array([1 * np.cos(a) - 2 * np.sin(a), 2 * np.cos(a) + 1 * np.sin(a)]))
    # router: weights are a soft-max over the chosen logits only
    ml = F.moe(experts=4, top=2)
    Wr = {"l0.mlp.router": np.eye(4, 6), "l0.mlp.router.b": np.array([0.0, 0.0, 0.0, 0.5])}
    idx, wt = SP.route(np.array([[1.0, 3.0, 2.0, 0.0, 0.0, 0.0]]), ml, Wr, "l0.")
    assert list(idx[0]) == [1, 2] and np.allclose(wt[0], np.exp([3.0, 2.0]) / np.exp([3.0, 2.0]).sum())
