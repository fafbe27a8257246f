"""Host-side pieces of the Begupel path that need no GPU: registry, configuration reader and its refusals, and the plain
oracle's own consistency (recurrences continued from a state, windows, rotated values, convolution, bigram rows)."""
import ctypes as C
import json

import numpy as np
import pytest

import begupel_fixture as F
import begupel_plain as BP


def probe(G, cfg):
    out = (C.c_int64 * 6)()
    rc = G.host_lib().bg_config_probe(json.dumps(cfg).encode(), out)
    return rc, list(out), G.host_lib().gm_last_error().decode()


def test_registry_knows_the_architecture(G):
    assert "Begupel" in G.architectures() and "Safolorn" in G.architectures()


def test_config_reader_takes_every_size_from_the_file(G):
    rc, out, _ = probe(G, F.small_config())
    assert rc == 0 and out == [4, 2, 53, 36, 3, 4]
    rc, out, _ = probe(G, F.config([F.lightning()], vocab=7, width=16, groups=1, taps=0, buckets=0, softcap=0))
    assert rc == 0 and out == [1, 0, 7, 16, 1, 0]


@pytest.mark.parametrize("breaker, word", [
    (lambda c: c["layers"][0].update(type="other_mixer"), "unknown mixer"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads must divide"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=5), "even"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(conv=12), "conv"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "'left' and 'right'"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "unknown mlp"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c.update(width=0), "positive"),
])
def test_config_reader_refuses_what_the_design_does_not_have(G, breaker, word):
    cfg = F.small_config()
    breaker(cfg)
    rc, _, msg = probe(G, cfg)
    assert rc != 0 and word in msg, msg


def test_plain_recurrences_continue_from_their_state():
    r = np.random.default_rng(0)
    T, H, G, D, Dv = 9, 4, 2, 5, 3
    q, k, v = r.standard_normal((T, G * D)), r.standard_normal((T, G * D)), r.standard_normal((T, H * Dv))
    beta, g = r.uniform(0, 1, (T, H)), r.uniform(0.5, 1, (T, H))
    o, S = BP.delta_core(q, k, v, beta, g, H, G)
    o1, S1 = BP.delta_core(q[:4], k[:4], v[:4], beta[:4], g[:4], H, G)
    o2, S2 = BP.delta_core(q[4:], k[4:], v[4:], beta[4:], g[4:], H, G, S1)
    assert np.allclose(np.concatenate([o1, o2]), o) and np.allclose(S2, S)
    # beta = 1, g = 1, a key seen twice: the second write replaces the value, the read-out returns the new one
    kk = np.zeros((2, D)); kk[:, 1] = 3.0
    vv = r.standard_normal((2, Dv))
    o, S = BP.delta_core(kk, kk, vv, np.ones((2, 1)), np.ones((2, 1)), 1, 1)
    assert np.allclose(o[1], vv[1] * D ** -0.5, atol=1e-5) and np.allclose(S[0, 1], vv[1], atol=1e-5)
    ql, kl, vl = r.standard_normal((T, H * D)), r.standard_normal((T, H * D)), r.standard_normal((T, H * Dv))
    dec = [0.3, 0.9, 0.99, 1.0]
    o, S = BP.lightning_core(ql, kl, vl, dec)
    o1, S1 = BP.lightning_core(ql[:2], kl[:2], vl[:2], dec)
    o2, S2 = BP.lightning_core(ql[2:], kl[2:], vl[2:], dec, S1)
    assert np.allclose(np.concatenate([o1, o2]), o) and np.allclose(S2, S)
    # closed form of one head: o_t = sum_s decay^(t - s) (q_t . k_s) v_s
    t = 6
    want = sum(dec[1] ** (t - s) * (ql[t, D:2 * D] @ kl[s, D:2 * D]) * vl[s, Dv:2 * Dv] for s in range(t + 1))
    assert np.allclose(o[t, Dv:2 * Dv], want)


def test_plain_window_and_rotated_values():
    r = np.random.default_rng(1)
    T, H, G, D, Dv = 12, 2, 1, 4, 6
    q, k, v = r.standard_normal((T, H * D)), r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
    fk, fv = BP.rot_freqs(30.0, D, 2.0), BP.rot_freqs(30.0, Dv)
    full = BP.window_core(q, k, v, H, G, None, 0.5, fk, fv)
    assert np.allclose(BP.window_core(q, k, v, H, G, T, 0.5, fk, fv), full)  # a window as long as the prompt hides nothing
    one = BP.window_core(q, k, v, H, G, 1, 0.5, fk, fv)                      # only itself: the value comes back unrotated
    assert np.allclose(one[:, :Dv], v) and np.allclose(one[:, Dv:], v)
    # what a key adds depends on the distance only: the same rows 7 positions later give the same output
    shifted = BP.window_core(q, k, v, H, G, 4, 0.5, fk, fv, pos=np.arange(T) + 7)
    assert np.allclose(shifted, BP.window_core(q, k, v, H, G, 4, 0.5, fk, fv))
    # the edge: with window 4 position 9 sees 6..9; making key 5 huge changes nothing, key 6 takes all the weight
    k2 = k.copy(); k2[5] *= 0; k3 = k.copy()
    assert np.allclose(BP.window_core(q, k2, v, H, G, 4, 0.5, None, None)[9], BP.window_core(q, k, v, H, G, 4, 0.5, None, None)[9])
    k3[6] = 100.0 * q[9, :D]
    assert np.allclose(BP.window_core(q, k3, v, H, G, 4, 0.5, None, None)[9, :Dv], v[6], atol=1e-6)


def test_plain_convolution_and_bigram_rows():
    r = np.random.default_rng(2)
    h, w = r.standard_normal((7, 3)), r.standard_normal((3, 4))
    y = BP.causal_conv(h, w)
    assert np.allclose(y[0], w[:, 3] * h[0]) and np.allclose(y[5], w[:, 0] * h[2] + w[:, 1] * h[3] + w[:, 2] * h[4] + w[:, 3] * h[5])
    table, big = r.standard_normal((10, 2)), r.standard_normal((6, 2))
    x = BP.embed([3, 9, 9], table, big, 5, 31, 7)
    assert np.allclose(x[0], table[3] + big[5]) and np.allclose(x[1], table[9] + big[(3 * 31 + 9 * 7) % 5])
    assert np.allclose(x[2], table[9] + big[(9 * 31 + 9 * 7) % 5])
    xg = BP.group_norm(np.array([[3.0, 4.0, 0.0, 2.0]]), np.ones(4), 2, 0.0)
    assert np.allclose(xg, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0.0, np.sqrt(2.0)]])


def test_plain_forward_runs_every_optional_part():
    cfg = F.config([F.lightning(mlp=8), F.parallel(F.left(window=0, base=0), F.right(conv=1), mlp=None)], groups=1, taps=0, buckets=0, softcap=0)
    W = BP.random_weights(cfg, 1)
    z = BP.forward([1, 2, 3, 4], W, cfg)
    assert z.shape == (4, cfg["vocab"]) and np.isfinite(z).all()
