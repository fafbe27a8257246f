"""The operators that Begupel added to the CUDA layer (dense.cu: bigram rows, grouped norm with residual, biased gate,
soft cap, normed gate; recurrent.cu: carried causal convolution, lightning attention, gated delta rule;
window_attention.cu), each alone against the plain float64 functions of tests/begupel_plain.py.  Recurrent operators
are fed in portions that continue from the state they left; windows get one key made to stand out just inside and
just outside the edge, at page borders, far back and at the first positions, in portions and in single-token steps."""
import numpy as np
import pytest

import begupel_fixture as F
import begupel_plain as BP

pytestmark = pytest.mark.gpu
BF16, F32 = 30, 0
_ALIVE = []


@pytest.fixture(autouse=True)
def _release_buffers():
    yield
    _ALIVE.clear()


def dev(G, a):
    _ALIVE.append(G.DeviceBuffer.from_numpy(np.ascontiguousarray(a)))
    return _ALIVE[-1]


def zeros(G, nbytes):
    b = G.DeviceBuffer(max(int(nbytes), 16))
    b.zero()
    _ALIVE.append(b)
    return b


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def as_dt(dt, a):
    if dt == BF16:
        return F.bf16_round(a)
    a32 = f32(a)
    return a32.astype(np.float64), a32


def from_dt(dt, buf, shape):
    n = int(np.prod(shape))
    if dt == BF16:
        return (buf.download(np.uint16, n).astype(np.uint32) << 16).view(np.float32).reshape(shape).astype(np.float64)
    return buf.download(np.float32, n).reshape(shape).astype(np.float64)


def tol(dt):
    return 6e-3 if dt == BF16 else 3e-6


def ptr(b):
    return b.ptr if b is not None else None


# ------------------------------------------------------------------------------------------------ dense.cu
@pytest.mark.parametrize("dt", [F32, BF16])
def test_embed_bigram_first_token_carried_token_and_hash(gpu, dt):
    r = np.random.default_rng(0)
    V, E, buckets, mp, mc = 23, 10, 7, 1000003, 19
    tv, tu = as_dt(dt, r.standard_normal((V, E)))
    bv, bu = as_dt(dt, r.standard_normal((buckets + 1, E)))
    toks = r.integers(0, V, 9)
    want = BP.embed(toks, tv, bv, buckets, mp, mc)
    table, big = dev(gpu, tu), dev(gpu, bu)
    state = dev(gpu, np.array([12345], dtype=np.int32))  # whatever a slot's last owner left: the first token ignores it
    got = []
    for lo, hi in ((0, 1), (1, 2), (2, 6), (6, 9)):
        y = zeros(gpu, (hi - lo) * E * 4)
        gpu.check(gpu.cuda_lib().ggb_op_embed_bigram(dt, table.ptr, big.ptr, dev(gpu, toks[lo:hi].astype(np.int32)).ptr, hi - lo, E, buckets, mp, mc,
                                                     dev(gpu, np.array([lo], dtype=np.int32)).ptr, state.ptr, y.ptr), "embed_bigram")
        got.append(y.download(np.float32, (hi - lo) * E).reshape(-1, E))
        assert state.download(np.int32, 1)[0] == toks[hi - 1]
    assert F.rel_err(np.concatenate(got), want) < 1e-6


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("groups", [1, 3])
def test_group_norm_add(gpu, dt, groups):
    r = np.random.default_rng(groups)
    T, E, eps = 5, 42, 1e-3
    a, b, bias, w, x = (f32(r.standard_normal(s)) for s in ((T, E), (T, E), (E,), (E,), (T, E)))
    a[1, :E // groups] *= 50.0  # one loud part must not quieten the others when there are several
    es = 2 if dt == BF16 else 4
    for use_b, use_bias, use_x in ((True, False, True), (False, True, True), (False, False, False)):
        v = 0.7 * a.astype(np.float64) + (1.9 * b if use_b else 0) + (bias if use_bias else 0)
        n = BP.group_norm(v, w.astype(np.float64), groups, eps)
        xd, y = dev(gpu, x), zeros(gpu, T * E * es)
        gpu.check(gpu.cuda_lib().ggb_op_group_norm_add(dt, dev(gpu, a).ptr, 0.7, dev(gpu, b).ptr if use_b else None, 1.9,
                                                       dev(gpu, bias).ptr if use_bias else None, dev(gpu, w).ptr, groups, eps, E, T,
                                                       xd.ptr if use_x else None, y.ptr), "group_norm_add")
        want = x + n if use_x else n
        assert F.rel_err(from_dt(dt, y, (T, E)), want) < tol(dt)
        if use_x:
            assert F.rel_err(xd.download(np.float32, T * E).reshape(T, E), want) < 1e-6


@pytest.mark.parametrize("dt", [F32, BF16])
def test_glu_bias_softcap_and_normed_gate(gpu, dt):
    r = np.random.default_rng(3)
    T, Fd = 6, 19
    gu, bg, bu = f32(r.standard_normal((T, 2 * Fd))), f32(r.standard_normal(Fd)), f32(r.standard_normal(Fd))
    es = 2 if dt == BF16 else 4
    y = zeros(gpu, T * Fd * es)
    gpu.check(gpu.cuda_lib().ggb_op_glu_bias(dt, dev(gpu, gu).ptr, Fd, T, dev(gpu, bg).ptr, dev(gpu, bu).ptr, 0, y.ptr), "glu_bias")
    want = np.maximum(gu[:, :Fd].astype(np.float64) + bg, 0) * (gu[:, Fd:] + bu)
    assert (want == 0).any() and F.rel_err(from_dt(dt, y, (T, Fd)), want) < tol(dt)
    z = f32(r.standard_normal(50) * 30)
    zd = dev(gpu, z)
    gpu.check(gpu.cuda_lib().ggb_op_softcap(zd.ptr, 50, 11.0), "softcap")
    assert F.rel_err(zd.download(np.float32, 50), 11.0 * np.tanh(z.astype(np.float64) / 11.0)) < 1e-6
    for n_groups, gs, period, act in ((1, 21, 21, 0), (3, 7, 7, 1), (2, 40, 80, 1), (1, 777, 777, 0), (2, 512, 512, 1)):
        ld_o, ld_g = n_groups * gs + 3, n_groups * gs + 5
        o, g, w = f32(r.standard_normal((T, ld_o))), f32(r.standard_normal((T, ld_g))), f32(1 + 0.2 * r.standard_normal(period))
        y = zeros(gpu, T * n_groups * gs * es)
        gpu.check(gpu.cuda_lib().ggb_op_norm_gate(dt, dev(gpu, o).ptr, ld_o, dev(gpu, g).ptr, ld_g, T, n_groups, gs, dev(gpu, w).ptr, period, 1e-4, act,
                                                  y.ptr), "norm_gate")
        oo = o[:, :n_groups * gs].astype(np.float64).reshape(T, n_groups, gs)
        gg = g[:, :n_groups * gs].astype(np.float64)
        want = (BP.rms(oo, 1e-4).reshape(T, -1) * np.tile(w, n_groups * gs // period)) * (BP.silu(gg) if act else BP.sigmoid(gg))
        assert F.rel_err(from_dt(dt, y, (T, n_groups * gs)), want) < tol(dt)


# ------------------------------------------------------------------------------------------------ recurrent.cu
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_causal_conv_continues_over_portions(gpu, taps):
    r = np.random.default_rng(taps)
    T, Cn, ld = 97, 150, 163
    x, w = f32(r.standard_normal((T, ld))), f32(r.standard_normal((Cn, taps)))
    conv = BP.causal_conv(x[:, :Cn].astype(np.float64), w.astype(np.float64))
    for add, act, cuts in ((1, 0, [T]), (0, 1, [1, 1, 1, 2, 1, 40, 33, 2, 16]), (1, 1, [2, 3, 64, 28])):
        want = conv + (x[:, :Cn] if add else 0)
        want = BP.silu(want) if act else want
        tail = zeros(gpu, max(taps - 1, 1) * Cn * 4)
        lo, got, got16 = 0, [], []
        for c in cuts:
            y, y16 = zeros(gpu, c * (Cn + 2) * 4), zeros(gpu, c * Cn * 2)
            gpu.check(gpu.cuda_lib().ggb_op_causal_conv(BF16, dev(gpu, x[lo:lo + c]).ptr, ld, c, Cn, dev(gpu, w).ptr, taps, add, act,
                                                        tail.ptr if taps > 1 else None, y.ptr, Cn + 2, y16.ptr), "causal_conv")
            got.append(y.download(np.float32, c * (Cn + 2)).reshape(c, Cn + 2)[:, :Cn])
            got16.append(from_dt(BF16, y16, (c, Cn)))
            lo += c
        assert lo == T and F.rel_err(np.concatenate(got), want) < 2e-6, (taps, cuts)
        assert F.rel_err(np.concatenate(got16), want) < 6e-3
        if taps > 1:  # the tail is the last taps - 1 inputs, oldest first
            assert np.array_equal(tail.download(np.float32, (taps - 1) * Cn).reshape(taps - 1, Cn), x[T - taps + 1:, :Cn])


@pytest.mark.parametrize("H,D,Dv", [(3, 10, 7), (2, 64, 32), (1, 130, 40), (5, 16, 33), (2, 256, 8)])
def test_lightning_attention_in_portions(gpu, H, D, Dv):
    r = np.random.default_rng(D)
    T = 75
    ld = 2 * H * D + H * Dv + 5
    raw = f32(r.standard_normal((T, ld)) * 0.7)
    decay = f32(np.concatenate([[1.0], r.uniform(0.3, 0.999, H - 1)]))  # a head that forgets nothing among them
    q, k, v = (BP.silu(raw[:, a:b].astype(np.float64)) for a, b in ((0, H * D), (H * D, 2 * H * D), (2 * H * D, 2 * H * D + H * Dv)))
    want, S = BP.lightning_core(q, k, v, decay.astype(np.float64))
    for cuts in ([T], [1] * 5 + [2, 17, 16, 33, 2]):
        st, lo, got = zeros(gpu, H * D * Dv * 4), 0, []
        for c in cuts:
            xr, o = dev(gpu, raw[lo:lo + c]), zeros(gpu, c * (H * Dv + 1) * 4)
            base = xr.ptr.value
            gpu.check(gpu.cuda_lib().ggb_op_lightning_attn(base, base + 4 * H * D, base + 8 * H * D, ld, c, H, D, Dv, dev(gpu, decay).ptr, st.ptr,
                                                           o.ptr, H * Dv + 1), "lightning")
            got.append(o.download(np.float32, c * (H * Dv + 1)).reshape(c, -1)[:, :H * Dv])
            lo += c
        assert F.rel_err(np.concatenate(got), want) < 3e-6, cuts
        assert F.rel_err(st.download(np.float32, H * D * Dv).reshape(H, D, Dv), S) < 3e-6


@pytest.mark.parametrize("H,Gk,D,Dv", [(4, 2, 12, 5), (2, 2, 64, 32), (3, 1, 130, 40), (6, 3, 7, 33)])
def test_gated_delta_rule_in_portions(gpu, H, Gk, D, Dv):
    G = Gk
    r = np.random.default_rng(D + H)
    T = 70
    ld, ldb = 2 * G * D + H * Dv + 3, 2 * H + 1
    x = f32(r.standard_normal((T, ld)))
    ba = f32(r.standard_normal((T, ldb)) * 2)
    A_log, dtb = f32(r.uniform(-2, 0.5, H)), f32(r.uniform(-1, 1, H))
    q, k, v = (x[:, a:b].astype(np.float64) for a, b in ((0, G * D), (G * D, 2 * G * D), (2 * G * D, 2 * G * D + H * Dv)))
    beta = BP.sigmoid(ba[:, :H].astype(np.float64))
    g = np.exp(-np.exp(A_log.astype(np.float64)) * BP.softplus(ba[:, H:2 * H].astype(np.float64) + dtb))
    want, S = BP.delta_core(q, k, v, beta, g, H, G)
    for cuts in ([T], [1, 1, 1, 2, 3, 16, 17, 27, 2]):
        st, lo, got = zeros(gpu, H * D * Dv * 4), 0, []
        for c in cuts:
            xr, br, o = dev(gpu, x[lo:lo + c]), dev(gpu, ba[lo:lo + c]), zeros(gpu, c * H * Dv * 4)
            xb, bb = xr.ptr.value, br.ptr.value
            gpu.check(gpu.cuda_lib().ggb_op_gated_delta(xb, xb + 4 * G * D, xb + 8 * G * D, ld, bb, bb + 4 * H, ldb, c, H, G, D, Dv, dev(gpu, A_log).ptr,
                                                        dev(gpu, dtb).ptr, st.ptr, o.ptr, H * Dv), "gated_delta")
            got.append(o.download(np.float32, c * H * Dv).reshape(c, -1))
            lo += c
        assert F.rel_err(np.concatenate(got), want) < 5e-6, cuts
        assert F.rel_err(st.download(np.float32, H * D * Dv).reshape(H, D, Dv), S) < 5e-6


def test_gated_delta_overwrites_a_key_seen_again(gpu):
    """beta = 1 and no decay: writing a key a second time replaces its value, and the read-out sees the new one"""
    H = G = 1
    D, Dv, T = 8, 4, 3
    k = np.zeros((T, D)); k[0, 2] = k[2, 2] = 5.0; k[1, 5] = 1.0
    v = np.random.default_rng(0).standard_normal((T, Dv))
    x = f32(np.concatenate([k, k, v], 1))
    ba = f32(np.concatenate([np.full((T, 1), 40.0), np.full((T, 1), -80.0)], 1))  # sigmoid -> 1, softplus -> 0: g = 1
    st, o = zeros(gpu, D * Dv * 4), zeros(gpu, T * Dv * 4)
    xb, bb = dev(gpu, x).ptr.value, dev(gpu, ba).ptr.value
    gpu.check(gpu.cuda_lib().ggb_op_gated_delta(xb, xb + 4 * D, xb + 8 * D, 2 * D + Dv, bb, bb + 4, 2, T, H, G, D, Dv, dev(gpu, f32([0.0])).ptr,
                                                dev(gpu, f32([0.0])).ptr, st.ptr, o.ptr, Dv), "gated_delta")
    got = o.download(np.float32, T * Dv).reshape(T, Dv)
    S = st.download(np.float32, D * Dv).reshape(D, Dv)
    assert np.allclose(got[2], v[2] * D ** -0.5, atol=1e-5) and np.allclose(S[2], v[2], atol=1e-5) and np.allclose(S[5], v[1], atol=1e-5)


# ------------------------------------------------------------------------------------------------ window_attention.cu
def cos_sin(freqs, n_pos):
    a = np.arange(n_pos)[:, None] * freqs[None, :]
    return f32(np.stack([np.cos(a), np.sin(a)], -1))


def run_window(gpu, dt, q, k, v, H, G, window, scale, fk, fv, cuts, page, qn=None, kn=None, eps=1e-5, seed=0, scratch=True):
    """feeds q, k, v rows in portions through qkv_store + window_attn over shuffled pages; returns [T, H Dv]"""
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    lib = gpu.cuda_lib()
    ld = int(lib.ggb_window_cache_ld(G, D, Dv))
    n_pages = (T + page - 1) // page + 3
    table = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
    es = 2 if dt == BF16 else 4
    cache = zeros(gpu, n_pages * page * ld * es)
    tb = dev(gpu, table)
    ck = dev(gpu, cos_sin(fk, T + 1)) if fk is not None else None
    cv = dev(gpu, cos_sin(fv, T + 1)) if fv is not None else None
    rows = f32(np.concatenate([q, k, v], 1))
    ldr = rows.shape[1]
    ws = zeros(gpu, lib.ggb_window_attn_scratch_bytes(H)) if scratch else None  # with it short steps spread over several CTAs
    lo, got = 0, []
    for c in cuts:
        xr, qo, out = dev(gpu, rows[lo:lo + c]), zeros(gpu, c * H * D * 4), zeros(gpu, c * H * Dv * es)
        pos0 = dev(gpu, np.array([lo], dtype=np.int32))
        b = xr.ptr.value
        gpu.check(lib.ggb_op_window_qkv_store(dt, b, b + 4 * H * D, b + 4 * (H + G) * D, ldr, c, H, G, D, Dv, ptr(dev(gpu, f32(qn)) if qn is not None else None),
                                              ptr(dev(gpu, f32(kn)) if kn is not None else None), eps, 2 * len(fk) if fk is not None else 0, ptr(ck), ptr(cv),
                                              scale, pos0.ptr, tb.ptr, page, cache.ptr, qo.ptr), "window_qkv_store")
        gpu.check(lib.ggb_op_window_attn(dt, qo.ptr, cache.ptr, tb.ptr, page, pos0.ptr, c, H, G, D, Dv, window or 0, ptr(cv), out.ptr, ptr(ws)), "window_attn")
        got.append(from_dt(dt, out, (c, H * Dv)))
        lo += c
    assert lo == T
    return np.concatenate(got)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,Gk,D,Dv,window,page", [(4, 2, 8, 6, 11, 8), (3, 3, 16, 16, 64, 16), (6, 1, 6, 34, 5, 7), (2, 2, 64, 128, 33, 64),
                                                  (2, 1, 24, 10, None, 16)])
def test_window_attention_portions_and_single_tokens(gpu, dt, H, Gk, D, Dv, window, page):
    G = Gk
    r = np.random.default_rng(H * 100 + D)
    T = 150
    q, k, v = r.standard_normal((T, H * D)), r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
    fk, fv = BP.rot_freqs(40.0, D - 2 if D > 6 else D, 3.0), BP.rot_freqs(40.0, Dv)
    qn, kn = 1 + 0.2 * r.standard_normal(H * D), 1 + 0.2 * r.standard_normal(G * D)
    want = BP.window_core(BP.rms(q, 1e-5) * qn, BP.rms(k, 1e-5) * kn, v, H, G, window, 0.3, fk, fv)
    for cuts in ([T], [40] + [1] * 30 + [2, 3, 33, 42], [1] * 20 + [130]):
        got = run_window(gpu, dt, q, k, v, H, G, window, 0.3, fk, fv, cuts, page, qn, kn, scratch=len(cuts) != 21)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), cuts


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("steps", ["portion", "single"])
def test_window_edge_far_keys_and_page_borders_with_one_key_standing_out(gpu, dt, steps):
    """Query i points at key j: inside the window (or at its last place) the head returns j's value turned by j - i,
    one place outside nothing of it.  j walks over page borders, the first positions and far back."""
    H, G, D, Dv, page = 2, 1, 8, 6, 16
    T = 200
    r = np.random.default_rng(9)
    fk, fv = None, BP.rot_freqs(25.0, Dv)
    for window, i, j in ((32, 199, 168), (32, 199, 167), (17, 63, 47), (17, 64, 47), (17, 64, 48), (None, 199, 0), (None, 150, 15), (None, 150, 16),
                         (200, 199, 1), (5, 4, 0), (5, 5, 0), (1, 77, 77), (1, 77, 76)):
        q, k, v = 0.05 * r.standard_normal((T, H * D)), 0.05 * r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
        u = r.standard_normal(D); u /= np.linalg.norm(u)
        q[i, :D] = 30.0 * u      # head 0 of token i
        k[j] = 30.0 * u
        want = BP.window_core(q, k, v, H, G, window, 1.0, fk, fv)
        visible = j <= i and (window is None or i - j < window)
        turned = BP.rotate_pairs(v[j:j + 1], [j - i], fv)[0]
        assert (np.abs(want[i, :Dv] - turned).max() < 1e-6) == visible  # the oracle itself tells inside from outside
        cuts = [T] if steps == "portion" else [i - 3] + [1] * (T - i + 3) if i > 3 else [1] * T
        got = run_window(gpu, dt, q, k, v, H, G, window, 1.0, fk, fv, cuts, page, seed=i)
        assert np.abs(got[i] - want[i]).max() < (3e-2 if dt == BF16 else 1e-5), (window, i, j)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), (window, i, j)
