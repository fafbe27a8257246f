"""The bf16 / fp32 operators of csrc/dense.cu, latent_attention.cu and moe.cu, each alone against numpy float64 on the
same (rounded) operands.  Inputs are built so that a fault shows: one key made to stand out at page borders, at the
first positions, far back and one past the causal edge; a sink that takes most of the weight; ties in the router."""
import ctypes as C

import numpy as np
import pytest

import safolorn_fixture as F

pytestmark = pytest.mark.gpu
BF16, F32 = 30, 0


_ALIVE = []


@pytest.fixture(autouse=True)
def _release_buffers():
    yield
    _ALIVE.clear()


def dev(G, a):
    """an uploaded copy that stays allocated until the test ends (launches are asynchronous)"""
    _ALIVE.append(G.DeviceBuffer.from_numpy(np.ascontiguousarray(a)))
    return _ALIVE[-1]


def as_dt(dt, a):
    """values representable in dt (float64) and the array to upload"""
    if dt == BF16:
        v, codes = F.bf16_round(a)
        return v, codes
    a32 = np.asarray(a, dtype=np.float32)
    return a32.astype(np.float64), a32


def from_dt(dt, buf, shape):
    n = int(np.prod(shape))
    if dt == BF16:
        return (buf.download(np.uint16, n).astype(np.uint32) << 16).view(np.float32).reshape(shape).astype(np.float64)
    return buf.download(np.float32, n).reshape(shape).astype(np.float64)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("T,N,K", [(1, 37, 50), (2, 64, 128), (8, 33, 72), (9, 70, 45), (130, 96, 64), (64, 65, 200), (5, 3, 7),
                                   (300, 544, 192), (64, 32, 64), (257, 1024, 512), (1100, 96, 1024)])
def test_linear_any_shape(gpu, dt, T, N, K):
    r = np.random.default_rng(T * 1000 + N)
    wv, wu = as_dt(dt, r.standard_normal((N, K)))
    av, au = as_dt(dt, r.standard_normal((T, K)))
    w, a, c = dev(gpu, wu), dev(gpu, au), gpu.DeviceBuffer(T * (N + 3) * 4)
    gpu.check(gpu.cuda_lib().ggb_op_linear(dt, w.ptr, N, K, a.ptr, K, T, c.ptr, N + 3), "linear")
    got = c.download(np.float32).reshape(T, N + 3)[:, :N]
    assert F.rel_err(got, av @ wv.T) < 2e-6


@pytest.mark.parametrize("dt", [F32, BF16])
def test_rms_norm_one_number_and_vector(gpu, dt):
    r = np.random.default_rng(0)
    T, E, eps = 5, 77, 1e-3
    x = r.standard_normal((T, E)).astype(np.float32)
    g1, g2 = np.array([1.7], dtype=np.float32), (1 + 0.1 * r.standard_normal(E)).astype(np.float32)
    es = 2 if dt == BF16 else 4
    y1, y2 = gpu.DeviceBuffer(T * E * es), gpu.DeviceBuffer(T * E * es)
    gpu.check(gpu.cuda_lib().ggb_op_rms_norm2(dt, dev(gpu, x).ptr, E, dev(gpu, g1).ptr, 0, dev(gpu, g2).ptr, 1, eps, E, T, y1.ptr, y2.ptr), "norm")
    xn = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps)
    tol = 5e-3 if dt == BF16 else 1e-6
    assert F.rel_err(from_dt(dt, y1, (T, E)), xn * 1.7) < tol and F.rel_err(from_dt(dt, y2, (T, E)), xn * g2) < tol


@pytest.mark.parametrize("dt", [F32, BF16])
def test_glu_clamp_and_residual_side(gpu, dt):
    r = np.random.default_rng(1)
    T, Fd, W, sd, V, L = 4, 19, 40, 5, 11, 3
    gu = (2 * r.standard_normal((T, 2 * Fd))).astype(np.float32)
    es = 2 if dt == BF16 else 4
    y = gpu.DeviceBuffer(T * Fd * es)
    gpu.check(gpu.cuda_lib().ggb_op_glu_clamp(dt, dev(gpu, gu).ptr, Fd, T, 1.5, 1.702, y.ptr), "glu")
    g, u = np.minimum(gu[:, :Fd].astype(np.float64), 1.5), np.clip(gu[:, Fd:].astype(np.float64), -1.5, 1.5)
    assert F.rel_err(from_dt(dt, y, (T, Fd)), g / (1 + np.exp(-1.702 * g)) * (u + 1)) < (5e-3 if dt == BF16 else 1e-6)
    assert (gu[:, :Fd] > 1.5).any() and (gu[:, Fd:] < -1.5).any()
    x, a, f = (r.standard_normal((T, W)).astype(np.float32) for _ in range(3))
    ids = np.array([3, 0, 10, 3], dtype=np.int32)
    sev, seu = as_dt(dt, r.standard_normal((V, L * sd)))
    wgv, wgu = as_dt(dt, r.standard_normal((sd, W)) / 6)
    wpv, wpu = as_dt(dt, r.standard_normal((W, sd)))
    nw = (0.3 * (1 + 0.1 * r.standard_normal(W))).astype(np.float32)
    for with_f in (True, False):
        for li in (0, 2):
            xb = dev(gpu, x)
            gpu.check(gpu.cuda_lib().ggb_op_residual_side(dt, xb.ptr, dev(gpu, a).ptr, dev(gpu, f).ptr if with_f else None, W, T, dev(gpu, ids).ptr,
                                                          dev(gpu, seu).ptr, L * sd, li * sd, sd, dev(gpu, wgu).ptr, dev(gpu, wpu).ptr,
                                                          dev(gpu, nw).ptr, 1e-5), "residual_side")
            x1 = x.astype(np.float64) + a + (f if with_f else 0)
            z = x1 @ wgv.T
            gg = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))) * sev[ids][:, li * sd:(li + 1) * sd]
            yy = gg @ wpv.T
            want = x1 + yy / np.sqrt((yy ** 2).mean(-1, keepdims=True) + 1e-5) * nw
            assert F.rel_err(xb.download(np.float32).reshape(T, W), want) < 2e-6
    xb = dev(gpu, x)  # no side input: the residual sum alone
    gpu.check(gpu.cuda_lib().ggb_op_residual_side(dt, xb.ptr, dev(gpu, a).ptr, None, W, T, None, None, 0, 0, 0, None, None, None, 1e-5), "residual")
    assert F.rel_err(xb.download(np.float32).reshape(T, W), x.astype(np.float64) + a) < 1e-7


def attention_reference(qa, rows, R, pos0, sink, wuv, Dv):
    """qa [T, H, R + Dr] (scaled), rows [n, R + Dr] by position: soft-max with sink over j <= pos0 + t, values c_j, then W_uv."""
    T, H, _ = qa.shape
    out = np.zeros((T, H * Dv))
    for t in range(T):
        n = pos0 + t + 1
        for h in range(H):
            s = rows[:n] @ qa[t, h]
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            o = (e[:, None] * rows[:n, :R]).sum(0) / (e.sum() + np.exp(sink[h] - m))
            out[t, h * Dv:(h + 1) * Dv] = wuv[h * Dv:(h + 1) * Dv] @ o
    return out


def run_attention(gpu, dt, qa, rows, R, Dr, pos0, sink, wuv_u, Dv, page, n_split, seed=0):
    """rows by position are scattered over shuffled pages; returns out [T, H * Dv] as float64"""
    T, H, _ = qa.shape
    n = rows.shape[0]
    ld = int(gpu.cuda_lib().ggb_latent_cache_ld(R, Dr))
    n_pages = (n + page - 1) // page
    table = np.random.default_rng(seed).permutation(n_pages + 3)[:n_pages].astype(np.int32)
    _, ru = as_dt(dt, rows)
    cache = np.zeros(((n_pages + 3) * page, ld), dtype=ru.dtype)
    for j in range(n):
        cache[table[j // page] * page + j % page, :R + Dr] = ru[j]
    part = gpu.DeviceBuffer(int(gpu.cuda_lib().ggb_latent_attn_scratch_bytes(T, H, R, n_split)))
    es = 2 if dt == BF16 else 4
    out = gpu.DeviceBuffer(T * H * Dv * es)
    L = gpu.cuda_lib()
    p0 = dev(gpu, np.array([pos0], dtype=np.int32))
    gpu.check(L.ggb_op_latent_attn(dt, dev(gpu, qa.astype(np.float32)).ptr, dev(gpu, cache).ptr, dev(gpu, table).ptr, page, p0.ptr, T, H, R, Dr,
                                   n_split, part.ptr), "latent_attn")
    gpu.check(L.ggb_op_latent_attn_out(dt, part.ptr, n_split, dev(gpu, sink.astype(np.float32)).ptr, dev(gpu, wuv_u).ptr, T, H, R, Dv, out.ptr),
              "latent_attn_out")
    return from_dt(dt, out, (T, H * Dv))


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,R,Dr,Dv", [(3, 12, 4, 6), (20, 40, 6, 5), (2, 70, 0, 9), (1, 33, 8, 2)])
def test_latent_attention_random(gpu, dt, H, R, Dr, Dv):
    r = np.random.default_rng(H)
    pos0, T, page = (37, 9, 8) if H != 3 else (70, 67, 8)  # 67 tokens: the form that takes two tokens per CTA
    n = pos0 + T
    rows_v, _ = as_dt(dt, r.standard_normal((n, R + Dr)))
    qa = (r.standard_normal((T, H, R + Dr)) * 0.4).astype(np.float32)
    sink = r.standard_normal(H)
    wv, wu = as_dt(dt, r.standard_normal((H * Dv, R)))
    want = attention_reference(qa.astype(np.float64), rows_v, R, pos0, sink, wv, Dv)
    for ns in (1, 3, 7):
        got = run_attention(gpu, dt, qa, rows_v, R, Dr, pos0, sink, wu, Dv, page, ns)
        assert F.rel_err(got, want) < (6e-3 if dt == BF16 else 3e-6), (ns,)


@pytest.mark.parametrize("dt", [F32, BF16])
def test_latent_attention_one_key_stands_out(gpu, dt):
    """A key whose score dwarfs the rest takes the whole weight: the output must be its value when it is visible (page
    borders, first positions, hundreds back, the token itself) and must not change when it lies one past the causal edge."""
    r = np.random.default_rng(7)
    H, R, Dr, Dv, page = 2, 16, 4, 3, 16
    wv, wu = as_dt(dt, r.standard_normal((H * Dv, R)))
    sink = np.array([-3.0, 0.5])
    direction = r.standard_normal(R + Dr)
    direction /= np.linalg.norm(direction)
    for pos0, T in ((420, 1), (400, 21), (0, 40), (30, 65)):
        n = pos0 + T
        for j_star in sorted({0, 1, page - 1, page, page + 1, n - 1, max(n - 300, 2), pos0, min(pos0 + 1, n - 1)}):
            rows = 0.05 * r.standard_normal((n, R + Dr))
            rows[j_star] = 4.0 * direction + 0.05 * r.standard_normal(R + Dr)
            rows_v, _ = as_dt(dt, rows)
            qa = np.tile(8.0 * direction, (T, H, 1)).astype(np.float32)  # score of the needle ~ 32, of the others ~ 0
            want = attention_reference(qa.astype(np.float64), rows_v, R, pos0, sink, wv, Dv)
            for ns in (1, 5):
                got = run_attention(gpu, dt, qa, rows_v, R, Dr, pos0, sink, wu, Dv, page, ns, seed=j_star)
                assert F.rel_err(got, want) < (8e-3 if dt == BF16 else 5e-6), (pos0, T, j_star, ns)
            # the rows of tokens that cannot see the needle differ from those that can: the test has teeth
            if T > 1 and pos0 < j_star < n - 1:
                t_edge = j_star - pos0
                assert np.abs(want[t_edge] - want[t_edge - 1]).max() > 0.1


@pytest.mark.parametrize("dt", [F32, BF16])
def test_latent_attention_sink_takes_the_weight(gpu, dt):
    r = np.random.default_rng(9)
    H, R, Dr, Dv = 3, 8, 2, 4
    rows_v, _ = as_dt(dt, r.standard_normal((5, R + Dr)))
    qa = (0.1 * r.standard_normal((2, H, R + Dr))).astype(np.float32)
    wv, wu = as_dt(dt, r.standard_normal((H * Dv, R)))
    sink = np.array([6.0, -40.0, 0.0])
    want = attention_reference(qa.astype(np.float64), rows_v, R, 3, sink, wv, Dv)
    got = run_attention(gpu, dt, qa, rows_v, R, Dr, 3, sink, wu, Dv, 4, 2)
    assert F.rel_err(got, want) < (8e-3 if dt == BF16 else 3e-6)
    assert np.abs(want[:, :Dv]).max() < 0.05 * np.abs(want[:, Dv:2 * Dv]).max()  # head 0 is almost all sink


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("T,E,top,Fe,W", [(1, 5, 2, 24, 40), (37, 12, 3, 20, 33), (200, 4, 1, 70, 48), (9, 3, 3, 8, 16), (4, 6, 3, 16, 32), (2, 7, 2, 9, 13),
                                          (300, 4, 2, 64, 128), (700, 6, 1, 96, 192), (1500, 3, 2, 128, 64)])
def test_mixture_of_experts(gpu, dt, T, E, top, Fe, W):
    r = np.random.default_rng(T + E)
    L = gpu.cuda_lib()
    hv, hu = as_dt(dt, r.standard_normal((T, W)))
    wr = (r.standard_normal((E, W)) / 3).astype(np.float32)
    if T > 1:
        wr[1] = wr[0]  # a tie between experts 0 and 1 for every token: the lower index goes first
    b = (0.3 * r.standard_normal(E)).astype(np.float32)
    if T > 1:
        b[1] = b[0]
    upv, upu = as_dt(dt, r.standard_normal((E, Fe, W)) / np.sqrt(W))
    dnv, dnu = as_dt(dt, r.standard_normal((E, W, Fe)) / np.sqrt(Fe))
    idx, wt = gpu.DeviceBuffer(T * top * 4), gpu.DeviceBuffer(T * top * 4)
    ws = gpu.DeviceBuffer(int(L.ggb_moe_group_ints(T * top, E)) * 4)
    es = 2 if dt == BF16 else 4
    y1, y2, out = gpu.DeviceBuffer(T * top * Fe * es), gpu.DeviceBuffer(T * top * W * 4), gpu.DeviceBuffer(T * W * 4)
    hb = dev(gpu, hu)
    zb = gpu.DeviceBuffer(T * E * 4)
    gpu.check(L.ggb_op_moe_route(dt, hb.ptr, W, T, dev(gpu, wr).ptr, dev(gpu, b).ptr, E, top, zb.ptr, idx.ptr, wt.ptr), "route")
    gpu.check(L.ggb_op_moe_group(idx.ptr, T, top, E, ws.ptr), "group")
    gpu.check(L.ggb_op_moe_linear(dt, dev(gpu, upu).ptr, Fe, W, hb.ptr, W, 1, T, top, E, ws.ptr, 1, y1.ptr, Fe), "up")
    gpu.check(L.ggb_op_moe_linear(dt, dev(gpu, dnu).ptr, W, Fe, y1.ptr, Fe, 0, T, top, E, ws.ptr, 0, y2.ptr, W), "down")
    gpu.check(L.ggb_op_moe_combine(y2.ptr, ws.ptr, wt.ptr, T, top, E, W, out.ptr), "combine")
    z = hv @ wr.astype(np.float64).T + b
    gi = idx.download(np.int32).reshape(T, top)
    want_i = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    margin = np.sort(z, axis=-1)[:, ::-1]
    safe = np.ones(T, dtype=bool) if top == E else (margin[:, top - 1] - margin[:, top] > 1e-4) | (margin[:, top - 1] == margin[:, top])
    assert (np.sort(gi[safe], axis=-1) == np.sort(want_i[safe], axis=-1)).all()
    for t in range(T):  # the tie: expert 0 is taken before expert 1
        g = list(gi[t])
        assert len(set(g)) == top and (1 not in g or T == 1 or (0 in g and g.index(0) < g.index(1)))
    want = np.zeros((T, W))
    for t in range(T):
        zs = z[t, gi[t]]
        p = np.exp(zs - zs.max())
        p /= p.sum()
        for k, e in enumerate(gi[t]):
            a = np.maximum(hv[t] @ upv[e].T, 0) ** 2
            if dt == BF16:
                a = F.bf16_round(a)[0]
            want[t] += p[k] * (a @ dnv[e].T)
    assert F.rel_err(out.download(np.float32).reshape(T, W), want) < (2e-3 if dt == BF16 else 3e-6)
