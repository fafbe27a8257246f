"""The kernels Begupel added, alone and twice each, on a small case (for one `ncu` capture): gated delta rule and lightning
attention over 1024 tokens (16 heads of 128 x 128), window attention of a 1024-token portion and of a one-token step
(window 1024) over a bf16 cache."""
import sys, numpy as np
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import gemma_ggml_b200 as G
G.init(0)
L = G.cuda_lib()
r = np.random.default_rng(0)
BF16 = 30
def dev(a): return G.DeviceBuffer.from_numpy(np.ascontiguousarray(a))
T, H, Gk, D, Dv = 1024, 16, 8, 128, 128
ld = 2 * Gk * D + H * Dv
x = dev((r.standard_normal((T, ld)) * 0.5).astype(np.float32))
ba = dev(r.standard_normal((T, 2 * H)).astype(np.float32))
A = dev(r.uniform(-2, 0, H).astype(np.float32)); dtb = dev(r.uniform(-1, 1, H).astype(np.float32))
st = G.DeviceBuffer(H * D * Dv * 4); st.zero()
o = G.DeviceBuffer(T * H * Dv * 4)
xb, bb = x.ptr.value, ba.ptr.value
for _ in range(2):
    G.check(L.ggb_op_gated_delta(xb, xb + 4 * Gk * D, xb + 8 * Gk * D, ld, bb, bb + 4 * H, 2 * H, T, H, Gk, D, Dv, A.ptr, dtb.ptr, st.ptr, o.ptr, H * Dv), "delta")
ldl = 2 * H * D + H * Dv
xl = dev((r.standard_normal((T, ldl)) * 0.5).astype(np.float32))
dec = dev(r.uniform(0.6, 0.999, H).astype(np.float32))
lb = xl.ptr.value
for _ in range(2):
    G.check(L.ggb_op_lightning_attn(lb, lb + 4 * H * D, lb + 8 * H * D, ldl, T, H, D, Dv, dec.ptr, st.ptr, o.ptr, H * Dv), "lightning")
# window attention: a cache of 2048 positions, a portion of 1024 tokens at position 1024, then a step of one token
Gw, page, window = 4, 64, 1024
cld = int(L.ggb_window_cache_ld(Gw, D, Dv)); n_pos = 2048 + 64
cache = G.DeviceBuffer(n_pos * cld * 2); cache.upload((r.standard_normal(n_pos * cld).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16))
table = dev(np.arange(n_pos // page, dtype=np.int32))
a = np.arange(n_pos)[:, None] * (10000.0 ** (-2.0 * np.arange(Dv // 2) / Dv))[None, :]
cs = dev(np.stack([np.cos(a), np.sin(a)], -1).astype(np.float32))
q = dev((r.standard_normal((T, H * D)) * 0.1).astype(np.float32))
out = G.DeviceBuffer(T * H * Dv * 2)
ws = G.DeviceBuffer(int(L.ggb_window_attn_scratch_bytes(H)))
pos_p, pos_s = dev(np.array([1024], dtype=np.int32)), dev(np.array([2047], dtype=np.int32))
for _ in range(2):
    G.check(L.ggb_op_window_attn(BF16, q.ptr, cache.ptr, table.ptr, page, pos_p.ptr, T, H, Gw, D, Dv, window, cs.ptr, out.ptr, ws.ptr), "attn portion")
for _ in range(2):
    G.check(L.ggb_op_window_attn(BF16, q.ptr, cache.ptr, table.ptr, page, pos_s.ptr, 1, H, Gw, D, Dv, window, cs.ptr, out.ptr, ws.ptr), "attn step")
G.sync()
print("ok")
