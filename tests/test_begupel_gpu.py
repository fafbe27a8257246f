"""Begupel through the serving engine against the plain numpy oracle (tests/begupel_plain.py): whole prompts and every
layer, portions down to two tokens, token-by-token decoding, several live sequences of unequal length, slots and pages
that are freed and used again (also by the same sequence, behind its windows), the first tokens of a sequence, long
decoding, other sizes and optional parts, and greedy generation through the engine's own entry point."""
import numpy as np
import pytest

import begupel_fixture as F
import begupel_plain as BP

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(gpu, tmp_path_factory):
    cfg = F.small_config()
    d, W = F.make_model(str(tmp_path_factory.mktemp("bg") / "m"), cfg, seed=11)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 150)
    return cfg, d, W, toks, BP.forward(toks, W, cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(gpu, small, dtype):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype=dtype, max_tokens=256, page_size=16)
    assert eng.architecture == "Begupel"
    eng.capture(True)
    got = eng.step([("a", toks, np.arange(len(toks)))], ["a"])
    assert F.close_enough(got, want, dtype)
    layers = []
    BP.forward(toks, W, cfg, layers)
    for i, x in enumerate(layers):
        assert F.close_enough(eng.captured(i, len(toks), cfg["width"]), x, dtype), i
    assert eng.stats()["live_seqs"] == 0 and eng.stats()["free_pages"] == eng.stats()["pages"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_equal_the_whole_prompt(gpu, small, dtype):
    cfg, d, W, toks, want = small
    for cuts, page, portion in (([1] * 40, 16, 0), ([2] * 20 + [3, 5, 2, 31, 17, 2, 1, 1, 48], 16, 0), ([150], 8, 7), ([63, 1, 1, 1, 64, 2, 18], 64, 32),
                                ([2, 1, 2, 4, 3, 33, 1, 1, 2, 60], 4, 0)):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=200, page_size=page, max_portion=portion)
        lo, rows = 0, []
        for c in cuts:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        got = np.concatenate(rows)
        assert F.close_enough(got, want[:lo], dtype), cuts[:3]
        eng.end("s")
        whole = eng.step([("w", toks[:lo], np.arange(lo))], ["w"])
        assert F.close_enough(got, whole, dtype), cuts[:3]
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_several_sequences_reused_slots_and_first_tokens(gpu, small, dtype):
    cfg, d, W, toks, want = small
    r = np.random.default_rng(8)
    seqs = {k: r.integers(0, cfg["vocab"], n) for k, n in (("a", 70), ("b", 9), ("c", 33), ("d", 50), ("e", 1), ("f", 3))}
    alone = {k: BP.forward(v, W, cfg) for k, v in seqs.items()}
    eng = gpu.Engine(d, dtype=dtype, max_tokens=140, page_size=8, max_seqs=3)
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}

    def feed(*items, end=()):
        entries = [(k, seqs[k][at[k]:at[k] + n], np.arange(n)) for k, n in items]
        out = eng.step(entries, end)
        lo = 0
        for k, n in items:
            got[k].append(out[lo:lo + n])
            lo += n
            at[k] += n
    feed(("a", 30), ("b", 2))
    feed(("c", 20), ("a", 1), ("b", 5))
    feed(("b", 2), ("a", 2), ("c", 13), end=["b", "c"])   # two slots and their pages come back
    free_mid = eng.stats()["free_pages"]
    feed(("d", 1), ("e", 1), end=["e"])                    # d and e start in slots that b and c used: state must be clean
    feed(("a", 37), ("d", 2), ("f", 3), end=["a", "f"])
    feed(("d", 47), end=["d"])
    for k in seqs:
        assert at[k] == len(seqs[k]) and F.close_enough(np.concatenate(got[k]), alone[k], dtype), k
    st = eng.stats()
    assert st["live_seqs"] == 0 and st["free_pages"] == st["pages"] and free_mid < st["pages"]
    with pytest.raises(gpu.GgbError):  # a fourth live sequence has no slot
        eng.step([(k, [1], []) for k in "wxyz"])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_behind_every_window_are_used_again_while_the_sequence_lives(gpu, small, dtype):
    cfg, d, W, toks, want = small   # windows of 11 and 5 positions
    other = toks[::-1].copy()
    want_other = BP.forward(other, W, cfg)
    # two prompts of 150 tokens live together in a cache sized for 150: only the rows inside the windows keep their pages
    eng = gpu.Engine(d, dtype=dtype, max_tokens=150, page_size=4, max_seqs=2)
    lo, rows, rows_o, seen = 0, [], [], set()
    cuts = [9, 1, 1, 7, 16, 2, 2, 1, 16, 13, 1, 1, 1, 16, 3, 16, 16, 12, 2, 14]
    for c in cuts:
        out = eng.step([("s", toks[lo:lo + c], np.arange(c)), ("o", other[lo:lo + c], np.arange(c))])
        rows.append(out[:c]); rows_o.append(out[c:])
        lo += c
        assert eng.seq_live_pages("s") <= 11 // 4 + 2 and eng.seq_live_pages("o") <= 11 // 4 + 2
        seen.update(int(p) for p in eng.seq_pages("s") if p >= 0)
    assert lo == 150 and F.close_enough(np.concatenate(rows), want, dtype) and F.close_enough(np.concatenate(rows_o), want_other, dtype)
    assert len(eng.seq_pages("s")) == (150 + 3) // 4 and (eng.seq_pages("s") >= 0).sum() == eng.seq_live_pages("s")
    with pytest.raises(gpu.GgbError, match="positions"):  # trimming frees pages, not positions
        eng.step([("s", toks[:20], [])])
    eng.end("s", "o")
    assert eng.stats()["free_pages"] == eng.stats()["pages"]
    # without a bound on every window nothing is trimmed and the same cache runs out, loudly
    cfg2 = F.config([F.parallel(F.left(window=0))])
    d2, _ = F.make_model(d + "_unbounded", cfg2, seed=1)
    eng2 = gpu.Engine(d2, dtype=dtype, max_tokens=16, page_size=4, max_seqs=2)
    eng2.step([("s", toks[:20], [19])])
    assert eng2.seq_live_pages("s") == 5
    with pytest.raises(gpu.GgbError, match="out of pages"):
        eng2.step([("t", toks[:8], [])])
    eng.close(); eng2.close()


def test_long_decoding(gpu, small):
    cfg, d, W, toks, _ = small
    long = np.random.default_rng(2).integers(0, cfg["vocab"], 330)
    want = BP.forward(long, W, cfg)
    for dtype in ("float32", "bfloat16"):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=400, page_size=32)
        rows = [eng.step([("s", long[:10], np.arange(10))])] + [eng.step([("s", long[i:i + 1], [0])]) for i in range(10, 330)]
        assert F.close_enough(np.concatenate(rows), want, dtype)
        eng.close()


OTHER = {
    # what the small configuration has unequal, equal; what it has, absent
    "equal_and_absent": lambda: F.config([F.parallel(F.left(heads=2, kv_heads=2, dim=8, vdim=8, window=0, dims=None, factor=None), F.right(heads=2, kv_heads=2, dim=6, vdim=6, conv=1), mlp=None),
                                          F.lightning(heads=1, dim=8, vdim=8, decay=[1.0])], vocab=17, width=16, groups=1, taps=0, buckets=0, softcap=0),
    "one_key_head": lambda: F.config([F.parallel(F.left(heads=6, kv_heads=1, dim=10, vdim=4, window=1, base=0), F.right(heads=3, kv_heads=1, dim=9, vdim=11, conv=8), mlp=7)],
                                     vocab=30, width=22, groups=2, taps=8, buckets=1),
    "only_lightning": lambda: F.config([F.lightning(heads=2, dim=6, vdim=12), F.lightning(heads=4, dim=5, vdim=3, mlp=11)], vocab=19, width=20, groups=5, taps=3, buckets=3),
    "only_parallel": lambda: F.config([F.parallel(mlp=None), F.parallel(F.left(heads=1, kv_heads=1, dim=4, vdim=2, window=200, dims=2), F.right(heads=1, kv_heads=1, dim=3, vdim=1, conv=5))],
                                      vocab=64, width=12, groups=2, taps=2),
    "wide": lambda: F.config([F.lightning(heads=2, dim=64, vdim=32, mlp=96), F.parallel(F.left(heads=4, kv_heads=2, dim=32, vdim=64, window=70, dims=16, factor=None),
                                                                                         F.right(heads=4, kv_heads=2, dim=128, vdim=48, conv=4), mlp=160),
                              F.parallel(F.left(heads=2, kv_heads=1, dim=64, vdim=34, window=9), F.right(heads=1, kv_heads=1, dim=20, vdim=70, conv=2), mlp=None)],
                             vocab=200, width=128, groups=4, taps=2, buckets=251),
}


@pytest.mark.parametrize("name", sorted(OTHER))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes_and_optional_parts(gpu, tmp_path, name, dtype):
    cfg = OTHER[name]()
    d, W = F.make_model(str(tmp_path / name), cfg, seed=3)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], 140)
    want = BP.forward(toks, W, cfg)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=300, page_size=16)
    whole = eng.step([("w", toks, np.arange(140))], ["w"])
    assert F.close_enough(whole, want, dtype)
    lo, rows = 0, []
    for c in [2, 2, 65, 1, 1, 3, 64, 2]:
        rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
        lo += c
    assert F.close_enough(np.concatenate(rows), want, dtype)
    eng.close()


def test_random_weight_engine_portions_agree_at_sizes_that_reach_the_tensor_cores(gpu):
    cfg = F.config([F.lightning(heads=4, dim=64, vdim=64, mlp=512), F.parallel(F.left(heads=8, kv_heads=2, dim=64, vdim=64, window=100, dims=None),
                                                                                 F.right(heads=4, kv_heads=2, dim=64, vdim=64, conv=4), mlp=512)],
                   vocab=512, width=256, groups=2, buckets=509)
    toks = np.random.default_rng(0).integers(0, 512, 400)
    for dtype in ("bfloat16", "float32"):
        eng = gpu.Engine(config=cfg, seed=7, dtype=dtype, max_tokens=1024)
        whole = eng.step([("w", toks, np.arange(400))], ["w"])
        lo, rows = 0, []
        for c in [130, 2, 1, 1, 64, 200, 2]:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        assert np.isfinite(whole).all() and F.close_enough(np.concatenate(rows), whole, dtype, loose=2.0)
        eng.close()


def test_greedy_generation_through_the_engine(gpu, small):
    cfg, d, W, toks, _ = small
    eng = gpu.Engine(d, dtype="float32", max_tokens=128)
    prompt = toks[:12]
    out = eng.generate("g", prompt, 25)
    assert len(out) == 25 and eng.seq_len("g") == 12 + 24
    z = BP.forward(np.concatenate([prompt, out]), W, cfg)
    for i, t in enumerate(out):  # every chosen token is the oracle's maximum at its place (up to rounding between near-equal logits)
        row = z[len(prompt) - 1 + i]
        assert row[t] >= row.max() - 1e-4, i
    eng.end("g")
    assert eng.stats()["live_seqs"] == 0
    eng.close()
