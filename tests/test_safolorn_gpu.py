"""Safolorn through the serving engine against the plain numpy oracle (tests/safolorn_plain.py): whole prompts, portions
down to two tokens, token-by-token decoding, several live sequences, pages that are freed and used again, long decoding,
other sizes, and greedy generation through the engine's own entry point."""
import numpy as np
import pytest

import safolorn_fixture as F
import safolorn_plain as SP

pytestmark = pytest.mark.gpu


def plain_logits(cfg, W, toks):
    return SP.Plain(cfg, W).forward(toks)


@pytest.fixture(scope="module")
def small(gpu, tmp_path_factory):
    cfg = F.small_config()
    d, W = F.make_model(str(tmp_path_factory.mktemp("sf") / "m"), cfg, seed=11)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 150)
    return cfg, d, W, toks, plain_logits(cfg, W, toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(gpu, small, dtype):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype=dtype, max_tokens=256, page_size=16)
    eng.capture(True)
    got = eng.step([("a", toks, np.arange(len(toks)))], ["a"])
    assert F.close_enough(got, want, dtype)
    layers = []
    SP.Plain(cfg, W).forward(toks, layers)
    for i, x in enumerate(layers):
        assert F.close_enough(eng.captured(i, len(toks), cfg["width"]), x, dtype), i
    assert eng.stats()["live_seqs"] == 0 and eng.stats()["free_pages"] == eng.stats()["pages"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_equal_the_whole_prompt(gpu, small, dtype):
    cfg, d, W, toks, want = small
    for cuts, page, portion in (([1] * 40, 16, 0), ([2] * 20 + [3, 5, 2, 31, 17, 2, 1, 1, 48], 16, 0), ([150], 8, 7), ([63, 1, 1, 1, 64, 2, 18], 64, 32)):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=200, page_size=page, max_portion=portion)
        lo, rows = 0, []
        for c in cuts:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        got = np.concatenate(rows)
        # against the oracle, and (tighter) against the engine's own whole-prompt run
        assert F.close_enough(got, want[:lo], dtype), cuts[:3]
        eng.end("s")
        whole = eng.step([("w", toks[:lo], np.arange(lo))], ["w"])
        assert F.close_enough(got, whole, dtype), cuts[:3]
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_several_sequences_and_reused_pages(gpu, small, dtype):
    cfg, d, W, toks, want = small
    r = np.random.default_rng(8)
    seqs = {k: r.integers(0, cfg["vocab"], n) for k, n in (("a", 70), ("b", 9), ("c", 33), ("d", 50))}
    alone = {k: plain_logits(cfg, W, v) for k, v in seqs.items()}
    eng = gpu.Engine(d, dtype=dtype, max_tokens=130, page_size=8, max_seqs=3)
    # a, b and c live together and advance in unequal portions, two and three to a step
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}

    def feed(*items, end=()):
        entries = []
        for k, n in items:
            entries.append((k, seqs[k][at[k]:at[k] + n], np.arange(n)))
        out = eng.step(entries, end)
        lo = 0
        for k, n in items:
            got[k].append(out[lo:lo + n])
            lo += n
            at[k] += n
    feed(("a", 30), ("b", 2))
    feed(("c", 20), ("a", 1), ("b", 5))
    pages_bc = set(eng.seq_pages("b").tolist()) | set(eng.seq_pages("c").tolist())
    feed(("b", 2), ("c", 13), end=["b", "c"])
    pages_a = set(eng.seq_pages("a").tolist())
    # d takes pages that b and c gave back, while a is still live and keeps its own
    feed(("d", 50), ("a", 39), end=["a"])
    pages_d = set(eng.seq_pages("d").tolist())
    assert len(pages_d) == 7 and not (pages_a & pages_d) and (pages_bc & pages_d)
    assert eng.stats()["live_seqs"] == 1 and eng.stats()["free_pages"] == eng.stats()["pages"] - 7
    eng.end("d")
    assert eng.stats()["free_pages"] == eng.stats()["pages"]
    for k in seqs:
        assert F.close_enough(np.concatenate(got[k]), alone[k], dtype), k
    # a new sequence on pages that others have used before: nothing of them is left
    again = eng.step([("e", seqs["a"], np.arange(70))], ["e"])
    assert F.close_enough(again, alone["a"], dtype)
    eng.close()


def test_cache_runs_out_loudly(gpu, small):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype="float32", max_tokens=16, page_size=8, max_seqs=1)
    eng.step([("a", toks[:24], [23])])  # one page of slack per sequence slot
    with pytest.raises(gpu.GgbError, match="out of pages"):
        eng.step([("a", toks[24:30], [0])])
    with pytest.raises(gpu.GgbError, match="slot"):
        eng.step([("b", toks[:2], [0])])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(gpu, small, dtype):
    cfg, d, W, toks, want = small
    r = np.random.default_rng(3)
    long = r.integers(0, cfg["vocab"], 420)
    ref = plain_logits(cfg, W, long)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=448, page_size=32)
    eng.step([("s", long[:100], [])])
    rows = [eng.step([("s", long[i:i + 1], [0])])[0] for i in range(100, 420)]
    assert F.close_enough(np.stack(rows), ref[100:], dtype)
    eng.close()


CONFIGS = {
    "one_head_no_side": lambda: F.config([F.layer(F.mixer(heads=1, dim=5, rot_dim=2, vdim=1, kv_rank=3), F.dense(ff=9))], vocab=17, width=20, side=0),
    "many_heads": lambda: F.config([F.layer(F.mixer(heads=19, dim=4, rot_dim=2, vdim=3, kv_rank=35, scale=0.7), F.moe(ff=10, experts=3, top=3)),
                                    F.layer(F.mixer(heads=19, dim=2, rot_dim=2, vdim=2, kv_rank=35, scale=0.7, kv_from=0), None)], vocab=40, width=36, side=1),
    "wide_latent": lambda: F.config([F.layer(F.mixer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=136, dims=4, base=5.0), F.dense(ff=70, limit=3.0)),
                                     F.layer(F.mixer(heads=4, dim=8, rot_dim=10, vdim=4, kv_rank=64, scaling=False, base=1e4), F.moe(ff=33, experts=9, top=4))],
                                    vocab=130, width=72, side=12, eps=1e-3),
    "no_rotation": lambda: F.config([F.layer(F.mixer(heads=3, rot_dim=0, dims=0, scaling=False), F.dense())], vocab=23, width=24, side=3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_other_sizes(gpu, tmp_path, name, dtype):
    cfg = CONFIGS[name]()
    d, W = F.make_model(str(tmp_path / "m"), cfg, seed=len(name))
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 75)
    want = plain_logits(cfg, W, toks)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=96, page_size=4)
    a = eng.step([("a", toks[:50], np.arange(50))])
    b = eng.step([("a", toks[50:52], [0, 1])])
    c = np.concatenate([eng.step([("a", toks[i:i + 1], [0])]) for i in range(52, 75)])
    assert F.close_enough(np.concatenate([a, b, c]), want, dtype)
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_reach_the_tensor_core_products(gpu, tmp_path, dtype):
    """Width, feed-forward and latent sizes in multiples of 64 and a portion of several hundred tokens: in bfloat16 the
    products run as tcgen05 GEMMs (plain and grouped by expert), the attention takes two tokens per CTA; then portions
    that fall back to the tile kernel and the mat-vec, all against the oracle."""
    cfg = F.config([F.layer(F.mixer(heads=5, dim=24, rot_dim=16, vdim=40, kv_rank=96, scale=0.15), F.moe(ff=64, experts=6, top=2)),
                    F.layer(F.mixer(heads=3, dim=32, rot_dim=16, vdim=64, kv_rank=96, scale=0.15, kv_from=0), F.dense(ff=320, limit=1.5)),
                    F.layer(F.mixer(heads=4, dim=16, rot_dim=32, vdim=16, kv_rank=64, scaling=False), F.moe(ff=128, experts=3, top=1))],
                   vocab=160, width=192, side=24)
    d, W = F.make_model(str(tmp_path / "m"), cfg, seed=21)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], 460)
    want = plain_logits(cfg, W, toks)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=512, page_size=64)
    a = eng.step([("a", toks[:330], np.arange(330))])
    b = eng.step([("a", toks[330:400], np.arange(70))])
    c = eng.step([("a", toks[400:437], np.arange(37))])
    e = np.concatenate([eng.step([("a", toks[i:i + 1], [0])]) for i in range(437, 460)])
    assert F.close_enough(np.concatenate([a, b, c, e]), want, dtype)
    eng.close()


def test_random_weight_engine_and_registry(gpu):
    cfg = F.small_config()
    eng = gpu.Engine(config=cfg, seed=4, dtype="bfloat16", max_tokens=64)
    assert eng.architecture == "Safolorn" and eng.vocab == cfg["vocab"]
    out = eng.step([("x", [1, 2, 3], [2])], ["x"])
    assert out.shape == (1, cfg["vocab"]) and np.isfinite(out).all() and out.std() > 0
    eng.close()
    bad = dict(cfg, architecture="Nothing")
    with pytest.raises(gpu.GgbError, match="not registered"):
        gpu.Engine(config=bad, seed=1)


def test_greedy_generation_through_the_engine(gpu, small):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype="float32", max_tokens=128, page_size=16)
    prompt = toks[:21]
    out = eng.generate("g", prompt, 30)
    m = SP.Plain(cfg, W)
    lg = m.forward(prompt)[-1]
    for i, tok in enumerate(out):
        top2 = np.sort(lg)[-2:]
        if top2[1] - top2[0] < 1e-3:  # a close call between two tokens proves nothing either way
            break
        assert int(np.argmax(lg)) == int(tok), i
        lg = m.forward([int(tok)])[-1]
    assert i >= 10
    assert eng.seq_len("g") == 21 + 29  # the last sampled token has not been fed yet
    eng.end("g")
    eng.close()
