"""The quantised Gemma model through the architecture registry and the serving engine: a folder whose config.json names
a GGUF file is served by the same step function as the other architectures, with the logits of its batched prefill."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O
from gguf_fixture import write_gemma_gguf

pytestmark = pytest.mark.gpu
DIMS = dict(n_embd=256, n_layer=2, n_head=4, n_head_kv=1, head_dim=64, n_ff=1024, n_vocab=2048, n_ctx=96)


def test_gemma_folder_through_the_engine(gpu, tmp_path):
    om = O.Model(wtype=O.TYPE_Q8_0, sigma_embd=0.002, **DIMS)
    write_gemma_gguf(os.path.join(tmp_path, "tiny.gguf"), om, DIMS, O.TYPE_Q8_0)
    om.close()
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"architecture": "gemma", "gguf": "tiny.gguf", "n_ctx": 96}, f)
    assert "gemma" in gpu.architectures()
    prompt = ((1 + 7919 * np.arange(20)) % DIMS["n_vocab"]).astype(np.int32)
    m = gpu.GemmaModel.load_model_from_file(os.path.join(tmp_path, "tiny.gguf"))
    m.init_kv_cache()
    m.build_compute_graph()
    nxt = m.prefill(prompt, 0)
    want = np.stack([m.prefill_logits(i) for i in (3, 19)])
    m.close()
    eng = gpu.Engine(str(tmp_path), max_tokens=96)
    assert eng.architecture == "gemma" and eng.vocab == DIMS["n_vocab"]
    a = eng.step([("s", prompt[:12], [3])])
    b = eng.step([("s", prompt[12:], [7])])
    got = np.concatenate([a, b])
    # the portions 12 + 8 against the whole prompt: bf16 activations, same kernels, another tiling of the rows
    assert np.abs(got - want).max() < 3e-2 * np.abs(want).max()
    assert int(np.argmax(got[1])) == int(nxt)
    with pytest.raises(gpu.GgbError, match="slot"):  # the Gemma path holds one sequence
        eng.step([("t", prompt[:2], [])])
    eng.end("s")
    out = eng.generate("u", prompt, 3)
    assert int(out[0]) == int(nxt)
    eng.close()
