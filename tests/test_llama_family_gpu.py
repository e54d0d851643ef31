"""The LLaMA engine opened through the registry (config.json "architecture": "llama"): the same step function,
scheduler and sampling entry points as the other families, checked against the engine driven directly."""
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPE = dict(num_layers=2, head_num=4, kv_head_num=2, head_size=128, inter_size=512, vocab_size=1000)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    d = tmp_path_factory.mktemp("llama")
    cfg = dict(architecture="llama", max_seq_len=512, rms_eps=1e-5, rotary_base=10000.0, random_init=dict(seed=5, std=0.05), **SHAPE)
    (d / "config.json").write_text(json.dumps(cfg))
    return str(d)


def rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def test_registry_serves_llama_like_the_engine(pkg, folder):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    S, E, capi = pkg.serve, pkg.engine, pkg.capi
    assert "llama" in S.lib().b200_model_families().decode().split(",")
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 1000, n).tolist() for n in (40, 7, 150)]
    m = S.Model(folder, dtype=S.BF16, max_tokens=1024, max_slots=2)
    assert m.family == "llama" and m.vocab == 1000 and m.page_rows == 128
    # each prompt alone through the engine itself: logits of its last token
    want = []
    for p in prompts:
        eng = E.Engine(1, 512, dtype=capi.F16, **SHAPE)
        eng.init_random(seed=5, std=0.05)
        eng.prefill(np.asarray([p], np.int32))
        want.append(eng.logits().float().cpu().numpy()[0].copy())
        eng.close()
    # through the registry: two prompts as one ragged batch, the third in portions in a slot that was used before
    got, ids = m.step([(0, prompts[0], [len(prompts[0]) - 1]), (1, prompts[1], [len(prompts[1]) - 1])], ids=True)
    assert rel(got[0], want[0]) < 2e-2 and rel(got[1], want[1]) < 2e-2
    assert ids.tolist() == [int(np.argmax(got[0])), int(np.argmax(got[1]))]
    m.release(1)
    m.step([(1, prompts[2][:100], [])])
    got2 = m.step([(1, prompts[2][100:], [49]), (0, [int(ids[0])], [0])])
    assert rel(got2[0], want[2]) < 2e-2
    assert m.slot_length(0) == 41 and m.slot_length(1) == 150
    with pytest.raises(RuntimeError):           # only the last place of an entry
        m.step([(0, [1, 2, 3], [0])])
    m.release(0)
    m.release(1)
    # the shared scheduler: three requests on two slots
    outs, steps = m.generate(prompts, max_new=6, chunk=64)
    assert [len(o) for o in outs] == [6, 6, 6] and steps >= 8
    for o, w in zip(outs, want):
        assert o[0] == int(np.argmax(w))         # the first token comes from the prompt's last logits
    m.close()
