"""Host side of the model-family layer on a machine without a GPU: the registry, config.json / safetensors parsing
and the error paths that end before any CUDA call."""
import json
import os

import pytest
import torch

import nekodra_oracle as O


@pytest.fixture(scope="module")
def S(pkg):
    if not os.path.exists(pkg.lib_path()):
        pytest.fail(f"{pkg.lib_path()} not built: run __graft_entry__.build()")
    return pkg.serve


def test_registry_lists_the_families(S):
    fams = S.lib().b200_model_families().decode().split(",")
    assert "Nekodra" in fams


def test_unknown_architecture_and_broken_config(S, tmp_path):
    with pytest.raises(RuntimeError, match="cannot read"):
        S.Model(tmp_path / "nowhere")
    (tmp_path / "config.json").write_text('{"architecture": "Other", "width": 8}')
    with pytest.raises(RuntimeError, match="no family registered"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text('{"architecture": "Nekodra", "width": 8,')
    with pytest.raises(RuntimeError, match="json"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text('{"architecture": "Nekodra", "width": 8}')
    with pytest.raises(RuntimeError, match="required"):
        S.Model(tmp_path)


def test_oracle_pieces_agree_with_torch():
    """the plain implementation itself: its norms and its sink softmax against closed forms"""
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(5, 12, generator=g), torch.randn(12, generator=g), torch.randn(12, generator=g)
    assert torch.allclose(O.layer_norm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (12,), w, b, 1e-5), atol=1e-6)
    q, k, v = torch.randn(3, 4, generator=g), torch.randn(6, 4, generator=g), torch.randn(6, 5, generator=g)
    sink = torch.tensor(0.3)
    got = O.sink_attention(q, k, v, 0.5, sink)
    for i in range(3):
        n = 4 + i                                                   # the last three positions of six
        s = torch.cat([(q[i] @ k[:n].T) * 0.5, sink[None]])
        p = torch.softmax(s, 0)[:-1]                                # the sink takes its share and gives nothing back
        assert torch.allclose(got[i], p @ v[:n], atol=1e-6)
    # a very negative sink is plain softmax attention
    plain = O.sink_attention(q, k, v, 0.5, torch.tensor(-1e9))
    assert torch.allclose(plain[2], torch.softmax((q[2] @ k.T) * 0.5, 0) @ v, atol=1e-6)


def test_written_checkpoint_has_the_documented_layout(tmp_path):
    cfg, w = O.random_model(seed=1)
    O.write_model(str(tmp_path), cfg, w)
    raw = (tmp_path / "model.safetensors").read_bytes()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    assert header["l0.mix.q"]["shape"] == [48, 64] and header["l0.mix.q"]["dtype"] == "BF16"
    assert "l1.mix.dkv" not in header and "l0.mix.dkv" in header    # the second layer reads the first one's rows
    assert json.loads((tmp_path / "config.json").read_text())["layers"][1]["mixer"]["kv_from"] == 0
