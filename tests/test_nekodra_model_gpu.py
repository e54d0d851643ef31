"""The Nekodra family through the library's own entry points (registry -> step function -> paged cache ->
scheduler) against the plain implementation in nekodra_oracle.py, on small random models of several shapes:
whole prompts, prefill against token-by-token decoding, prompt portions down to two tokens, unequal batches against
each request alone, pages and slots that are freed and used again, page borders, long decoding, sizes that are 1 or
equal to each other, and greedy generation through the continuous-batching scheduler."""
import numpy as np
import pytest
import torch

import nekodra_oracle as O

pytestmark = pytest.mark.gpu

MLP_A = dict(kind="moe", expert=dict(ff=48), router=dict(experts=5, identity=2, top=3, scale=1.25), shared=dict(ff=32))
SHAPES = {
    # two layers, the second reads the first one's cached rows
    "pair": dict(width=64, vocab=97, layers=[dict(heads=3, dim=16, vdim=24, kv_rank=40, scale=0.25, mlp=MLP_A),
                                              dict(heads=3, dim=16, vdim=24, kv_rank=40, scale=0.25, kv_from=0, mlp=MLP_A)]),
    # sizes that are 1 or equal; a layer without feed-forward; no identity experts; no shared expert; top 1; a far kv_from
    "odd": dict(width=40, vocab=33, layers=[
        dict(heads=1, dim=8, vdim=8, kv_rank=8, scale=0.35, mlp=None),
        dict(heads=2, dim=12, vdim=20, kv_rank=24, scale=0.3,
             mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=3, identity=0, top=1, scale=1.0), shared=None)),
        dict(heads=4, dim=6, vdim=10, kv_rank=16, scale=0.4,
             mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=1, identity=3, top=2, scale=2.0), shared=dict(ff=8))),
        dict(heads=5, dim=4, vdim=4, kv_rank=24, scale=0.5, kv_from=1,
             mlp=dict(kind="moe", expert=dict(ff=24), router=dict(experts=6, identity=1, top=7, scale=0.5), shared=dict(ff=56))),
    ]),
    # only identity experts beside the shared one; a rank above one warp pass
    "wide": dict(width=96, vocab=50, layers=[
        dict(heads=2, dim=32, vdim=16, kv_rank=136, scale=0.18,
             mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=0, identity=4, top=2, scale=1.0), shared=dict(ff=40)))]),
    # nothing a multiple of 8: every vector path has to fall back; more heads than one attention tile has rows
    "ragged": dict(width=36, vocab=41, layers=[
        dict(heads=3, dim=5, vdim=7, kv_rank=12, scale=0.45,
             mlp=dict(kind="moe", expert=dict(ff=10), router=dict(experts=3, identity=1, top=2, scale=1.5), shared=dict(ff=6))),
        dict(heads=40, dim=3, vdim=2, kv_rank=12, scale=0.6, kv_from=0,
             mlp=dict(kind="moe", expert=dict(ff=7), router=dict(experts=2, identity=2, top=3, scale=0.75), shared=dict(ff=9)))]),
}
RTOL = {"f32": 2e-4, "bf16": 6e-2}


@pytest.fixture(scope="module")
def S(pkg):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    return pkg.serve


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, sh) in enumerate(SHAPES.items()):
        cfg, w = O.random_model(seed=10 + i, max_positions=400, **sh)
        folder = tmp_path_factory.mktemp(name)
        O.write_model(str(folder), cfg, w)
        out[name] = (str(folder), O.Oracle(cfg, w), cfg)
    return out


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def row_errors(got, want):
    """per row: rms of the difference with its mean taken off, over the rms of the wanted row"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return (np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))).reshape(-1)


def err(got, want):
    return float(row_errors(got, want).max())


def check(got, want, kind, what=""):
    """fp32: every row within the tolerance. bfloat16: rounding may flip a router's close call for a token, which moves
    that row by much more than rounding does, so nine rows in ten have to be within the tolerance and the median well
    inside it."""
    e = row_errors(got, want)
    assert np.all(np.isfinite(e)), what
    if kind == "f32":
        assert e.max() < RTOL[kind], (what, float(e.max()))
    else:
        assert np.quantile(e, 0.9) < RTOL[kind] and np.median(e) < RTOL[kind] / 3, (what, float(np.quantile(e, 0.9)), float(np.median(e)))


def open_model(S, folder, kind, max_tokens=1024, slots=4):
    return S.Model(folder, dtype=S.BF16 if kind == "bf16" else S.F32, max_tokens=max_tokens, max_slots=slots)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_and_every_layer(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    assert m.family == "Nekodra" and m.vocab == cfg["vocab"] and m.n_layers == len(cfg["layers"])
    toks = tokens(150, cfg["vocab"], 1)
    m.capture_layers(True)
    got = m.step([(0, toks, list(range(150)))])
    want, trail = oracle.forward(toks, return_layers=True)
    layers = m.captured_layers(150)
    for i in range(len(cfg["layers"])):
        check(layers[i], trail[i].numpy(), kind, f"residual after layer {i}")
    check(got, want.numpy(), kind)
    assert m.step_launches > 0
    m.close()


def test_the_sink_and_the_correction_reach_the_logits(models):
    """sensitivity of the comparison itself: without the sink, or with the router's correction left out, the oracle's
    logits move by far more than the tolerance the library is held to"""
    _, oracle, cfg = models["pair"]
    toks = tokens(40, cfg["vocab"], 2)
    base = oracle.forward(toks).numpy()
    w2 = {k: (torch.full_like(v, -1e9) if k.endswith("mix.sink") else v) for k, v in oracle.w.items()}
    assert err(O.Oracle(cfg, w2).forward(toks).numpy(), base) > 20 * RTOL["f32"]
    w3 = {k: (torch.zeros_like(v) if k.endswith("mlp.correction") else v) for k, v in oracle.w.items()}
    assert err(O.Oracle(cfg, w3).forward(toks).numpy(), base) > 20 * RTOL["f32"]


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["pair", "odd", "ragged"])
def test_prefill_then_token_by_token_across_page_borders(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    PR = m.page_rows
    n = 2 * PR + 9
    toks = tokens(n, cfg["vocab"], 3)
    want = oracle.forward(toks).numpy()
    cut = PR - 3                          # decoding crosses the first and the second page border
    rows = [m.step([(1, toks[:cut], [0, cut - 1])])]
    for p in range(cut, n):
        rows.append(m.step([(1, [toks[p]], [0])]))
    got = np.concatenate(rows)
    check(got, want[[0] + list(range(cut - 1, n))], kind)
    assert m.slot_length(1) == n and len(m.slot_pages(1)) == 3
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_portions_of_changing_size_down_to_two_tokens(S, models, kind):
    folder, oracle, cfg = models["pair"]
    m = open_model(S, folder, kind)
    PR = m.page_rows
    sizes = [2, 3, PR - 5, 2, PR, 1, 1, 2, PR + 1, 5]     # portions that end at, before and after page borders
    n = sum(sizes)
    toks = tokens(n, cfg["vocab"], 4)
    want = oracle.forward(toks).numpy()
    got, at = [], 0
    for s in sizes:
        got.append(m.step([(2, toks[at:at + s], list(range(s)))]))
        at += s
    check(np.concatenate(got), want, kind)
    m.close()


def test_a_position_does_not_depend_on_the_cut_or_the_batch(S, models):
    """fp32: the same request alone in one step, in portions, and inside unequal batches gives the same logits to
    rounding (far below the tolerance against the oracle)"""
    folder, oracle, cfg = models["odd"]
    V = cfg["vocab"]
    reqs = [tokens(n, V, 20 + i) for i, n in enumerate([1, 23, 97, 140])]
    m = open_model(S, folder, "f32")
    alone = []
    for i, t in enumerate(reqs):
        alone.append(m.step([(i, t, list(range(len(t))))]))
        m.release(i)
    assert m.pages_free == m.pages_total
    # a schedule of unequal portions beside single tokens; request 0 joins late, request 1 sits steps out
    plan = {0: [0, 0, 0, 1], 1: [5, 0, 1, 1, 0, 16], 2: [64, 1, 1, 2, 29], 3: [2, 62, 3, 64, 1, 1, 7]}
    at = {i: 0 for i in plan}
    got = {i: [] for i in plan}
    for step in range(8):
        entries, who = [], []
        for i, sizes in plan.items():
            s = sizes[step] if step < len(sizes) else 0
            if s:
                entries.append((i, reqs[i][at[i]:at[i] + s], list(range(s))))
                who.append((i, s))
                at[i] += s
        if not entries:
            continue
        out = m.step(entries)
        r = 0
        for i, s in who:
            got[i].append(out[r:r + s])
            r += s
    for i, t in enumerate(reqs):
        assert at[i] == len(t)
        g = np.concatenate(got[i])
        assert err(g, alone[i]) < 2e-6, i
        assert err(g, oracle.forward(t).numpy()) < RTOL["f32"], i
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_pages_and_slots_are_used_again(S, models, kind):
    """a pool of three pages serves five requests one after the other and two at a time; stale rows of earlier owners
    stay in the pages and must not be seen"""
    folder, oracle, cfg = models["pair"]
    m = open_model(S, folder, kind, max_tokens=3 * 64, slots=2)
    PR, V = m.page_rows, cfg["vocab"]
    assert m.pages_total == 3
    a, b, c = tokens(PR + 10, V, 30), tokens(PR - 1, V, 31), tokens(2 * PR + 1, V, 32)
    m.step([(0, a, [])])
    with pytest.raises(RuntimeError):          # b fits (1 page), c would need 3 more
        m.step([(1, c, [0])])
    assert m.slot_length(1) == 0 and m.pages_free == 1     # the failed step took nothing
    got_b = m.step([(1, b, list(range(len(b))))])
    check(got_b, oracle.forward(b).numpy(), kind)
    pages_a = m.slot_pages(0)
    m.release(0)
    m.release(1)
    assert m.pages_free == 3
    got_c = m.step([(1, c[:5], [4]), ])
    got_c2 = m.step([(1, c[5:], list(range(len(c) - 5)))])
    assert set(pages_a) <= set(m.slot_pages(1))            # c sits in pages that a filled before
    want = oracle.forward(c).numpy()
    check(np.concatenate([got_c, got_c2]), want[4:], kind)
    m.release(1)
    # the freed slot and pages again, now for a short request next to a growing one
    got_a = m.step([(0, a[:PR], [PR - 1]), (1, b[:7], [6])])
    got_a2 = m.step([(0, a[PR:], [len(a) - PR - 1]), (1, b[7:], [len(b) - 8])])
    wa, wb = oracle.forward(a).numpy(), oracle.forward(b).numpy()
    check(np.stack([got_a[0], got_a2[0]]), wa[[PR - 1, len(a) - 1]], kind)
    check(np.stack([got_a[1], got_a2[1]]), wb[[6, len(b) - 1]], kind)
    m.close()


def test_long_decoding(S, models):
    folder, oracle, cfg = models["wide"]
    m = open_model(S, folder, "f32")
    toks = tokens(330, cfg["vocab"], 40)
    want = oracle.forward(toks).numpy()
    m.step([(3, toks[:10], [])])
    got = [m.step([(3, [t], [0])])[0] for t in toks[10:]]
    assert err(np.stack(got), want[10:]) < RTOL["f32"]
    m.close()


def test_bad_steps_are_refused(S, models):
    folder, _, cfg = models["pair"]
    m = open_model(S, folder, "f32", max_tokens=128, slots=2)
    for bad in ([(2, [1, 2], [0])], [(0, [1], [1])], [(0, [1], [0]), (0, [2], [0])], [(0, [1] * 401, [])]):
        with pytest.raises(RuntimeError):
            m.step(bad)
    assert m.pages_free == m.pages_total
    m.close()


@pytest.mark.parametrize("name", ["pair", "odd"])
def test_greedy_generation_through_the_scheduler(S, models, name):
    """six requests on two slots, prompts fed in portions of seven tokens beside the others' single tokens"""
    folder, oracle, cfg = models[name]
    V = cfg["vocab"]
    prompts = [tokens(n, V, 50 + i) for i, n in enumerate([1, 30, 9, 64, 15, 2])]
    m = open_model(S, folder, "f32", max_tokens=4 * 64, slots=2)
    outs, steps = m.generate(prompts, max_new=12, chunk=7)
    assert steps > 12
    for p, o in zip(prompts, outs):
        assert o == oracle.greedy(p, 12)
    assert m.pages_free == m.pages_total
    # an end token stops a request early: take a token the third request produces as the end token
    eos = outs[2][5]
    outs2, _ = m.generate(prompts, max_new=12, eos_id=eos, chunk=0)
    for o, o2 in zip(outs, outs2):
        stop = next((k for k in range(1, len(o)) if o[k] == eos), len(o))
        assert o2 == o[:stop]
    m.close()
