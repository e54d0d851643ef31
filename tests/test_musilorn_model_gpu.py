"""The Musilorn family through the library's own entry points (registry -> step function -> paged cache and slot state
-> scheduler) against the plain implementation in musilorn_oracle.py, on small random models of several shapes: whole
prompts with every layer run, prefill against token-by-token decoding, prompt portions down to two tokens (shorter than
the convolution), unequal batches against each request alone, pages, slots and carried state that are freed and used
again, page borders, long decoding, sizes that are 1 or equal to each other, layer spans that repeat, and greedy
generation through the continuous-batching scheduler."""
import numpy as np
import pytest
import torch

import musilorn_oracle as O

pytestmark = pytest.mark.gpu

SCALING = dict(factor=8.0, low=1.0, high=3.0, original=64)
SHAPES = {
    # the span [attention, retention] runs twice, then one more attention layer; grouped heads, scaled frequencies
    "mix": dict(width=48, vocab=61, loop=(0, 2, 2), layers=[
        dict(type="attention", heads=4, kv_heads=2, dim=16, conv=4, scaling=SCALING, base=100.0, ff=40),
        dict(type="retention", heads=3, dim=8, vdim=12, decay=[0.9, 0.97, 0.995], ff=None),
        dict(type="attention", heads=2, kv_heads=2, dim=8, conv=3, softcap=2.0, scale=0.9, ff=24)]),
    # sizes that are 1 or equal; a one-tap convolution; partial rotation; one key head for six query heads; a span in
    # the middle that runs three times; an attention layer without feed-forward and a retention layer with one
    "odd": dict(width=40, vocab=33, loop=(1, 3, 3), residual_mult=1.0, logit_softcap=3.0, layers=[
        dict(type="attention", heads=1, kv_heads=1, dim=8, conv=1, rot_dims=4, ff=None),
        dict(type="retention", heads=1, dim=4, vdim=4, rot_dims=2, decay=[0.5], ff=16),
        dict(type="attention", heads=6, kv_heads=1, dim=6, conv=2, ff=8),
        dict(type="retention", heads=2, dim=6, vdim=10, rot_dims=0, decay=[0.99, 1.0], ff=None)]),
    # no span at all; retention first; nothing a multiple of 8; five taps; a span of one layer would be the same weights
    "plain": dict(width=36, vocab=41, layers=[
        dict(type="retention", heads=5, dim=10, vdim=7, decay=[0.8, 0.9, 0.95, 0.98, 0.999], ff=20),
        dict(type="attention", heads=3, kv_heads=3, dim=10, conv=5, rot_dims=6, scaling=SCALING, ff=None),
        dict(type="attention", heads=4, kv_heads=2, dim=12, conv=4, base=50.0, ff=28)]),
    # heads as wide as the tensor-core tiles take them, a value size above one warp pass, a span of one layer
    "wide": dict(width=64, vocab=50, loop=(0, 1, 2), layers=[
        dict(type="attention", heads=4, kv_heads=2, dim=64, conv=4, scaling=SCALING, ff=128),
        dict(type="retention", heads=2, dim=32, vdim=72, decay=[0.95, 0.999], ff=None),
        dict(type="attention", heads=2, kv_heads=1, dim=128, conv=2, ff=None)]),
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
        cfg, w = O.random_model(seed=70 + i, **sh)
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
    """fp32: every row within the tolerance. bfloat16: the unit-RMS norm of a retention head whose output is nearly zero
    (q.k close to 0 with one small head) turns a rounding error into a change of sign, which moves that row by much more
    than rounding does elsewhere; so nine rows in ten have to be within the tolerance, the median well inside it, and
    no row anywhere near a wrong answer."""
    e = row_errors(got, want)
    assert np.all(np.isfinite(e)), what
    if kind == "f32":
        assert e.max() < RTOL[kind], (what, float(e.max()))
    else:
        assert np.quantile(e, 0.9) < RTOL[kind] and np.median(e) < RTOL[kind] / 3 and e.max() < 0.6, \
            (what, float(np.quantile(e, 0.9)), float(np.median(e)), float(e.max()))


def open_model(S, folder, kind, max_tokens=1024, slots=4):
    return S.Model(folder, dtype=S.BF16 if kind == "bf16" else S.F32, max_tokens=max_tokens, max_slots=slots)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_and_every_layer_run(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    runs = O.layer_runs(cfg)
    assert m.family == "Musilorn" and m.vocab == cfg["vocab"] and m.n_layers == len(runs)
    toks = tokens(150, cfg["vocab"], 1)
    m.capture_layers(True)
    got = m.step([(0, toks, list(range(150)))])
    want, trail = oracle.forward(toks, return_layers=True)
    layers = m.captured_layers(150)
    for i in range(len(runs)):
        check(layers[i], trail[i].numpy(), kind, f"residual after layer run {i} (layer {runs[i][0]})")
    check(got, want.numpy(), kind)
    assert m.step_launches > 0
    m.close()


def test_every_mechanism_reaches_the_logits(models):
    """sensitivity of the comparison itself: with the added one of the softmax denominator, the cap, the convolution's
    history, the frequency scaling, the decay, the repeated span's input projection or the post norms changed, the
    oracle's logits move by far more than the tolerance the library is held to"""
    _, oracle, cfg = models["mix"]
    toks = tokens(60, cfg["vocab"], 2)
    base = oracle.forward(toks).numpy()
    import copy

    def moved(change_cfg=None, change_w=None):
        c, w = copy.deepcopy(cfg), dict(oracle.w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(w)
        return err(O.Oracle(c, w).forward(toks).numpy(), base)

    def cap(c): c["layers"][2]["mixer"]["softcap"] = 1e6
    def scaling(c): del c["layers"][0]["mixer"]["rot"]["scaling"]
    def decay(c): c["layers"][1]["mixer"]["decay"] = [0.9, 0.97, 0.99]
    def times(c): c["loop"]["times"] = 1
    def conv(w): w["l0.mix.k.conv"] = torch.cat([torch.zeros_like(w["l0.mix.k.conv"][:, :1]), w["l0.mix.k.conv"][:, 1:]], 1)
    def loop_in(w): w["loop.in"] = torch.cat([w["loop.in"][:, :48], torch.zeros_like(w["loop.in"][:, 48:])], 1)
    def post(w): w["l1.norm1b.b"] = torch.zeros_like(w["l1.norm1b.b"])
    for change in (cap, scaling, decay, times):
        assert moved(change_cfg=change) > 20 * RTOL["f32"], change.__name__
    for change in (conv, loop_in, post):
        assert moved(change_w=change) > 20 * RTOL["f32"], change.__name__
    # the sink: a plain softmax instead
    plain = O.capped_sink_attention
    try:
        def no_sink(q, k, v, scale, cap):
            T = q.shape[0]
            s = cap * torch.tanh((q @ k.T) * scale / cap)
            s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
            return torch.softmax(s, -1) @ v
        O.capped_sink_attention = no_sink
        assert err(oracle.forward(toks).numpy(), base) > 20 * RTOL["f32"]
    finally:
        O.capped_sink_attention = plain


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", list(SHAPES))
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
@pytest.mark.parametrize("name", ["mix", "plain"])
def test_decoding_from_the_very_first_token(S, models, name, kind):
    """no prompt portion at all: the convolution's history and the state grow one token at a time from nothing"""
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    toks = tokens(12, cfg["vocab"], 5)
    got = np.concatenate([m.step([(0, [t], [0])]) for t in toks])
    check(got, oracle.forward(toks).numpy(), kind)
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["mix", "odd", "plain"])
def test_portions_of_changing_size_down_to_two_tokens(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    PR = m.page_rows
    # portions shorter than the convolution, ending at, before and after page borders
    sizes = [2, 3, PR - 5, 2, PR, 1, 1, 2, 2, 1, 3, PR + 1, 5, 2]
    n = sum(sizes)
    toks = tokens(n, cfg["vocab"], 4)
    want = oracle.forward(toks).numpy()
    got, at = [], 0
    for s in sizes:
        got.append(m.step([(2, toks[at:at + s], list(range(s)))]))
        at += s
    check(np.concatenate(got), want, kind)
    m.close()


@pytest.mark.parametrize("name", ["odd", "mix"])
def test_a_position_does_not_depend_on_the_cut_or_the_batch(S, models, name):
    """fp32: the same request alone in one step, in portions, and inside unequal batches gives the same logits to
    rounding (far below the tolerance against the oracle)"""
    folder, oracle, cfg = models[name]
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
        assert err(g, alone[i]) < 1e-5, i
        assert err(g, oracle.forward(t).numpy()) < RTOL["f32"], i
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_pages_slots_and_state_are_used_again(S, models, kind):
    """a pool of three pages serves requests one after the other and two at a time; stale rows, stale convolution
    inputs and a stale retention state of earlier owners stay in place and must not be seen"""
    folder, oracle, cfg = models["mix"]
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
    got_c = m.step([(1, c[:2], [1]), ])        # slot 1 held b's state a moment ago
    got_c2 = m.step([(1, c[2:], list(range(len(c) - 2)))])
    assert set(pages_a) <= set(m.slot_pages(1))            # c sits in pages that a filled before
    want = oracle.forward(c).numpy()
    check(np.concatenate([got_c, got_c2]), want[1:], kind)
    m.release(1)
    # the freed slots and pages again, now for a short request next to a growing one
    got_a = m.step([(0, a[:PR], [PR - 1]), (1, b[:7], [6])])
    got_a2 = m.step([(0, a[PR:], [len(a) - PR - 1]), (1, b[7:], [len(b) - 8])])
    wa, wb = oracle.forward(a).numpy(), oracle.forward(b).numpy()
    check(np.stack([got_a[0], got_a2[0]]), wa[[PR - 1, len(a) - 1]], kind)
    check(np.stack([got_a[1], got_a2[1]]), wb[[6, len(b) - 1]], kind)
    m.close()


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_long_decoding(S, models, name):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, "f32")
    toks = tokens(330, cfg["vocab"], 40)
    want = oracle.forward(toks).numpy()
    m.step([(3, toks[:10], [])])
    got = [m.step([(3, [t], [0])])[0] for t in toks[10:]]
    assert err(np.stack(got), want[10:]) < RTOL["f32"]
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_a_long_prompt_in_one_step_and_in_large_portions(S, models, kind):
    """several hundred tokens at once (the tiled prompt kernels, chunked retention), then the same in portions that
    are not multiples of any tile"""
    folder, oracle, cfg = models["wide"]
    m = open_model(S, folder, kind, max_tokens=2048)
    n = 700
    toks = tokens(n, cfg["vocab"], 41)
    want = oracle.forward(toks).numpy()
    ask = list(range(0, n, 7)) + [n - 1]
    check(m.step([(0, toks, ask)]), want[ask], kind)
    got, at = [], 0
    for s in (333, 1, 130, 236):
        got.append(m.step([(1, toks[at:at + s], list(range(0, s, 5)))]))
        at += s
    rows = [a + k for a, s in zip((0, 333, 334, 464), (333, 1, 130, 236)) for k in range(0, s, 5)]
    check(np.concatenate(got), want[rows], kind)
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_repeated_single_token_steps_while_buffers_grow(S, models, kind):
    """single-token steps of one shape repeat (the engine replays them as a captured graph); in between a longer
    portion arrives and makes the scratch buffers grow, contexts pass 256 and 384 tokens (other splits of the decoding
    attention), and two sequences decode side by side"""
    folder, oracle, cfg = models["wide"]
    m = open_model(S, folder, kind, max_tokens=2048)
    V = cfg["vocab"]
    a, b = tokens(420, V, 60), tokens(770, V, 61)
    wa, wb = oracle.forward(a).numpy(), oracle.forward(b).numpy()
    got_a = [m.step([(0, a[:5], [4])])]
    for p in range(5, 12):                                   # one shape, seven times
        got_a.append(m.step([(0, [a[p]], [0])]))
    got_b = [m.step([(1, b[:600], [599])])]                  # the buffers grow
    for p in range(12, 20):
        got_a.append(m.step([(0, [a[p]], [0])]))
    got_a.append(m.step([(0, a[20:250], [229])]))
    for p in range(250, 420):                                # across 256 and 384 tokens of context, beside the other sequence
        out = m.step([(0, [a[p]], [0]), (1, [b[350 + p]], [0])])
        got_a.append(out[:1])
        got_b.append(out[1:])
    check(np.concatenate(got_a), wa[[4] + list(range(5, 20)) + [249] + list(range(250, 420))], kind)
    check(np.concatenate(got_b), wb[[599] + list(range(600, 770))][: len(got_b)], kind)
    m.close()


def test_bad_steps_are_refused(S, models):
    folder, _, cfg = models["mix"]
    m = open_model(S, folder, "f32", max_tokens=128, slots=2)
    for bad in ([(2, [1, 2], [0])], [(0, [1], [1])], [(0, [1], [0]), (0, [2], [0])], [(0, [1] * 129, [])]):
        with pytest.raises(RuntimeError):
            m.step(bad)
    assert m.pages_free == m.pages_total
    m.close()


def test_bad_configurations_are_refused(S, tmp_path):
    cfg, w = O.random_model(3, layers=[dict(type="attention", heads=4, kv_heads=2, dim=8, ff=16)])
    for change in (lambda c: c["layers"][0].update(type="window"), lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
                   lambda c: c["layers"][0]["mixer"].update(vdim=16), lambda c: c["layers"][0]["mlp"].update(kind="moe"),
                   lambda c: c.update(loop=dict(start=0, stop=2, times=2)), lambda c: c["layers"][0]["mixer"].update(dim=16)):
        import copy
        c2 = copy.deepcopy(cfg)
        change(c2)
        O.write_model(str(tmp_path), c2, w)
        with pytest.raises(RuntimeError):
            open_model(S, str(tmp_path), "f32")


@pytest.mark.parametrize("name", ["mix", "odd"])
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
