"""Each kernel that the Musilorn family brought to include/b200_serve.h, alone, against the plain functions of
musilorn_oracle.py (or a line of torch): the sandwich norm, concatenation, caps, rotary angle tables, the q / k
preparation (short convolution with carried inputs, head norm, both rotary pairings, page stores), paged grouped-query
attention with a cap and a sink, retention with a carried state, the unit-RMS gate, and the tanh-gelu GLU epilogue."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import musilorn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S(pkg):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    return pkg.serve


_alive = []


def dev(t, dtype=None):
    t = torch.as_tensor(t).cuda()
    t = t.to(dtype).contiguous() if dtype is not None else t.contiguous()
    _alive.append(t)
    return t


def ints(a):
    return dev(torch.as_tensor(a, dtype=torch.int32))


@pytest.fixture(autouse=True)
def _drop_device_tensors():
    yield
    torch.cuda.synchronize()
    _alive.clear()


def tdt(S, code):
    return torch.bfloat16 if code == S.BF16 else torch.float32


def code_of(S, kind):
    return S.BF16 if kind == "bf16" else S.F32


def rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def sync_ok(rc):
    assert rc == 0, f"rc={rc}"
    torch.cuda.synchronize()


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("width", [1, 48, 1000, 2048, 2049, 5000])
@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_layernorm_residual_and_next_norm(S, width, kind):
    code, g = code_of(S, kind), gen(width)
    x, y = torch.randn(5, width, generator=g) * 2 + 3, torch.randn(5, width, generator=g) * 4 - 7
    w, b, w2, b2 = (torch.randn(width, generator=g) for _ in range(4))
    xd, out2 = dev(x), torch.empty(5, width, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_layernorm_residual(xd.data_ptr(), dev(y).data_ptr(), 5, width, 1e-5, 0.3, dev(w).data_ptr(), dev(b).data_ptr(),
                                            dev(w2).data_ptr(), dev(b2).data_ptr(), out2.data_ptr(), code, None))
    want_x = x.double() + 0.3 * O.layer_norm(y.double(), w.double(), b.double(), 1e-5)
    assert rel(xd, want_x) < 2e-6                     # the residual is fp32 in both serving dtypes
    if width > 1:
        assert rel(out2.float(), O.layer_norm(want_x, w2.double(), b2.double(), 1e-5)) < (2e-2 if kind == "bf16" else 2e-5)
    xd2 = dev(x)
    sync_ok(S.lib().b200_layernorm_residual(xd2.data_ptr(), dev(y).data_ptr(), 5, width, 1e-5, 0.3, dev(w).data_ptr(), dev(b).data_ptr(),
                                            None, None, None, code, None))
    assert torch.equal(xd2, xd)


def test_concat_softcap_and_embedding_without_positions(S):
    g = gen(1)
    a, b = torch.randn(6, 20, generator=g), torch.randn(6, 20, generator=g)
    for code in (S.F32, S.BF16):
        out = torch.empty(6, 40, dtype=tdt(S, code), device="cuda")
        sync_ok(S.lib().b200_concat_cast(dev(a).data_ptr(), dev(b).data_ptr(), out.data_ptr(), 6, 20, code, None))
        assert torch.equal(out.cpu(), torch.cat([a, b], 1).to(tdt(S, code)))
    v = torch.randn(1000, generator=g) * 40
    vd = dev(v)
    sync_ok(S.lib().b200_softcap(vd.data_ptr(), 1000, 11.0, None))
    assert rel(vd, O.capped(v.double(), 11.0)) < 1e-6
    table = torch.randn(9, 12, generator=g)
    out = torch.empty(4, 12, device="cuda")
    sync_ok(S.lib().b200_embed_positions(ints([8, 0, 3, 3]).data_ptr(), None, dev(table).data_ptr(), None, out.data_ptr(), 4, 12, S.F32, None))
    assert torch.equal(out.cpu(), table[[8, 0, 3, 3]])


def test_rope_angles_stay_exact_far_out(S):
    rot = dict(base=10000.0, dims=16, scaling=dict(factor=8.0, low=1.0, high=4.0, original=64))
    f = O.rot_frequencies(rot)
    pos = torch.tensor([0, 1, 63, 64, 4097, 1_000_003], dtype=torch.int32)
    c, s = torch.empty(6, 8, device="cuda"), torch.empty(6, 8, device="cuda")
    sync_ok(S.lib().b200_rope_angles(dev(pos).data_ptr(), 6, dev(f).data_ptr(), 8, c.data_ptr(), s.data_ptr(), None))
    ang = pos.double()[:, None] * f[None, :]
    assert float((c.double().cpu() - torch.cos(ang)).abs().max()) < 1e-7
    assert float((s.double().cpu() - torch.sin(ang)).abs().max()) < 1e-7
    # the scaled set differs from the plain one exactly where the wavelengths are long
    plain = O.rot_frequencies(dict(base=10000.0, dims=16))
    assert torch.equal(f[:1], plain[:1]) and plain[1] / 8 < f[1] < plain[1] and torch.allclose(f[-1], plain[-1] / 8.0)


def angles(S, pos, rot):
    f = O.rot_frequencies(rot)
    n = len(f)
    c, s = torch.empty(len(pos), max(n, 1), device="cuda"), torch.empty(len(pos), max(n, 1), device="cuda")
    if n:
        c, s = c[:, :n].contiguous(), s[:, :n].contiguous()
        sync_ok(S.lib().b200_rope_angles(ints(pos).data_ptr(), len(pos), dev(f).data_ptr(), n, c.data_ptr(), s.data_ptr(), None))
    _alive.extend([c, s])
    return c, s


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,taps,rot_dims,layout", [(4, 2, 16, 4, 16, "interleaved"), (3, 1, 6, 2, 4, "half"),
                                                               (1, 1, 40, 1, 0, "interleaved"), (2, 2, 130, 5, 64, "interleaved")])
def test_qk_prepare_over_portions_with_carried_inputs(S, kind, heads, kv, dim, taps, rot_dims, layout):
    """two sequences in two slots, fed in portions of different sizes (shorter than the filter too); the convolution
    reaches back into earlier steps through the ring, into this step through the batch, and into zeros before position 0"""
    code, g = code_of(S, kind), gen(dim)
    PR, n_pages, max_pages = 4, 12, 6
    Cq, Ck = heads * dim, kv * dim
    ch = Cq + Ck
    lens = {0: 11, 1: 7}
    u = {b: torch.randn(n, ch, generator=g) for b, n in lens.items()}
    cw = torch.randn(ch, taps, generator=g)
    qn, kn = torch.rand(dim, generator=g) + 0.5, torch.rand(dim, generator=g) + 0.5
    rot = dict(base=100.0, dims=rot_dims)
    pages = torch.tensor([[7, 2, 9, 0, 0, 0], [4, 11, 1, 0, 0, 0]], dtype=torch.int32)
    state = torch.full((2, max(taps - 1, 1), ch), 1e4)        # stale inputs of an earlier owner
    kp, vp = (torch.full((n_pages * PR, kv, dim), 7.0, dtype=tdt(S, code), device="cuda") for _ in range(2))
    state_d, pages_d, cw_d, qn_d, kn_d = dev(state), dev(pages), dev(cw), dev(qn), dev(kn)
    # steps in which every sequence brings one token file their inputs in the ring inside the same launch
    plan = [[(0, 3), (1, 1)], [(0, 1), (1, 1)], [(0, 1), (1, 1)], [(1, 4)], [(0, 6)]]
    at = {0: 0, 1: 0}
    got_q = {0: [], 1: []}
    for step in plan:
        rows, slot, pos, start, end = [], [], [], [], []
        for b, n in step:
            rows.append(u[b][at[b]:at[b] + n])
            slot += [b] * n
            pos += list(range(at[b], at[b] + n))
            start += [at[b]] * n
            end += [at[b] + n] * n
            at[b] += n
        proj = dev(torch.cat(rows))
        T = len(slot)
        cs, sn = angles(S, pos, rot)
        q_out = torch.empty(T, Cq, dtype=tdt(S, code), device="cuda")
        a = S.QkPrepareArgs(proj.data_ptr(), ch, cw_d.data_ptr(), taps, state_d.data_ptr(), qn_d.data_ptr(), kn_d.data_ptr(), 1e-5,
                            cs.data_ptr(), sn.data_ptr(), rot_dims, S.ROPE_HALF if layout == "half" else S.ROPE_INTERLEAVED,
                            q_out.data_ptr(), kp.data_ptr(), vp.data_ptr(), 1, pages_d.data_ptr(), max_pages, PR,
                            ints(slot).data_ptr(), ints(pos).data_ptr(), ints(start).data_ptr(), T, heads, kv, dim, code,
                            int(all(n == 1 for _, n in step)))
        sync_ok(S.lib().b200_qk_prepare(C.byref(a), None))
        if not all(n == 1 for _, n in step):
            sync_ok(S.lib().b200_conv_state_update(proj.data_ptr(), ch, state_d.data_ptr(), ints(slot).data_ptr(), ints(pos).data_ptr(),
                                               ints(end).data_ptr(), T, ch, taps, None))
        r = 0
        for b, n in step:
            got_q[b].append(q_out[r:r + n].float().cpu())
            r += n
    tol = 2e-2 if kind == "bf16" else 2e-5
    for b, n in lens.items():
        y = O.short_conv(u[b].double(), cw.double())
        q = O.rotate(O.unit_rms(y[:, :Cq].reshape(n, heads, dim), 1e-5) * qn.double(), rot, layout).reshape(n, Cq)
        k = O.rotate(O.unit_rms(y[:, Cq:].reshape(n, kv, dim), 1e-5) * kn.double(), rot, layout)
        v = y[:, Cq:].reshape(n, kv, dim)
        assert rel(torch.cat(got_q[b]), q) < tol
        rows = [int(pages[b, p // PR]) * PR + p % PR for p in range(n)]
        assert rel(kp[rows].float(), k) < tol
        assert rel(vp[rows].float(), v) < tol
    used = {int(pages[b, p // PR]) * PR + p % PR for b, n in lens.items() for p in range(n)}
    other = [r for r in range(n_pages * PR) if r not in used]
    assert bool((kp[other].float() == 7.0).all()) and bool((vp[other].float() == 7.0).all())   # nothing else was written


def paged(S, code, k, v, PR, perm_seed):
    """k, v: dict slot -> [n, kv, d]; scatters them into shuffled pages. Returns pools, page table, max_pages"""
    n_slots, max_pages = len(k), max((len(x) + PR - 1) // PR for x in k.values())
    total = n_slots * max_pages + 3
    order = torch.randperm(total, generator=gen(perm_seed)).tolist()
    table = torch.zeros(n_slots, max_pages, dtype=torch.int32)
    kv, dk, dv = next(iter(k.values())).shape[1], next(iter(k.values())).shape[2], next(iter(v.values())).shape[2]
    kp = torch.full((total * PR, kv, dk), 300.0)       # rows nobody owns would dominate every softmax if they were read
    vp = torch.full((total * PR, kv, dv), -500.0)
    for b in k:
        for i in range((len(k[b]) + PR - 1) // PR):
            pg = order.pop()
            table[b, i] = pg
            n = min(PR, len(k[b]) - i * PR)
            kp[pg * PR: pg * PR + n] = k[b][i * PR: i * PR + n]
            vp[pg * PR: pg * PR + n] = v[b][i * PR: i * PR + n]
    return dev(kp, tdt(S, code)), dev(vp, tdt(S, code)), dev(table), max_pages


def run_attention(S, code, q, slot, pos, kp, vp, table, max_pages, PR, heads, kv, dim, vdim, scale, cap, bias, longest):
    T = len(slot)
    out = torch.empty(T, heads * vdim, dtype=tdt(S, code), device="cuda")
    need = S.lib().b200_paged_attention_workspace_bytes(T, heads, vdim)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    _alive.append(ws)
    a = S.PagedAttentionArgs(dev(q, tdt(S, code)).data_ptr(), out.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), max_pages, PR,
                             ints(slot).data_ptr(), ints(pos).data_ptr(), T, heads, kv, dim, vdim, scale, cap, bias, code, longest,
                             max(pos) + 1, ws.data_ptr(), need)
    sync_ok(S.lib().b200_paged_attention(C.byref(a), None))
    return out.float().cpu()


def plain_attention(q, k, v, pos, heads, kv, scale, cap, bias):
    """q [T, heads, d] at positions pos of ONE sequence with keys k [n, kv, d]"""
    out = []
    for t, p in enumerate(pos):
        row = []
        for h in range(heads):
            g = h // (heads // kv)
            s = (k[: p + 1, g] @ q[t, h]) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            row.append((e / (e.sum() + bias * math.exp(-m))) @ v[: p + 1, g])
        out.append(torch.cat(row))
    return torch.stack(out)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,cap,bias", [(4, 2, 16, 5.0, 1.0), (6, 1, 64, 30.0, 1.0), (3, 3, 10, 0.0, 0.0), (2, 1, 128, 8.0, 1.0)])
def test_paged_attention_prompts_tokens_and_mixed_batches(S, kind, heads, kv, dim, cap, bias):
    code, g = code_of(S, kind), gen(heads * dim)
    PR, scale = 16, 1.7 / math.sqrt(dim)
    lens = {0: 150, 1: 33, 2: 1}
    bf = (lambda t: t.bfloat16().float()) if kind == "bf16" else (lambda t: t)
    k = {b: bf(torch.randn(n, kv, dim, generator=g)) for b, n in lens.items()}
    v = {b: bf(torch.randn(n, kv, dim, generator=g)) for b, n in lens.items()}
    q = {b: bf(torch.randn(n, heads, dim, generator=g)) for b, n in lens.items()}
    kp, vp, table, max_pages = paged(S, code, k, v, PR, 5)
    tol = 2e-2 if kind == "bf16" else 2e-5
    # whole prompts of unequal length in one batch; the last tokens alone (a decode batch); portions beside single tokens
    batches = [[(0, 0, 150), (1, 0, 33), (2, 0, 1)], [(0, 149, 150), (1, 32, 33)], [(1, 15, 33), (0, 149, 150), (0, 0, 0)],
               [(0, 61, 131), (2, 0, 1), (1, 16, 17)]]
    for batch in batches:
        rows = [(b, p) for b, lo, hi in batch for p in range(lo, hi)]
        slot, pos = [b for b, _ in rows], [p for _, p in rows]
        qq = torch.stack([q[b][p] for b, p in rows]).reshape(len(rows), heads * dim)
        longest = max(hi - lo for _, lo, hi in batch)
        got = run_attention(S, code, qq, slot, pos, kp, vp, table, max_pages, PR, heads, kv, dim, dim, scale, cap, bias, longest)
        want = torch.cat([plain_attention(q[b][lo:hi].double(), k[b].double(), v[b].double(), list(range(lo, hi)), heads, kv, scale, cap, bias)
                          for b, lo, hi in batch if hi > lo])
        assert rel(got, want) < tol, batch


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("far", [0, 15, 16, 700])
def test_a_far_key_stands_out_and_the_sink_weighs_in(S, kind, far):
    """among a thousand keys one (the first, the last of a page, the first of the next, one in the middle) matches the
    query: its value must come through, damped exactly by the cap and by the one in the denominator"""
    code, g = code_of(S, kind), gen(far)
    heads, kv, dim, PR, n = 2, 1, 32, 16, 1000
    k = torch.randn(n, kv, dim, generator=g) * 0.05
    v = torch.randn(n, kv, dim, generator=g)
    q = torch.randn(2, heads, dim, generator=g) * 0.05       # the last token of a prompt portion, and the same decoded
    k[far, 0, :] = 1.0
    q[:, 1, :] = 1.0                                          # head 1 looks for it: raw score = dim * scale
    if kind == "bf16":
        k, v, q = k.bfloat16().float(), v.bfloat16().float(), q.bfloat16().float()
    kp, vp, table, max_pages = paged(S, code, {0: k}, {0: v}, PR, 9)
    for cap in (12.0, 0.0):
        want = plain_attention(q.double(), k.double(), v.double(), [n - 2, n - 1], heads, kv, 0.5, cap, 1.0)
        assert (want[0, dim:] - v[far, 0].double()).abs().max() < (0.8 if cap else 0.05)   # head 1 returns (nearly) that value
        for longest in (2, 1):
            got = run_attention(S, code, q.reshape(2, heads * dim), [0, 0], [n - 2, n - 1], kp, vp, table, max_pages, PR, heads, kv, dim, dim,
                                0.5, cap, 1.0, longest)
            assert rel(got, want) < (2e-2 if kind == "bf16" else 2e-5), (cap, longest)
    # a query that matches nothing: the sink takes its share, the output shrinks by sum e / (1 + sum e)
    z = plain_attention(q.double() * 0, k.double(), v.double(), [3], heads, kv, 0.5, 6.0, 1.0)
    got = run_attention(S, code, q.reshape(2, heads * dim)[:1] * 0, [0], [3], kp, vp, table, max_pages, PR, heads, kv, dim, dim, 0.5, 6.0, 1.0, 1)
    assert rel(got, z) < (2e-2 if kind == "bf16" else 2e-5)
    assert rel(z[0, :dim], v[:4, 0].double().sum(0) / 5.0) < 1e-9


@pytest.mark.parametrize("heads,dim,vdim,rot_dims,layout", [(3, 8, 12, 8, "half"), (1, 4, 4, 2, "interleaved"), (2, 40, 70, 0, "half"),
                                                            (2, 32, 96, 32, "half")])
def test_retention_in_portions_with_a_carried_state(S, heads, dim, vdim, rot_dims, layout):
    g = gen(dim + vdim)
    lens = {0: 300, 1: 45, 2: 3}
    ld = heads * (2 * dim + vdim) + 5                      # a wider row: the projections of a layer lie side by side
    q_off, k_off, v_off = 2, 2 + heads * dim, 5 + 2 * heads * dim
    proj = {b: torch.randn(n, ld, generator=g) for b, n in lens.items()}
    decay = torch.tensor([0.9, 1.0, 0.999][:heads])
    rot = dict(base=50.0, dims=rot_dims)
    state = dev(torch.full((3, heads, dim, vdim), 1e3))    # what an earlier owner of the slots left behind
    decay_d = dev(decay)
    plan = [[(0, 130), (1, 1), (2, 1)], [(0, 1), (1, 44), (2, 2)], [(0, 2)], [(0, 167)]]
    at = {b: 0 for b in lens}
    got = {b: [] for b in lens}
    for step in plan:
        rows, slot, pos, ent_row, ent_len = [], [], [], [], []
        for b, n in step:
            ent_row.append(len(slot))
            ent_len.append(n)
            rows.append(proj[b][at[b]:at[b] + n])
            slot += [b] * n
            pos += list(range(at[b], at[b] + n))
            at[b] += n
        T = len(slot)
        pd = dev(torch.cat(rows))
        cs, sn = angles(S, pos, rot)
        out = torch.empty(T, heads * vdim, device="cuda")
        need = S.lib().b200_retention_workspace_bytes(T, len(step), heads, dim, vdim)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        a = S.RetentionArgs(pd.data_ptr(), ld, q_off, k_off, v_off, cs.data_ptr(), sn.data_ptr(), rot_dims,
                            S.ROPE_HALF if layout == "half" else S.ROPE_INTERLEAVED, decay_d.data_ptr(), dim ** -0.5, state.data_ptr(),
                            out.data_ptr(), ints(ent_row).data_ptr(), ints(ent_len).data_ptr(), ints(slot).data_ptr(), ints(pos).data_ptr(),
                            len(step), T, heads, dim, vdim, max(ent_len), ws.data_ptr(), need)
        sync_ok(S.lib().b200_retention(C.byref(a), None))
        r = 0
        for b, n in step:
            got[b].append(out[r:r + n].cpu())
            r += n
    for b, n in lens.items():
        p = proj[b].double()
        q = O.rotate(p[:, q_off:q_off + heads * dim].reshape(n, heads, dim), rot, layout)
        k = O.rotate(p[:, k_off:k_off + heads * dim].reshape(n, heads, dim), rot, layout) * dim ** -0.5
        v = p[:, v_off:v_off + heads * vdim].reshape(n, heads, vdim)
        want = torch.stack([O.retention_state_walk(q[:, h], k[:, h], v[:, h], float(decay[h].double())) for h in range(heads)], 1)
        assert rel(torch.cat(got[b]), want.reshape(n, heads * vdim)) < 3e-5, b


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_unit_rms_gate(S, kind):
    code, g = code_of(S, kind), gen(3)
    o, gate = torch.randn(5, 3, 20, generator=g) * 50, torch.randn(5, 3 * 20 + 4, generator=g)
    out = torch.empty(5, 60, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_unit_rms_gate(dev(o).data_ptr(), dev(gate).data_ptr() + 16, 64, out.data_ptr(), 5, 3, 20, 1e-5, code, None))
    want = O.unit_rms(o.double(), 1e-5).reshape(5, 60) * O.silu(gate[:, 4:].double())
    assert rel(out.float(), want) < (2e-2 if kind == "bf16" else 2e-5)


@pytest.mark.parametrize("M,N,K,kind", [(5, 24, 40, "f32"), (70, 24, 40, "bf16"), (300, 128, 64, "bf16"), (9, 256, 192, "bf16"), (130, 100, 72, "f32")])
def test_glu_with_tanh_gelu_in_the_gemm_epilogue(S, M, N, K, kind):
    code, g = code_of(S, kind), gen(M)
    x, w = torch.randn(M, K, generator=g), torch.randn(2 * N, K, generator=g) / math.sqrt(K)
    if kind == "bf16":
        x, w = x.bfloat16().float(), w.bfloat16().float()
    out = torch.empty(M, N, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_linear_ex(dev(x, tdt(S, code)).data_ptr(), dev(w, tdt(S, code)).data_ptr(), out.data_ptr(), M, N, K, code, code,
                                   S.GG_GLU_GELU, None, 0, None))
    want = O.gelu_tanh(x.double() @ w[:N].double().T) * (x.double() @ w[N:].double().T)
    assert rel(out.float(), want) < (2e-2 if kind == "bf16" else 2e-5)
    # the unfused form of small batches: plain product, then the activation kernel
    gu = dev((x @ w.T).float())
    out2 = torch.empty(M, N, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_glu_act(gu.data_ptr(), out2.data_ptr(), M, N, S.GG_GLU_GELU, code, None))
    assert rel(out2.float(), want) < (2e-2 if kind == "bf16" else 2e-5)
    sync_ok(S.lib().b200_glu_act(gu.data_ptr(), out2.data_ptr(), M, N, S.GG_GLU, code, None))
    assert rel(out2.float(), O.silu(x.double() @ w[:N].double().T) * (x.double() @ w[N:].double().T)) < (2e-2 if kind == "bf16" else 2e-5)
