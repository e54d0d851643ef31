"""Each kernel of include/b200_serve.h alone against the plain fp32 functions of nekodra_oracle.py (or one line of
torch): layer norm pairs, embedding with positions, grouped / strided / gathered GEMM with its epilogues, latent rows
into pages, latent attention with a sink over pages, router, dispatch, residual update."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import nekodra_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S(pkg):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    return pkg.serve


_alive = []   # device tensors whose pointers were handed to the library stay referenced until the test ends


def dev(t, dtype=None):
    t = t.cuda()
    t = t.to(dtype).contiguous() if dtype is not None else t.contiguous()
    _alive.append(t)
    return t


@pytest.fixture(autouse=True)
def _drop_device_tensors():
    yield
    torch.cuda.synchronize()
    _alive.clear()


def tdt(S, code):
    return torch.bfloat16 if code == S.BF16 else torch.float32


def tol(S, code):
    return 2e-2 if code == S.BF16 else 2e-5


def rel(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def sync_ok(rc):
    assert rc == 0, f"rc={rc}"
    torch.cuda.synchronize()


@pytest.mark.parametrize("width", [1, 48, 192, 1000])
@pytest.mark.parametrize("code", ["f32", "bf16"])
def test_layernorm_pair(S, width, code):
    code = S.BF16 if code == "bf16" else S.F32
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3 + 5      # a large mean: one-pass variance would lose digits
    w1, b1, w2, b2 = (torch.randn(width, generator=g) for _ in range(4))
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32)
    xd, o1, o2 = dev(x), torch.empty(4, width, dtype=tdt(S, code), device="cuda"), torch.empty(4, width, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_layernorm_pair(xd.data_ptr(), dev(rows).data_ptr(), 4, width, 1e-5, dev(w1).data_ptr(), dev(b1).data_ptr(),
                                        o1.data_ptr(), dev(w2).data_ptr(), dev(b2).data_ptr(), o2.data_ptr(), code, None))
    xs = x[rows.long()]
    if width > 1:
        assert rel(o1.float().cpu(), O.layer_norm(xs, w1, b1, 1e-5)) < tol(S, code)
        assert rel(o2.float().cpu(), O.layer_norm(xs, w2, b2, 1e-5)) < tol(S, code)
    else:   # a single feature: the deviation is zero, the output is the bias
        assert torch.allclose(o1.float().cpu(), b1.expand(4, 1).to(tdt(S, code)).float())
    # single output form
    o3 = torch.empty(7, width, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_layernorm_pair(xd.data_ptr(), None, 7, width, 1e-5, dev(w1).data_ptr(), dev(b1).data_ptr(), o3.data_ptr(),
                                        None, None, None, code, None))
    if width > 1:
        assert rel(o3.float().cpu(), O.layer_norm(x, w1, b1, 1e-5)) < tol(S, code)


def test_embed_positions(S):
    g = torch.Generator().manual_seed(1)
    table, ptab = torch.randn(11, 20, generator=g), torch.randn(9, 20, generator=g)
    ids, pos = torch.tensor([3, 3, 10, 0], dtype=torch.int32), torch.tensor([0, 8, 2, 2], dtype=torch.int32)
    for code in (S.F32, S.BF16):
        t, p = dev(table, tdt(S, code)), dev(ptab, tdt(S, code))
        out = torch.empty(4, 20, device="cuda")
        sync_ok(S.lib().b200_embed_positions(dev(ids).data_ptr(), dev(pos).data_ptr(), t.data_ptr(), p.data_ptr(), out.data_ptr(), 4, 20, code, None))
        assert torch.equal(out.cpu(), t.float().cpu()[ids.long()] + p.float().cpu()[pos.long()])


def gg(S, **kw):
    a = S.GemmGroupedArgs()
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 70, 33), (130, 64, 96), (77, 200, 300)])
@pytest.mark.parametrize("combo", ["fff", "bbf", "bbb", "fbf", "fbb"])
def test_gemm_dense(S, M, N, K, combo):
    code = {"f": S.F32, "b": S.BF16}
    ta, tw, tc = (code[c] for c in combo)
    g = torch.Generator().manual_seed(M * 1000 + N)
    A = dev(torch.randn(M, K + 3, generator=g), tdt(S, ta))[:, :K]          # a leading dimension wider than K
    W = dev(torch.randn(N, K, generator=g), tdt(S, tw))
    Cm = torch.zeros(M, N + 5, dtype=tdt(S, tc), device="cuda")
    args = gg(S, A=A.data_ptr(), W=W.data_ptr(), C=Cm.data_ptr(), lda=K + 3, ldw=K, ldc=N + 5, M=M, N=N, K=K, batch=1, trans_b=1,
              a_dtype=ta, w_dtype=tw, c_dtype=tc)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(args), None))
    a_used = A.float().bfloat16().float() if tw == S.BF16 else A.float()       # bf16 products round A on load
    want = a_used.cpu().double() @ W.float().cpu().double().T
    assert rel(Cm[:, :N].float().cpu(), want) < (1e-2 if tc == S.BF16 else 1e-5)
    assert float(Cm[:, N:].float().abs().max()) == 0.0                           # nothing written beyond N


@pytest.mark.parametrize("code", ["f32", "bf16"])
def test_gemm_strided_heads_both_layouts_and_gate(S, code):
    """per-head products addressed inside wider activations: [K, N] weights (query absorption), [N, K] weights with
    the sigmoid gate in the epilogue (value up-projection)"""
    code = S.BF16 if code == "bf16" else S.F32
    T, H, dq, dv, R = 37, 3, 10, 12, 24
    g = torch.Generator().manual_seed(5)
    ld = H * dq + H * dv + 7
    proj = dev(torch.randn(T, ld, generator=g))
    uk = dev(torch.randn(H * dq, R, generator=g), tdt(S, code))
    uv = dev(torch.randn(H * dv, R, generator=g), tdt(S, code))
    qa = torch.zeros(T, H, R, device="cuda")
    a1 = gg(S, A=proj.data_ptr(), lda=ld, stride_a=dq, W=uk.data_ptr(), ldw=R, stride_w=dq * R, trans_b=0, C=qa.data_ptr(), ldc=H * R,
            stride_c=R, M=T, N=R, K=dq, batch=H, a_dtype=S.F32, w_dtype=code, c_dtype=S.F32)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(a1), None))
    rnd = (lambda t: t.bfloat16().float()) if code == S.BF16 else (lambda t: t)
    q = rnd(proj[:, :H * dq]).cpu().double().reshape(T, H, dq)
    want = torch.einsum("thd,hdr->thr", q, uk.float().cpu().double().reshape(H, dq, R))
    assert rel(qa.cpu(), want) < 1e-5
    oa = dev(torch.randn(T, H, R, generator=g))
    att = torch.zeros(T, H * dv, dtype=tdt(S, code), device="cuda")
    gate = proj[:, H * dq:]
    a2 = gg(S, A=oa.data_ptr(), lda=H * R, stride_a=R, W=uv.data_ptr(), ldw=R, stride_w=dv * R, trans_b=1, C=att.data_ptr(), ldc=H * dv,
            stride_c=dv, aux=gate.data_ptr(), ld_aux=ld, stride_aux=dv, epi=S.GG_SIGMOID_MUL, M=T, N=dv, K=R, batch=H,
            a_dtype=S.F32, w_dtype=code, c_dtype=code)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(a2), None))
    v = torch.einsum("thr,hvr->thv", rnd(oa).cpu().double(), uv.float().cpu().double().reshape(H, dv, R)).reshape(T, H * dv)
    want = v * torch.sigmoid(gate[:, :H * dv].cpu().double())
    assert rel(att.float().cpu(), want) < tol(S, code)


@pytest.mark.parametrize("code", ["f32", "bf16"])
def test_gemm_groups_gather_glu(S, code):
    """experts: rows sorted by group, gathered from the token matrix, GLU epilogue; an empty group and a group with
    more rows than a tile"""
    code = S.BF16 if code == "bf16" else S.F32
    T, D, F, E = 150, 40, 24, 4
    g = torch.Generator().manual_seed(9)
    h = dev(torch.randn(T, D, generator=g), tdt(S, code))
    Wgu = dev(torch.randn(E, 2 * F, D, generator=g) / math.sqrt(D), tdt(S, code))
    counts = [100, 0, 49, 1]
    off = torch.tensor([0, 100, 100, 149, 150], dtype=torch.int32)
    src = torch.randint(0, T, (150,), generator=g, dtype=torch.int32)
    out = torch.zeros(150, F, dtype=tdt(S, code), device="cuda")
    a = gg(S, A=h.data_ptr(), lda=D, a_rows=dev(src).data_ptr(), group_off=dev(off).data_ptr(), W=Wgu.data_ptr(), ldw=D,
           stride_w=2 * F * D, trans_b=1, epi=S.GG_GLU, C=out.data_ptr(), ldc=F, M=T, N=F, K=D, batch=E, a_dtype=code, w_dtype=code, c_dtype=code)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(a), None))
    hc, wc = h.float().cpu(), Wgu.float().cpu()
    r0 = 0
    for e, n in enumerate(counts):
        rows = hc[src[r0:r0 + n].long()]
        want = O.silu(rows @ wc[e, :F].T) * (rows @ wc[e, F:].T)
        if n:
            assert rel(out[r0:r0 + n].float().cpu(), want) < tol(S, code), e
        r0 += n


def paged(S, lengths, rank, page_rows, code, seed=0, shuffle=True):
    """random latent rows for sequences of the given lengths in a shuffled page pool -> (rows per seq, pool, table)"""
    g = torch.Generator().manual_seed(seed)
    max_pages = max((n + page_rows - 1) // page_rows for n in lengths) + 1
    n_pages = sum((n + page_rows - 1) // page_rows for n in lengths) + 3
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    table = torch.zeros(len(lengths), max_pages, dtype=torch.int32)
    pool = torch.zeros(n_pages, page_rows, rank, dtype=tdt(S, code))
    seqs = []
    for b, n in enumerate(lengths):
        c = torch.randn(n, rank, generator=g).to(tdt(S, code))
        for p in range((n + page_rows - 1) // page_rows):
            pg = order.pop()
            table[b, p] = pg
            part = c[p * page_rows:(p + 1) * page_rows]
            pool[pg, :len(part)] = part
        seqs.append(c.float())
    return seqs, pool, table, max_pages


@pytest.mark.parametrize("code", ["f32", "bf16"])
@pytest.mark.parametrize("rank", [8, 40, 96, 512])
def test_latent_attention_with_sink_over_pages(S, code, rank):
    code = S.BF16 if code == "bf16" else S.F32
    PR, H = 16, 3
    lengths = [1, 16, 17, 75]
    seqs, pool, table, max_pages = paged(S, lengths, rank, PR, code, seed=rank)
    g = torch.Generator().manual_seed(2)
    # queries: every position of sequences 0..2, the last 5 and position 15 / 16 (a page border) of sequence 3
    slot, pos = [], []
    for b in range(3):
        slot += [b] * lengths[b]
        pos += list(range(lengths[b]))
    slot += [3] * 7
    pos += [15, 16, 70, 71, 72, 73, 74]
    T = len(slot)
    qa = torch.randn(T, H, rank, generator=g) * (2.0 / math.sqrt(rank))
    sink = torch.tensor([-30.0, 0.5, 4.0])     # one head whose sink is negligible, one whose sink dominates
    out = torch.zeros(T, H, rank, device="cuda")
    scale = 0.7
    sync_ok(S.lib().b200_latent_attention(dev(qa).data_ptr(), out.data_ptr(), dev(pool).data_ptr(), dev(table).data_ptr(), max_pages, PR,
                                          dev(torch.tensor(slot, dtype=torch.int32)).data_ptr(), dev(torch.tensor(pos, dtype=torch.int32)).data_ptr(),
                                          dev(sink).data_ptr(), scale, T, H, rank, code, 0, 0, None, 0, None))
    got = out.cpu()
    for t in range(T):
        c = seqs[slot[t]][:pos[t] + 1]
        for h in range(H):
            want = O.sink_attention(qa[t, h][None], c, c, scale, sink[h])[0]      # keys = values = the cached rows
            assert rel(got[t, h], want) < (1e-4 if code == S.F32 else 2e-2), (t, h)   # bf16: the query and the weights are rounded for the tensor cores


def test_latent_attention_far_key_stands_out(S):
    """one row far back (beyond several pages) scaled so that its score dominates: the output must be that row"""
    PR, R = 64, 32
    seqs, pool, table, max_pages = paged(S, [700], R, PR, S.F32, seed=4)
    qa = torch.zeros(1, 1, R)
    qa[0, 0] = seqs[0][3] * 4.0                      # aligned with row 3
    out = torch.zeros(1, 1, R, device="cuda")
    sync_ok(S.lib().b200_latent_attention(dev(qa).data_ptr(), out.data_ptr(), dev(pool).data_ptr(), dev(table).data_ptr(), max_pages, PR,
                                          dev(torch.tensor([0], dtype=torch.int32)).data_ptr(), dev(torch.tensor([699], dtype=torch.int32)).data_ptr(),
                                          dev(torch.tensor([0.0])).data_ptr(), 1.0, 1, 1, R, S.F32, 0, 0, None, 0, None))
    want = O.sink_attention(qa[0, 0][None], seqs[0], seqs[0], 1.0, torch.tensor(0.0))[0]
    assert rel(out.cpu()[0, 0], want) < 1e-4
    assert rel(out.cpu()[0, 0], seqs[0][3]) < 1e-2   # and it IS row 3, to within the softmax tail


@pytest.mark.parametrize("heads", [1, 5, 16])
def test_latent_attention_decode_batch_with_split_contexts(S, heads):
    """one token per sequence over contexts of very different lengths: the bf16 kernel splits the rows over several CTAs
    and merges the shares with the sink afterwards; a context shorter than one share, and one of a single row"""
    PR, R = 64, 72
    lengths = [1, 50, 700, 1300]
    seqs, pool, table, max_pages = paged(S, lengths, R, PR, S.BF16, seed=heads)
    g = torch.Generator().manual_seed(3)
    T = len(lengths)
    qa = torch.randn(T, heads, R, generator=g) * (3.0 / math.sqrt(R))
    sink = torch.randn(heads, generator=g) * 2
    out = torch.zeros(T, heads, R, device="cuda")
    nbytes = S.lib().b200_latent_attention_workspace_bytes(T, heads, R)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    sync_ok(S.lib().b200_latent_attention(dev(qa).data_ptr(), out.data_ptr(), dev(pool).data_ptr(), dev(table).data_ptr(), max_pages, PR,
                                          dev(torch.arange(T, dtype=torch.int32)).data_ptr(),
                                          dev(torch.tensor([n - 1 for n in lengths], dtype=torch.int32)).data_ptr(),
                                          dev(sink).data_ptr(), 0.6, T, heads, R, S.BF16, 1, max(lengths), ws.data_ptr(), nbytes, None))
    got = out.cpu()
    for t in range(T):
        for h in range(heads):
            want = O.sink_attention(qa[t, h][None], seqs[t], seqs[t], 0.6, sink[h])[0]
            assert rel(got[t, h], want) < 2e-2, (t, h)


@pytest.mark.parametrize("code", ["f32", "bf16"])
def test_latent_store_rms_norm_into_pages(S, code):
    code = S.BF16 if code == "bf16" else S.F32
    PR, R, ld = 8, 20, 33
    g = torch.Generator().manual_seed(3)
    raw = torch.randn(6, ld, generator=g) * 3
    w = torch.randn(R, generator=g)
    table = torch.tensor([[4, 1, 0], [2, 3, 0]], dtype=torch.int32)
    slot = torch.tensor([0, 0, 1, 1, 1, 0], dtype=torch.int32)
    pos = torch.tensor([7, 8, 0, 15, 16 - 8, 0], dtype=torch.int32)
    pool = torch.zeros(5, PR, R, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_latent_store(dev(raw).data_ptr(), ld, dev(w).data_ptr(), 1e-6, pool.data_ptr(), dev(table).data_ptr(), 3, PR,
                                      dev(slot).data_ptr(), dev(pos).data_ptr(), 6, R, code, None))
    want = O.rms_norm(raw[:, :R], w, 1e-6)
    pc = pool.float().cpu()
    for t in range(6):
        pg = int(table[slot[t], pos[t] // PR])
        assert rel(pc[pg, pos[t] % PR], want[t]) < (1e-2 if code == S.BF16 else 1e-5)
    assert int((pc.abs().sum(-1) > 0).sum()) == 6    # nothing else was written


@pytest.mark.parametrize("n_out,n_exp,top", [(7, 5, 3), (4, 4, 1), (12, 8, 4), (3, 0, 2)])
def test_router_dispatch_combine(S, n_out, n_exp, top):
    T, D = 50, 24
    g = torch.Generator().manual_seed(n_out)
    h = torch.randn(T, D, generator=g)
    wr = torch.randn(n_out, D, generator=g) * 0.5
    corr = torch.randn(n_out, generator=g) * 0.3    # large enough to change the choice against the plain scores
    chosen = torch.zeros(T, top, dtype=torch.int32, device="cuda")
    weight = torch.zeros(T, top, device="cuda")
    sync_ok(S.lib().b200_moe_route(dev(h).data_ptr(), S.F32, dev(wr).data_ptr(), dev(corr).data_ptr(), T, D, n_out, top, 1.5,
                                   chosen.data_ptr(), weight.data_ptr(), None))
    want_c, want_w = O.route(h, wr, corr, top, 1.5)
    assert torch.equal(chosen.cpu().long().sort(-1).values, want_c.sort(-1).values)
    s = torch.softmax(h @ wr.T, -1)
    assert rel(weight.cpu(), torch.gather(s, 1, chosen.cpu().long()) * 1.5) < 1e-5
    plain = torch.topk(s, top, dim=-1).indices.sort(-1).values
    if n_out > top:
        assert not torch.equal(plain, want_c.sort(-1).values)     # the correction matters in this test
    off = torch.zeros(n_exp + 1, dtype=torch.int32, device="cuda")
    src = torch.full((T * top,), -7, dtype=torch.int32, device="cuda")
    dest = torch.zeros(T, top, dtype=torch.int32, device="cuda")
    sync_ok(S.lib().b200_moe_dispatch(chosen.data_ptr(), T, top, n_exp, off.data_ptr(), src.data_ptr(), dest.data_ptr(), None))
    ch, offc, srcc, destc = chosen.cpu(), off.cpu(), src.cpu(), dest.cpu()
    for e in range(n_exp):
        assert int(offc[e + 1] - offc[e]) == int((ch == e).sum())
    for t in range(T):
        for k in range(top):
            e, d = int(ch[t, k]), int(destc[t, k])
            if e >= n_exp:
                assert d == -1
            else:
                assert offc[e] <= d < offc[e + 1] and int(srcc[d]) == t
    n_rows = int(offc[n_exp])
    assert len(set(destc[destc >= 0].tolist())) == n_rows
    # residual update: gathers expert rows by dest, identity experts take the token's own input
    eo = torch.randn(max(n_rows, 1), D, generator=g)
    x, mix, sh = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)
    xd = dev(x.clone())
    sync_ok(S.lib().b200_residual_combine(xd.data_ptr(), dev(mix).data_ptr(), dev(sh).data_ptr(), dev(eo).data_ptr(), dest.data_ptr(),
                                          weight.data_ptr(), dev(h).data_ptr(), S.F32, T, D, top, None))
    want = x + mix + sh
    wc = weight.cpu()
    for t in range(T):
        for k in range(top):
            d = int(destc[t, k])
            want[t] += wc[t, k] * (eo[d] if d >= 0 else h[t])
    assert rel(xd.cpu(), want) < 1e-5


@pytest.mark.parametrize("M", [1, 8, 200, 257, 700])
@pytest.mark.parametrize("N,K,glu", [(136, 64, False), (512, 192, False), (1000, 520, False), (128, 64, True), (384, 200, True)])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_linear_ex_bf16_on_the_tcgen05_gemm(S, M, N, K, glu, out):
    """contiguous bf16 products: weight-streaming (swapped, split-K) up to 256 rows, token-major above, GLU epilogue,
    fp32 and bf16 outputs, ragged M / N / K tails"""
    oc = S.BF16 if out == "bf16" else S.F32
    g = torch.Generator().manual_seed(M + N)
    x = dev(torch.randn(M, K, generator=g), torch.bfloat16)
    W = dev(torch.randn((2 if glu else 1) * N, K, generator=g) / math.sqrt(K), torch.bfloat16)
    y = torch.zeros(M, N, dtype=tdt(S, oc), device="cuda")
    nbytes = S.lib().b200_linear_ex_workspace_bytes(M, N, K)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    sync_ok(S.lib().b200_linear_ex(x.data_ptr(), W.data_ptr(), y.data_ptr(), M, N, K, S.BF16, oc, S.GG_GLU if glu else S.GG_NONE,
                                   ws.data_ptr(), nbytes, None))
    xc, wc = x.float().cpu().double(), W.float().cpu().double()
    want = (O.silu(xc @ wc[:N].T) * (xc @ wc[N:].T)) if glu else xc @ wc.T
    assert rel(y.float().cpu(), want) < (1e-2 if oc == S.BF16 else 2e-5)
