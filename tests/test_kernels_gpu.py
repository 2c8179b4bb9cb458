"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same operation, at sizes
other than the engine's tiny models: head sizes in steps of 16, odd head counts and groups, widths
and vocabularies that are no power of two.  Inputs are built so that a fault would show: one far key
made to dominate, a window's edge, pages in scrambled order."""

import math
import random

import pytest
import torch

from tests.plain import minimax_m3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from quanta_b200 import kernels
    return kernels


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding(table_dtype):
    V, H, T = 1001, 328, 37
    table = torch.randn(V, H, device=DEV).to(table_dtype)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    h = torch.empty(T, H, device=DEV)
    st = K().new_status(DEV)
    K().embedding(h, table, ids, st)
    assert torch.equal(h, table[ids.long()].float())
    assert int(st[0]) == 0
    ids[5] = V + 3                              # refused, recorded, row zeroed; nothing faults
    K().embedding(h, table, ids, st)
    assert st.tolist()[:3] == [1, V + 3, 1] and float(h[5].abs().max()) == 0.0


@pytest.mark.parametrize("H", [72, 3072, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(H, out_dtype):
    T, S, eps = 19, 3, 1e-5
    h = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, S, H, device=DEV)
    w = 1 + 0.1 * torch.randn(H, device=DEV)
    h0 = h.clone()
    out = torch.empty(T, H, device=DEV, dtype=out_dtype)
    K().add_rmsnorm(h, delta, w, eps, out)
    want_h = h0.clone()
    for s in range(S):
        want_h += delta[:, s]
    assert torch.allclose(h, want_h, atol=1e-6)
    want = P.rms_norm(want_h, w, eps)
    assert torch.allclose(out.float(), want.to(out_dtype).float(), **tol(out_dtype))
    # rows subset, h untouched, bfloat16 delta
    rows = torch.tensor([7, 0, 18], device=DEV, dtype=torch.int32)
    d16 = torch.randn(T, H, device=DEV).bfloat16()
    h1 = h.clone()
    out3 = torch.empty(3, H, device=DEV, dtype=out_dtype)
    K().add_rmsnorm(h, d16, w, eps, out3, rows=rows, store_h=False)
    assert torch.equal(h, h1)
    want3 = P.rms_norm(h1[rows.long()] + d16[rows.long()].float(), w, eps)
    assert torch.allclose(out3.float(), want3.to(out_dtype).float(), **tol(out_dtype))


def _paged(kc, vc, table, req, length, kvh):
    """Gather a request's keys/values [length, hd] of one kv head from the pages."""
    P_ = kc.shape[2]
    pos = torch.arange(length)
    pages = torch.as_tensor(table[req])[pos // P_].long()
    return kc[pages, kvh, pos % P_].float(), vc[pages, kvh, pos % P_].float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rd,norm,page", [(6, 3, 48, 24, "per_head", 4), (5, 5, 16, 16, None, 16),
                                                     (12, 2, 128, 64, "per_layer", 8), (7, 1, 80, 0, "per_layer", 3)])
def test_qknorm_rope_write(dtype, nq, nkv, hd, rd, norm, page):
    k = K()
    T, theta, eps = 23, 12345.0, 1e-5
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV).to(dtype)
    if norm == "per_layer":
        qw, kw = 1 + 0.1 * torch.randn(nq * hd, device=DEV), 1 + 0.1 * torch.randn(nkv * hd, device=DEV)
    else:
        qw, kw = 1 + 0.1 * torch.randn(hd, device=DEV), 1 + 0.1 * torch.randn(hd, device=DEV)
    # two requests; positions start anywhere; pages scrambled
    lens = [(0, 9), (57, 14)]                     # (first position, tokens) per request
    pos = torch.tensor([p for a, n in lens for p in range(a, a + n)], dtype=torch.int32)
    req = torch.tensor([r for r, (a, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    max_pages = max(-(-(a + n) // page) for a, n in lens)
    num_pages = 2 * max_pages + 3
    ids = list(range(num_pages))
    random.Random(0).shuffle(ids)
    table = torch.tensor([ids[:max_pages], ids[max_pages:2 * max_pages]], dtype=torch.int32)
    kc = torch.zeros(num_pages, nkv, page, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nq, hd, device=DEV, dtype=dtype)
    inv = (1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / max(rd, 1)))).to(DEV) if rd else \
        torch.empty(0, device=DEV)
    st = k.new_status(DEV)
    kind = {None: k.NORM_NONE, "per_layer": k.NORM_PER_LAYER, "per_head": k.NORM_PER_HEAD}[norm]
    k.qknorm_rope_write(qkv, q_out, kc, vc, qw if norm else None, kw if norm else None, kind, eps, inv, None,
                        pos.to(DEV), pos.to(DEV), req.to(DEV), table.to(DEV), nq, nkv, hd, rd, page, st)
    assert int(st[0]) == 0
    x = qkv.float().cpu()
    q = x[:, : nq * hd].reshape(T, nq, hd)
    kk = x[:, nq * hd: (nq + nkv) * hd].reshape(T, nkv, hd)
    v = x[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if norm:
        q = P.qk_norm(q, qw.cpu(), nq, hd, norm, eps)
        kk = P.qk_norm(kk, kw.cpu(), nkv, hd, norm, eps)
    if rd:
        q, kk = P.partial_rope(q, pos, rd, theta), P.partial_rope(kk, pos, rd, theta)
    assert torch.allclose(q_out.float().cpu(), q.to(dtype).float(), **tol(dtype))
    for t in range(T):
        pg, sl = int(table[req[t], pos[t] // page]), int(pos[t]) % page
        assert torch.allclose(kc[pg, :, sl].float().cpu(), kk[t].to(dtype).float(), **tol(dtype))
        assert torch.equal(vc[pg, :, sl].cpu(), v[t].to(dtype))
    if rd < hd:      # dims past rotary_dim are exactly the normed values
        kk2 = x[:, nq * hd: (nq + nkv) * hd].reshape(T, nkv, hd)
        if norm is None:
            assert torch.equal(q_out.cpu()[..., rd:], x[:, : nq * hd].reshape(T, nq, hd)[..., rd:].to(dtype))
    # a block table entry outside the pool is refused, not followed
    bad = table.clone()
    bad[1, 0] = num_pages + 5
    bad[1, 1:] = num_pages + 5
    bad[0, :] = -1
    k.qknorm_rope_write(qkv, q_out, kc, vc, qw if norm else None, kw if norm else None, kind, eps, inv, None,
                        pos.to(DEV), pos.to(DEV), req.to(DEV), bad.to(DEV), nq, nkv, hd, rd, page, st)
    assert int(st[0]) == 2


def attention_reference(q, kc, vc, table, tok_pos, tok_req, scale, window):
    T, nq, hd = q.shape
    nkv = kc.shape[1]
    out = torch.zeros(T, nq, hd)
    kc, vc, G = kc.cpu(), vc.cpu(), nq // nkv
    for t in range(T):
        p, r = int(tok_pos[t]), int(tok_req[t])
        lo = max(0, p - window + 1) if window else 0
        for kvh in range(nkv):
            ks, vs = _paged(kc, vc, table, r, p + 1, kvh)
            for h in range(kvh * G, (kvh + 1) * G):
                s = (ks[lo:] @ q[t, h].float().cpu()) * scale
                out[t, h] = torch.softmax(s, 0) @ vs[lo:]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(6, 3, 48, 4, 0), (4, 4, 16, 16, 0), (12, 2, 128, 8, 0),
                                                   (5, 1, 256, 5, 0), (6, 2, 64, 4, 11), (40, 2, 32, 16, 0),
                                                   (48, 8, 128, 16, 0), (8, 2, 128, 16, 100), (4, 2, 48, 8, 37),
                                                   (48, 1, 64, 16, 0), (72, 1, 64, 8, 0), (32, 2, 128, 32, 50),
                                                   (4, 2, 256, 16, 0), (6, 1, 192, 8, 0), (16, 2, 128, 128, 0)])
@pytest.mark.parametrize("impl", ["simt", "mma", "mma_only"])
def test_paged_attention(dtype, nq, nkv, hd, page, window, impl, monkeypatch):
    """impl: the float32 SIMT kernel; the bfloat16 tensor-core kernels as the engine picks them (tcgen05 with
    O in TMEM for portions where the shapes allow); the same with the mma.sync kernel for every portion."""
    k = K()
    if impl != "simt" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernels are the bfloat16 path")
    if impl == "mma_only":
        if not k.attn_span_tc_supported(nq, nkv, hd, page):
            pytest.skip("these shapes run on the mma.sync kernels anyway")
        monkeypatch.setenv("QUANTA_B200_SPAN_KERNEL", "mma")
    torch.manual_seed(1)
    # (first position, tokens): prompt portions beside decode tokens; a portion that starts past a split edge
    spans = [(0, 13), (70, 1), (33, 9), (129, 1), (250, 30), (600, 1)]
    tok_pos = torch.tensor([p for a, n in spans for p in range(a, a + n)], dtype=torch.int32)
    tok_req = torch.tensor([r for r, (a, n) in enumerate(spans) for _ in range(n)], dtype=torch.int32)
    T = tok_pos.numel()
    max_pages = max(-(-(a + n) // page) for a, n in spans)
    num_pages = len(spans) * max_pages
    ids = list(range(num_pages))
    random.Random(2).shuffle(ids)
    table = torch.tensor([ids[r * max_pages:(r + 1) * max_pages] for r in range(len(spans))], dtype=torch.int32)
    kc = torch.randn(num_pages, nkv, page, hd, device=DEV).to(dtype)
    vc = torch.randn(num_pages, nkv, page, hd, device=DEV).to(dtype)
    q = torch.randn(T, nq, hd, device=DEV).to(dtype)
    # make one far key stand out for the last token of request 3: its score dominates, so a kernel that
    # skips or misplaces that key is far off
    far = 5 if not window else 600 - window + 1      # the oldest key still inside the window
    pg, sl = int(table[5,far // page]), far % page
    kc[pg, :, sl] = 0
    kc[pg, :, sl, 0] = 30.0
    q[T - 1, :, 0] = 8.0
    scale = hd ** -0.5
    out = torch.empty_like(q)
    st = k.new_status(DEV)
    def run():
        if impl == "simt":
            k.paged_attention_simt(q, kc, vc, out, tok_pos.to(DEV), tok_req.to(DEV), table.to(DEV), scale, window, st)
            return
        out.fill_(float("nan"))
        G, row0 = nq // nkv, 0
        dec, tiles = [], []
        for r, (a, n) in enumerate(spans):
            if n == 1 and G <= k.ATTN_DECODE_MAX_GROUP:      # larger groups: a single token is a portion of one
                dec.append(row0)
            else:
                tiles += [[r, row0, n, x] for x in range(0, n * G, k.attn_span_rows(hd, nq, nkv, page))]
            row0 += n
        n_parts = k.attn_decode_parts(nkv, max(a + n for a, n in spans))
        po = torch.full((len(dec) * nq * n_parts * hd,), float("nan"), device=DEV)
        pml = torch.full((len(dec) * nq * n_parts * 2,), float("nan"), device=DEV)
        if dec:
            k.attn_decode(q, kc, vc, out, po, pml, torch.tensor(dec, dtype=torch.int32, device=DEV), len(dec),
                          tok_pos.to(DEV), tok_req.to(DEV), table.to(DEV), scale, window, n_parts, st)
        k.attn_span(q, kc, vc, out, tok_pos.to(DEV), table.to(DEV), torch.tensor(tiles, dtype=torch.int32, device=DEV),
                    scale, window, st)

    run()
    assert int(st[0]) == 0
    want = attention_reference(q, kc, vc, table.tolist(), tok_pos, tok_req, scale, window)
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))
    # the far key carried the last token's output
    assert torch.allclose(out[T - 1, 0].float().cpu(), vc[pg, 0, sl].float().cpu(), atol=0.05)
    if window:       # one position further back is outside the window: it must not count
        pg2, sl2 = int(table[5,(far - 1) // page]), (far - 1) % page
        kc[pg2, :, sl2] = 0
        kc[pg2, :, sl2, 0] = 60.0
        run()
        assert torch.allclose(out[T - 1].float().cpu(), want[T - 1], **tol(dtype))
        # pages that lie wholly before the window of a request's first token have been given back: the
        # table holds -1 there, and the kernels must neither read them nor report them
        for r, (a, n) in enumerate(spans):
            table[r, : max(0, a - window + 1) // page] = -1
        assert int((table < 0).sum()) > 0
        run()
        assert int(st[0]) == 0
        assert torch.allclose(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("impl", ["tc", "mma_only"])
def test_span_attention_maximum_grows_late_in_some_rows(impl, monkeypatch):
    """A portion whose rows meet a key that dwarfs all earlier ones only in a LATER block of keys, and only
    some rows of each warp do (others never, others in two blocks): the kernel that keeps O in TMEM rescales
    it then, with instructions that the whole warp must run together whichever of its rows need it."""
    k = K()
    nq, nkv, hd, page = 4, 2, 128, 16
    assert k.attn_span_tc_supported(nq, nkv, hd, page)
    if impl != "tc":
        monkeypatch.setenv("QUANTA_B200_SPAN_KERNEL", "mma")
    torch.manual_seed(7)
    first, n = 300, 100                        # 200 rows a kv head: two tiles, the second not full
    tok_pos = torch.arange(first, first + n, dtype=torch.int32)
    tok_req = torch.zeros(n, dtype=torch.int32)
    max_pages = -(-(first + n) // page)
    ids = list(range(max_pages + 3))
    random.Random(3).shuffle(ids)
    table = torch.tensor([ids[:max_pages]], dtype=torch.int32)
    kc = torch.randn(len(ids), nkv, page, hd, device=DEV).bfloat16()
    vc = torch.randn(len(ids), nkv, page, hd, device=DEV).bfloat16()
    q = torch.randn(n, nq, hd, device=DEV).bfloat16()
    q[:, :, :2] = 0
    # keys 200 (second block of 128) and 290 (third) stand out along dimensions 0 and 1; only the rows
    # that look along a dimension see it
    for key, dim in ((200, 0), (290, 1)):
        pg, sl = int(table[0, key // page]), key % page
        kc[pg, :, sl] = 0
        kc[pg, :, sl, dim] = 30.0 * (dim + 1)
    rows_a = torch.arange(n) % 3 == 0          # grows in the second block
    rows_b = torch.arange(n) % 5 == 0          # grows in the third (again, for the rows of both)
    q[rows_a, :, 0] = 8.0
    q[rows_b, 1::2, 1] = 8.0                   # every other head: the two rows of a token differ
    scale = hd ** -0.5
    out = torch.full_like(q, float("nan"))
    st = k.new_status(DEV)
    G = nq // nkv
    tiles = [[0, 0, n, x] for x in range(0, n * G, k.attn_span_rows(hd, nq, nkv, page))]
    k.attn_span(q, kc, vc, out, tok_pos.to(DEV), table.to(DEV), torch.tensor(tiles, dtype=torch.int32, device=DEV),
                scale, 0, st)
    assert int(st[0]) == 0
    want = attention_reference(q, kc, vc, table.tolist(), tok_pos, tok_req, scale, 0)
    assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16))
    pg, sl = int(table[0, 290 // page]), 290 % page
    assert torch.allclose(out[0, 1].float().cpu(), vc[pg, 0, sl].float().cpu(), atol=0.05)     # token 0: both subsets


@pytest.mark.parametrize("n_dec,nq,nkv,hd,page", [(300, 4, 2, 64, 16), (70, 6, 1, 128, 8), (530, 2, 2, 32, 4)])
def test_decode_attention_many_tokens(n_dec, nq, nkv, hd, page):
    """More single tokens than one launch of the decode kernel takes (their positions live in shared
    memory), contexts from 1 to a few hundred keys, every request with pages of its own."""
    k = K()
    torch.manual_seed(n_dec)
    g = torch.Generator().manual_seed(n_dec)
    ctx_len = torch.randint(1, 400, (n_dec,), generator=g)
    ctx_len[0], ctx_len[1], ctx_len[-1] = 1, 64, 65
    max_pages = int(-(-ctx_len.max() // page))
    num_pages = n_dec * max_pages
    table = torch.randperm(num_pages, generator=g, dtype=torch.int64).to(torch.int32).view(n_dec, max_pages)
    kc = torch.randn(num_pages, nkv, page, hd, device=DEV).bfloat16()
    vc = torch.randn(num_pages, nkv, page, hd, device=DEV).bfloat16()
    q = torch.randn(n_dec, nq, hd, device=DEV).bfloat16()
    tok_pos = (ctx_len - 1).to(torch.int32)
    tok_req = torch.arange(n_dec, dtype=torch.int32)
    out = torch.full_like(q, float("nan"))
    n_parts = k.attn_decode_parts(nkv, int(ctx_len.max()))
    po = torch.full((n_dec * nq * n_parts * hd,), float("nan"), device=DEV)
    pml = torch.full((n_dec * nq * n_parts * 2,), float("nan"), device=DEV)
    st = k.new_status(DEV)
    k.attn_decode(q, kc, vc, out, po, pml, torch.arange(n_dec, dtype=torch.int32, device=DEV), n_dec, tok_pos.to(DEV),
                  tok_req.to(DEV), table.to(DEV), hd ** -0.5, 0, n_parts, st)
    assert int(st[0]) == 0
    want = attention_reference(q, kc, vc, table.tolist(), tok_pos, tok_req, hd ** -0.5, 0)
    assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("T,E,Kd", [(300, 256, 3072), (64, 100, 200), (1, 8, 64), (1000, 520, 328), (257, 33, 72)])
def test_router_gemm_mma(T, E, Kd):
    """Router logits on the tensor cores from the gate as three bfloat16 pieces: float32 accuracy against
    a float64 product, the pieces add up to the gate, and a row does not depend on the rows beside it."""
    k = K()
    torch.manual_seed(E)
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    gate = torch.randn(E, Kd, device=DEV) / Kd ** 0.5
    pieces = k.split3_bf16(gate)
    assert pieces.shape == (3, E, Kd)
    back = pieces[0].double() + pieces[1].double() + pieces[2].double()
    assert float((back - gate.double()).abs().max()) <= 2.0 ** -22 * float(gate.abs().max())
    parts = k.router_gemm_mma_parts(Kd)
    assert parts == -(-Kd // 768)               # ranges of the inner dimension, a function of its size alone
    logits = torch.full((parts, T, E), float("nan"), device=DEV)
    k.router_gemm_mma(x, pieces, logits)
    want = x.double() @ gate.double().T
    assert torch.allclose(logits.double().sum(0), want, atol=2e-5, rtol=1e-5)
    alone = torch.empty((parts, 1, E), device=DEV)
    k.router_gemm_mma(x[T // 2: T // 2 + 1].contiguous(), pieces, alone)
    assert torch.equal(alone[:, 0], logits[:, T // 2])


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,Kd", [(45, 257, 1000), (1, 256, 3072), (9, 12, 72), (300, 33, 1003), (64, 256, 3072)])
def test_router_small_logits(x_dtype, T, E, Kd):
    """Float32 logits of the CUDA-core router kernel: widths that are no multiple of 8 (the scalar form),
    more experts and tokens than one block takes; a token's logits alone are bit-identical."""
    x = torch.randn(T, Kd, device=DEV).to(x_dtype)
    gate = torch.randn(E, Kd, device=DEV)
    out = torch.full((T, E), float("nan"), device=DEV)
    K().router_small(x, gate, None, out)
    want = x.double() @ gate.double().T
    assert torch.allclose(out.double(), want, atol=1e-3, rtol=1e-5)
    t = T // 2
    alone = torch.empty(1, E, device=DEV)
    K().router_small(x[t: t + 1].contiguous(), gate, None, alone)
    assert torch.equal(alone[0], out[t])
    with pytest.raises(ValueError, match="shared-memory tile"):
        K().router_small(torch.zeros(2, 30000, device=DEV), torch.zeros(4, 30000, device=DEV), None, torch.empty(2, 4, device=DEV))


@pytest.mark.parametrize("E,k,bias,renorm,scale", [(8, 2, True, True, 1.0), (100, 7, False, True, 2.5),
                                                   (256, 8, True, True, 1.0), (33, 1, True, True, 1.0),
                                                   (520, 5, True, False, 0.5)])
def test_router_topk(E, k, bias, renorm, scale):
    _router_topk_case(29, 1, E, k, bias, renorm, scale)


@pytest.mark.parametrize("T,P,E,k", [(300, 1, 256, 8), (300, 4, 256, 8), (64, 3, 12, 3), (1000, 2, 520, 5), (77, 1, 1000, 9),
                                     (129, 2, 33, 33)])
def test_router_topk_many_tokens(T, P, E, k):
    """Steps of many tokens select with one warp a token; partial logits are added in index order."""
    _router_topk_case(T, P, E, k, True, True, 1.5)


def _router_topk_case(T, P, E, k, bias, renorm, scale):
    parts = torch.randn(P, T, E, device=DEV)
    parts[:, 3, :] = 0.0
    parts[0, 3, :] = 0.25                   # a full tie: lower expert indices win
    logits = parts[0].clone()
    for p in range(1, P):
        logits += parts[p]                  # the kernel's order of additions
    if P == 1:
        parts = parts[0].contiguous()
    _router_topk_check(parts, logits, T, E, k, bias, renorm, scale)


def _router_topk_check(parts, logits, T, E, k, bias, renorm, scale):
    b = (0.05 * torch.randn(E, device=DEV)) if bias else None
    if bias:
        b[: E // 2] = 0.0
    idx = torch.empty(T, k, device=DEV, dtype=torch.int32)
    w = torch.empty(T, k, device=DEV)
    K().router_topk(parts, b, idx, w, renorm, scale)
    scores = torch.sigmoid(logits)
    choice = scores + b[None] if bias else scores
    want_idx = torch.argsort(-choice, dim=-1, stable=True)[:, :k]
    want_w = torch.gather(scores, 1, want_idx)
    if renorm and k > 1:
        want_w = want_w / (want_w.sum(-1, keepdim=True) + 1e-20)
    want_w = want_w * scale
    assert torch.equal(idx.long(), want_idx)
    assert torch.allclose(w, want_w, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("T,E,k,Kd,bm", [(1, 256, 8, 3072, 16), (8, 256, 8, 3072, 16), (3, 12, 3, 72, 32), (64, 200, 6, 328, 128),
                                         (37, 16, 4, 100, 32), (300, 256, 8, 256, 128)])
def test_router_logits_selection_and_plan_in_one_launch(T, E, k, Kd, bm):
    """The router kernel of small steps (logits, selection, expert plan in one launch) against the three
    kernels it stands for, several times over (the counters of finished blocks must be back at zero after
    every launch).  300 tokens: 38 token tiles, each selected by the block that finished it last."""
    kern = K()
    assert kern.router_small_selects(T, E, k)
    torch.manual_seed(T * 7 + E)
    bias = 0.05 * torch.randn(E, device=DEV)
    gate = torch.randn(E, Kd, device=DEV) / Kd ** 0.5
    counters = torch.zeros(1 + -(-T // 8), dtype=torch.int32, device=DEV)
    st = kern.new_status(DEV)
    plan_words, max_tiles = kern.moe_plan_sizes(T * k, E, bm)
    for rep in range(3):
        x = torch.randn(T, Kd, device=DEV).bfloat16()
        logits = torch.empty(T, E, device=DEV)
        kern.router_small(x, gate, bias, logits)
        assert torch.allclose(logits.double(), x.double() @ gate.double().T, atol=1e-4)
        idx_a = torch.empty(T, k, device=DEV, dtype=torch.int32)
        w_a = torch.empty(T, k, device=DEV)
        kern.router_topk(logits, bias, idx_a, w_a, True, 1.5)
        a = [torch.zeros(n, dtype=torch.int32, device=DEV) for n in (plan_words, T * k, max_tiles, max_tiles)]
        kern.moe_plan(idx_a, E, bm, *a, st)
        idx_b = torch.empty_like(idx_a)
        w_b = torch.empty_like(w_a)
        logits_b = torch.empty_like(logits)
        b = [torch.zeros(n, dtype=torch.int32, device=DEV) for n in (plan_words, T * k, max_tiles, max_tiles)]
        kern.router_small(x, gate, bias, logits_b, idx_b, w_b, True, 1.5, counters=counters, bm=bm, plan=b[0],
                          sorted_pair=b[1], tile_expert=b[2], tile_row0=b[3], status=st)
        assert int(counters.abs().sum()) == 0
        assert torch.equal(logits, logits_b)
        assert torch.equal(idx_a, idx_b) and torch.equal(w_a, w_b)
        counts, offsets = a[0][:E], a[0][2 * E: 3 * E + 1]
        assert torch.equal(counts, b[0][:E]) and torch.equal(offsets, b[0][2 * E: 3 * E + 1])
        assert torch.equal(a[0][3 * E + 1: 3 * E + 3], b[0][3 * E + 1: 3 * E + 3])       # tiles, active experts
        n_tiles, n_active = int(a[0][3 * E + 1]), int(a[0][3 * E + 2])
        assert torch.equal(a[0][3 * E + 4: 3 * E + 4 + n_active], b[0][3 * E + 4: 3 * E + 4 + n_active])
        assert torch.equal(a[2][:n_tiles], b[2][:n_tiles]) and torch.equal(a[3][:n_tiles], b[3][:n_tiles])
        # the rows of an expert may come in any order: compare them as sets
        off = offsets.tolist()
        pa, pb = a[1].tolist(), b[1].tolist()
        for e in range(E):
            assert sorted(pa[off[e]: off[e + 1]]) == sorted(pb[off[e]: off[e + 1]])
        assert sorted(pb) == list(range(T * k))
    kern.raise_on_status(st.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("path", ["simt", "tc"])
@pytest.mark.parametrize("T,H,I,E,k", [(1, 72, 40, 12, 3), (37, 96, 48, 16, 4), (130, 328, 200, 9, 2), (9, 1024, 520, 6, 2),
                                       (300, 256, 136, 7, 2), (700, 64, 40, 9, 8), (600, 328, 200, 7, 4),
                                       (1100, 136, 264, 7, 4)])
def test_expert_products(dtype, T, H, I, E, k, path):
    kern = K()
    if path != "simt" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernels are the bfloat16 path")
    # the last three cases have some hundred rows an expert: tiles of 256 rows, taken by pairs of blocks (inner
    # sizes that are no multiple of the 64-wide k block, feature counts that end inside a block's 128 or leave
    # the pair's second block without any, experts of three tiles with a ragged last one)
    bm = kern.expert_tile_rows(T, T * k / E) if path == "tc" else kern.MOE_SIMT_BM
    assert path != "tc" or bm == (256 if T * k / E >= 112 else min(128, max(16, 1 << (T - 1).bit_length())))
    torch.manual_seed(3)
    x = torch.randn(T, H, device=DEV).to(dtype)
    # scaled so that outputs stay of order one at every size (the tolerance is absolute)
    w13 = (torch.randn(E, 2 * I, H, device=DEV) / math.sqrt(H)).to(dtype)
    w2 = (torch.randn(E, H, I, device=DEV) / math.sqrt(I)).to(dtype)
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    if T > 30:
        idx[:30, 0] = 5                       # one expert with many rows (several tiles), some with none
        idx[:30, 1:] = torch.where(idx[:30, 1:] == 5, (idx[:30, 1:] + 1) % E, idx[:30, 1:])
        idx[:30, 1] = torch.where(idx[:30, 1] == idx[:30, 0], 6, idx[:30, 1])
    pw = torch.rand(T, k, device=DEV)
    n_pairs = T * k
    words, max_tiles = kern.moe_plan_sizes(n_pairs, E, bm)
    plan = torch.empty(words, device=DEV, dtype=torch.int32)
    sorted_pair = torch.empty(n_pairs, device=DEV, dtype=torch.int32)
    te = torch.empty(max_tiles, device=DEV, dtype=torch.int32)
    tr = torch.empty(max_tiles, device=DEV, dtype=torch.int32)
    st = kern.new_status(DEV)
    kern.moe_plan(idx, E, bm, plan, sorted_pair, te, tr, st)
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    assert plan[:E].tolist() == counts.tolist()
    assert sorted(sorted_pair.tolist()) == list(range(n_pairs))
    flat = idx.flatten()
    assert all(int(flat[p]) <= int(flat[q]) for p, q in zip(sorted_pair.tolist(), sorted_pair.tolist()[1:]))
    act = torch.empty(n_pairs, I, device=DEV, dtype=dtype)
    y = torch.full((T, k, H), float("nan"), device=DEV)
    if path == "simt":
        kern.moe_grouped_simt(1, x, w13, act, sorted_pair, pw, plan, te, tr, E, k)
        kern.moe_grouped_simt(2, act, w2, y.view(n_pairs, H), sorted_pair, pw.view(-1), plan, te, tr, E, k)
    elif path == "tc":
        xg = torch.empty(n_pairs, H, device=DEV, dtype=dtype)
        kern.gather_rows(x, xg, sorted_pair, k)
        assert torch.equal(xg, x[(sorted_pair // k).long()])
        kern.expert_gemm_tc(1, xg, w13, act, sorted_pair, pw.view(-1), plan, te, tr, E, bm, st)
        kern.expert_gemm_tc(2, act, w2, y.view(n_pairs, H), sorted_pair, pw.view(-1), plan, te, tr, E, bm, st)
        torch.cuda.synchronize()
        assert st.tolist()[0] == 0, f"device status {st.tolist()}"
    xf = x.float()
    want = torch.empty(T, k, H, device=DEV)
    for t in range(T):
        for s in range(k):
            e = int(idx[t, s])
            g = xf[t] @ w13[e, :I].float().T
            u = xf[t] @ w13[e, I:].float().T
            a = (g * torch.sigmoid(g) * u).to(dtype).float()
            want[t, s] = pw[t, s] * (a @ w2[e].float().T)
    assert torch.allclose(y, want, **tol(dtype))
    assert int(st[0]) == 0


@pytest.mark.parametrize("T,in_kernel_gather", [(1, True), (8, True), (8, False), (64, True), (300, False), (300, True),
                                                (2048, False), (2048, True), (4096, False), (4096, True)])
def test_expert_products_at_the_full_widths(T, in_kernel_gather):
    """Hidden 3072, experts of width 1536, 256 experts with 8 chosen: the launch geometry of the full-size
    model (24 and 24 blocks of 128 features a tile, token tiles of 16 to 256 rows, rings of several stages; from
    128-row tiles on the down product takes two blocks of 128 features a block), with the token rows fetched by
    the kernel (one TMA box a row, steps of at most 64 tokens) and from a gathered copy.  4,096 tokens: 128 rows
    an expert, tiles of 256 rows.  Against float32 products taken expert by expert."""
    kern = K()
    H, I, E, k = 3072, 1536, 256, 8
    torch.manual_seed(T)
    x = torch.randn(T, H, device=DEV).bfloat16()
    w13 = torch.empty(E, 2 * I, H, device=DEV, dtype=torch.bfloat16).normal_(0, H ** -0.5)
    w2 = torch.empty(E, H, I, device=DEV, dtype=torch.bfloat16).normal_(0, I ** -0.5)
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    if T >= 300:
        # one expert with more rows than a token tile holds: half the tokens choose expert 77 first
        others = torch.stack([torch.randperm(E - 1, device=DEV)[: k - 1] for _ in range(T // 2)]).int()
        idx[: T // 2, 0] = 77
        idx[: T // 2, 1:] = others + (others >= 77).int()
    pw = torch.rand(T, k, device=DEV)
    n_pairs = T * k
    bm = kern.expert_tile_rows(T, n_pairs / E)
    assert bm == {1: 16, 8: 16, 64: 64, 300: 128, 2048: 128, 4096: 256}[T]
    words, max_tiles = kern.moe_plan_sizes(n_pairs, E, bm)
    plan = torch.empty(words, device=DEV, dtype=torch.int32)
    sorted_pair = torch.empty(n_pairs, device=DEV, dtype=torch.int32)
    te = torch.empty(max_tiles, device=DEV, dtype=torch.int32)
    tr = torch.empty(max_tiles, device=DEV, dtype=torch.int32)
    st = kern.new_status(DEV)
    kern.moe_plan(idx, E, bm, plan, sorted_pair, te, tr, st)
    act = torch.full((n_pairs, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    y = torch.full((T, k, H), float("nan"), device=DEV)
    if in_kernel_gather:
        kern.expert_gemm_tc(1, x, w13, act, sorted_pair, pw.view(-1), plan, te, tr, E, bm, st, gather_top_k=k)
    else:
        xg = torch.empty(n_pairs, H, device=DEV, dtype=torch.bfloat16)
        kern.gather_rows(x, xg, sorted_pair, k)
        kern.expert_gemm_tc(1, xg, w13, act, sorted_pair, pw.view(-1), plan, te, tr, E, bm, st)
    kern.expert_gemm_tc(2, act, w2, y.view(n_pairs, H), sorted_pair, pw.view(-1), plan, te, tr, E, bm, st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0, f"device status {st.tolist()}"
    torch.backends.cuda.matmul.allow_tf32 = False
    want = torch.empty(T, k, H, device=DEV)
    want_act = torch.empty(T, k, I, device=DEV)
    xf = x.float()
    for e in idx.unique().tolist():
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        g = xf[tok] @ w13[e, :I].float().T
        u = xf[tok] @ w13[e, I:].float().T
        a = (g * torch.sigmoid(g) * u).bfloat16().float()
        want_act[tok, slot] = a
        want[tok, slot] = pw[tok, slot][:, None] * (a @ w2[e].float().T)
    got_act = torch.empty_like(want_act)
    got_act.view(n_pairs, I)[sorted_pair.long()] = act.float()
    assert torch.allclose(got_act, want_act, **tol(torch.bfloat16))
    assert torch.allclose(y, want, **tol(torch.bfloat16))


def test_sampling_matches_plain():
    kern = K()
    import numpy as np
    V, n = 1003, 12
    torch.manual_seed(4)
    logits = (3 * torch.randn(n, V)).float()
    logits[2, 100] = logits[2, 7] = 50.0                    # greedy tie: first index
    cases = [dict(temperature=0.0), dict(temperature=0.8, seed=1), dict(temperature=0.0),
             dict(temperature=1.3, seed=2 ** 40 + 17), dict(temperature=0.7, top_k=5, seed=3),
             dict(temperature=1.0, top_p=0.6, seed=4), dict(temperature=1.0, min_p=0.2, seed=5),
             dict(temperature=0.9, top_k=50, top_p=0.8, min_p=0.05, seed=6), dict(temperature=2.0, top_k=1, seed=7),
             dict(temperature=1.0, top_p=0.999, seed=8), dict(temperature=0.5, seed=9), dict(temperature=1.0, top_k=V + 5, seed=10)]
    # the rows' options live in state records; the rows use the slots in a scrambled order
    row_slot = torch.tensor([5, 0, 11, 3, 9, 1, 14, 2, 7, 12, 4, 8], dtype=torch.int32)
    for draw in (0, 1, 77):
        slots = torch.zeros(16, kern.SLOT_WORDS, dtype=torch.int32)
        for r, c in enumerate(cases):
            slots[row_slot[r]] = kern.slot_record(drawn=draw, position=r, **c)
        slots, out = slots.to(DEV), torch.empty(n, dtype=torch.int32, device=DEV)
        before = slots.clone()
        kern.sample_rows(logits.to(DEV), slots, row_slot.to(DEV), out)
        for r, c in enumerate(cases):
            want = P.sample(logits[r].numpy(), draw=draw, **c)
            if int(out[r]) != want:
                # only a near tie of (logit + noise) may differ: the kept sets of top-k and top-p are
                # exact (integer histograms), the noise is float32 on both sides
                lg = logits[r].numpy() * np.float32(1 / c["temperature"]) + P.gumbel_noise(c["seed"], draw, V)
                assert abs(lg[int(out[r])] - lg[want]) < 1e-5, (r, draw, c)
        # the kernel counted the draw and left the token in the record, and touched nothing else
        rows = row_slot.long().to(DEV)
        assert slots[rows, kern.SLOT_DRAWN].tolist() == [draw + 1] * n
        assert slots[rows, kern.SLOT_LAST].tolist() == out.tolist()
        before[rows, kern.SLOT_DRAWN] += 1
        before[rows, kern.SLOT_LAST] = out
        assert torch.equal(slots, before)
        again = torch.empty_like(out)                # the same row twice: the same token (nothing depends on order)
        slots[rows, kern.SLOT_DRAWN] -= 1
        kern.sample_rows(logits.to(DEV), slots, row_slot.to(DEV), again)
        assert torch.equal(again, out)
    greedy = torch.empty(n, dtype=torch.int32, device=DEV)
    kern.sample_rows(logits.to(DEV), None, None, greedy)
    assert greedy.tolist() == logits.argmax(-1).tolist() and int(greedy[2]) == 7


def test_sampling_distribution_and_penalties():
    kern = K()
    import numpy as np
    p = torch.tensor([0.5, 0.25, 0.15, 0.1])
    n = 4000
    logits = torch.log(p).repeat(n, 1).to(DEV)
    slots = torch.stack([kern.slot_record(temperature=1.0, seed=11, drawn=d) for d in range(n)]).to(DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    kern.sample_rows(logits, slots, torch.arange(n, dtype=torch.int32, device=DEV), out)
    freq = torch.bincount(out.long().cpu(), minlength=4).float() / n
    assert float((freq - p).abs().max()) < 0.03
    want = [P.sample(torch.log(p).numpy(), temperature=1.0, seed=11, draw=d) for d in range(50)]
    assert out[:50].tolist() == want
    lg = torch.tensor([[2.0, -2.0, 1.0, 0.5], [1.0, 1.0, 1.0, 1.0]], device=DEV)
    prev = torch.tensor([0, 1, 1, 3], dtype=torch.int32, device=DEV)
    off = torch.tensor([0, 3, 4], dtype=torch.int32, device=DEV)
    pp = torch.tensor([[2.0, 0.5, 0.25], [1.0, 0.0, 0.0]], device=DEV)
    kern.apply_penalties(lg, prev, off, pp)
    w0 = P.apply_penalties(np.array([2.0, -2.0, 1.0, 0.5], dtype=np.float32), [0, 1, 1], 2.0, 0.5, 0.25)
    assert np.allclose(lg[0].cpu().numpy(), w0) and lg[1].tolist() == [1.0] * 4


def test_greedy_over_a_large_vocabulary():
    """Rows cut over many blocks still give the first maximum."""
    kern = K()
    V, n = 200064, 5
    torch.manual_seed(6)
    logits = torch.randn(n, V, device=DEV)
    logits[1, 150000] = logits[1, 7] = logits[1, 199999] = 9.0         # a tie across chunks: the lowest index wins
    logits[2, V - 1] = 11.0
    logits[3, 0] = 12.0
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    kern.sample_rows(logits, None, None, out)
    assert out.tolist()[1:4] == [7, V - 1, 0]
    for r in (0, 4):
        assert int(out[r]) == int(logits[r].argmax())          # no ties in a random row
    # with state records whose temperature is 0 the same tokens come out, by either kernel, and are recorded
    slots = torch.stack([kern.slot_record(drawn=3) for _ in range(n)]).to(DEV)
    rows = torch.arange(n, dtype=torch.int32, device=DEV)
    for all_greedy in (True, False):
        got = torch.empty_like(out)
        kern.sample_rows(logits, slots, rows, got, all_greedy=all_greedy)
        assert torch.equal(got, out) and torch.equal(slots[:, kern.SLOT_LAST], out)
    assert slots[:, kern.SLOT_DRAWN].tolist() == [5] * n
