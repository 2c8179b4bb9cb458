"""Attention over long contexts: requests of more than 2,048 pages (the kernels for prompt portions then
read page ids from global memory instead of a shared-memory copy), portions that start past key 32,768,
single tokens over 131,072 keys (a (token, kv head) pair cut into many segments that a second step merges),
and one engine replay of a request of more than 9,000 tokens against the plain implementation on the GPU
(prompt portions of 1,024, as the reference feeds long prompts in chunks,
src/quanta/minimax/runtime_m3.py:190-259, then 64 single tokens).

The per-token Python reference of the kernel tests is too slow here; the reference below is the same
arithmetic vectorised in float32 on the GPU: gather a request's keys through its block table, scores
``q.k * scale``, mask by position (and window), softmax, ``P V``.  One key in the request's FIRST page is
made to dominate for some query rows, so a kernel that loses the far end of a long context is far off.
"""

import pytest
import torch

from tests import helpers as H
from tests.conftest import TINY
from tests.plain import minimax_m3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(atol=2e-2, rtol=2e-2)


def K():
    from quanta_b200 import kernels
    return kernels


def reference(q, kc, vc, table, tok_pos, tok_req, scale, window=0):
    """float32 attention of every token over its request's cached keys ``[0, pos]`` (or the window)."""
    T, nq, hd = q.shape
    nkv, page = kc.shape[1], kc.shape[2]
    out = torch.empty(T, nq, hd, device=q.device)
    for r in tok_req.unique().tolist():
        rows = torch.nonzero(tok_req == r).flatten().to(q.device)
        pos = tok_pos[rows.cpu()].to(q.device).long()
        L = int(pos.max()) + 1
        pages = table[r, : -(-L // page)].to(q.device).long()
        ks = kc[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].float()      # [nkv, L, hd]
        vs = vc[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].float()
        qr = q[rows].float().view(len(rows), nkv, nq // nkv, hd)
        s = torch.einsum("tgjd,gld->gjtl", qr, ks) * scale                           # [nkv, G, n, L]
        keys = torch.arange(L, device=q.device)
        mask = keys[None, :] <= pos[:, None]
        if window:
            mask &= keys[None, :] > pos[:, None] - window
        s = s.masked_fill(~mask, float("-inf"))
        o = torch.einsum("gjtl,gld->tgjd", torch.softmax(s, dim=-1), vs)
        out[rows] = o.reshape(len(rows), nq, hd)
    return out


def _cache(n_req, length, nkv, hd, page, seed):
    g = torch.Generator().manual_seed(seed)
    max_pages = -(-length // page)
    num_pages = n_req * max_pages + 5
    table = torch.randperm(num_pages, generator=g)[: n_req * max_pages].to(torch.int32).view(n_req, max_pages)
    torch.manual_seed(seed)
    kc = torch.randn(num_pages, nkv, page, hd, device=DEV).bfloat16()
    vc = torch.randn(num_pages, nkv, page, hd, device=DEV).bfloat16()
    return table, kc, vc


def _far_key(kc, table, req, key, page, gain=30.0):
    """Key ``key`` of request ``req`` points along dimension 0 with a large norm."""
    pg, sl = int(table[req, key // page]), key % page
    kc[pg, :, sl] = 0
    kc[pg, :, sl, 0] = gain
    return pg, sl


@pytest.mark.parametrize("impl", ["tc", "mma_only"])
@pytest.mark.parametrize("page,first,n", [(4, 8900, 200), (16, 33000, 130)])
def test_portion_of_a_request_with_more_than_2048_pages(impl, page, first, n, monkeypatch):
    """page 4 x 9,100 keys = 2,275 pages; page 16 from key 33,000 on = 2,071 pages."""
    k = K()
    nq, nkv, hd = 4, 2, 128
    assert k.attn_span_tc_supported(nq, nkv, hd, page)
    if impl == "mma_only":
        monkeypatch.setenv("QUANTA_B200_SPAN_KERNEL", "mma")
    length = first + n
    assert -(-length // page) > 2048
    table, kc, vc = _cache(1, length, nkv, hd, page, seed=page)
    q = torch.randn(n, nq, hd, device=DEV).bfloat16()
    pg, sl = _far_key(kc, table, 0, 2, page)                 # in the first page of the request
    q[::3, :, 0] = 8.0                                       # every third token looks along it
    tok_pos = torch.arange(first, length, dtype=torch.int32)
    tok_req = torch.zeros(n, dtype=torch.int32)
    out = torch.full_like(q, float("nan"))
    st = k.new_status(DEV)
    G = nq // nkv
    tiles = [[0, 0, n, x] for x in range(0, n * G, k.attn_span_rows(hd, nq, nkv, page))]
    k.attn_span(q, kc, vc, out, tok_pos.to(DEV), table.to(DEV), torch.tensor(tiles, dtype=torch.int32, device=DEV),
                hd ** -0.5, 0, st)
    assert int(st[0]) == 0
    want = reference(q, kc, vc, table, tok_pos, tok_req, hd ** -0.5)
    assert torch.allclose(out.float(), want, **TOL)
    assert torch.allclose(out[0, 0].float(), vc[pg, 0, sl].float(), atol=0.05)       # the far key carried that row


@pytest.mark.parametrize("batch,length,page,nq,nkv,hd", [(1, 131072, 16, 6, 1, 128), (4, 131072, 16, 6, 1, 128),
                                                         (2, 9100, 4, 4, 2, 128), (3, 40000, 16, 8, 2, 64)])
def test_single_tokens_over_long_contexts(batch, length, page, nq, nkv, hd):
    """Contexts so long that every (token, kv head) pair is cut into many segments over the blocks; the
    requests differ in length so that the cuts fall differently in each."""
    k = K()
    table, kc, vc = _cache(batch, length, nkv, hd, page, seed=batch + page)
    lengths = [length - 37 * r * r for r in range(batch)]
    q = torch.randn(batch, nq, hd, device=DEV).bfloat16()
    pg, sl = _far_key(kc, table, 0, 1, page)
    q[0, : nq // 2, 0] = 8.0                                  # half the heads of the first request look along it
    tok_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    tok_req = torch.arange(batch, dtype=torch.int32)
    out = torch.full_like(q, float("nan"))
    n_parts = k.attn_decode_parts(nkv, length)
    po = torch.full((batch * nq * n_parts * hd,), float("nan"), device=DEV)
    pml = torch.full((batch * nq * n_parts * 2,), float("nan"), device=DEV)
    st = k.new_status(DEV)
    k.attn_decode(q, kc, vc, out, po, pml, torch.arange(batch, dtype=torch.int32, device=DEV), batch, tok_pos.to(DEV),
                  tok_req.to(DEV), table.to(DEV), hd ** -0.5, 0, n_parts, st)
    assert int(st[0]) == 0
    want = reference(q, kc, vc, table, tok_pos, tok_req, hd ** -0.5)
    assert torch.allclose(out.float(), want, **TOL)
    assert torch.allclose(out[0, 0].float(), vc[pg, 0, sl].float(), atol=0.05)
    # random keys over 131,072 positions average out: the other heads' rows are small but not zero
    assert float(out[0, nq - 1].float().abs().max()) < 0.2


def test_float32_kernel_over_a_long_context():
    """The float32 kernel with the same inputs (portion and single token, more than 2,048 pages)."""
    k = K()
    nq, nkv, hd, page, first, n = 4, 2, 64, 4, 9000, 40
    length = first + n
    table, kc, vc = _cache(2, length, nkv, hd, page, seed=9)
    kc, vc = kc.float(), vc.float()
    q = torch.randn(n + 1, nq, hd, device=DEV)
    pg, sl = _far_key(kc, table, 0, 3, page)
    q[0, :, 0] = 8.0
    tok_pos = torch.tensor(list(range(first, length)) + [length - 1], dtype=torch.int32)
    tok_req = torch.tensor([0] * n + [1], dtype=torch.int32)
    out = torch.full_like(q, float("nan"))
    st = k.new_status(DEV)
    k.paged_attention_simt(q, kc, vc, out, tok_pos.to(DEV), tok_req.to(DEV), table.to(DEV), hd ** -0.5, 0, st)
    assert int(st[0]) == 0
    want = reference(q, kc, vc, table, tok_pos, tok_req, hd ** -0.5)
    assert torch.allclose(out, want, atol=2e-5, rtol=2e-5)
    assert torch.allclose(out[0, 0], vc[pg, 0, sl], atol=0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_replay_of_a_long_request(model_dirs, plain_models, dtype):
    """Configuration D (head size 128, the tensor-core kernels of the full-size model): 9,300 tokens, page
    size 4 so that the request holds more than 2,048 pages, fed in portions of 1,024 and then 64 single
    tokens, beside a short request that shares the steps; logits at every 50th place and at all the single
    tokens against the plain implementation on the GPU."""
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.step import Engine
    name, n, tail, page = "D", 9300, 64, 4
    vocab = TINY[name]["vocab_size"]
    reqs = {"long": H.random_tokens(n, vocab, seed=501), "short": H.random_tokens(90, vocab, seed=502)}
    weights, cfg = plain_models[name]
    on_gpu = {k_: v.to(DEV) for k_, v in weights.items()}
    places = {"long": sorted(set(range(0, n - tail, 50)) | set(range(n - tail, n))), "short": list(range(0, 90, 7))}

    def plain(act):
        rids = list(reqs)
        with torch.no_grad():
            out = P.forward_logits_many(on_gpu, cfg, [reqs[r] for r in rids], rows=[places[r] for r in rids], act=act)
        return {(rid, p): out[i][j] for i, rid in enumerate(rids) for j, p in enumerate(places[rid])}

    exact = plain(None)
    want = exact if dtype == "float32" else plain(torch.bfloat16)
    tol = 2e-5 if dtype == "float32" else 2.0 * max(float((want[k_] - exact[k_]).abs().max()) for k_ in want)
    steps, fed = [], 0
    while fed < n - tail:
        m = min(1024, n - tail - fed)
        entries = [{"id": "long", "tokens": reqs["long"][fed:fed + m], "want": list(range(m))}]
        if fed == 2048:          # the short request's prompt shares a step with a portion of the long one
            entries.append({"id": "short", "tokens": reqs["short"][:60], "want": list(range(60))})
        steps.append({"entries": entries, "end": []})
        fed += m
    for i in range(tail):        # single tokens; the short request decodes beside the first 30 of them
        entries = [{"id": "long", "tokens": [reqs["long"][n - tail + i]], "want": [0]}]
        if i < 30:
            entries.append({"id": "short", "tokens": [reqs["short"][60 + i]], "want": [0]})
        steps.append({"entries": entries, "end": (["short"] if i == 29 else []) + (["long"] if i == tail - 1 else [])})
    keep = {rid: set(p) for rid, p in places.items()}
    seen = {}
    for s in steps:              # ask only for the compared places
        for e in s["entries"]:
            base = seen.get(e["id"], 0)
            e["want"] = [w for w in e["want"] if base + w in keep[e["id"]]]
            seen[e["id"]] = base + len(e["tokens"])
    model, _ = load_model(model_dirs[name], dtype=dtype)
    eng = Engine(model, num_pages=H.tokens_in_flight(steps, page) // page, page_size=page, max_requests=4)
    got = H.replay(eng, steps)
    assert eng.manager.stats()["groups"][0]["high_water"] > 2048
    assert set(got) == set(want)
    worst = max(float((got[k_] - want[k_].cpu()).abs().max()) for k_ in got)
    bad = sorted((k_ for k_ in got if float((got[k_] - want[k_].cpu()).abs().max()) > tol), key=lambda k_: (k_[0], k_[1]))
    assert not bad, f"first wrong place {bad[0]}, worst error {worst:.3e}, tolerance {tol:.3e}"
