"""Times single kernels of the engine on synthetic inputs, one JSON line a case.

    python bench_kernels.py attn_decode  --batch 4 --context 131072
    python bench_kernels.py attn_span    --tokens 8192 --start 122880
    python bench_kernels.py attn_sweep                      # the cases quoted under profiles/
    python bench_kernels.py router       --tokens 2048      # router logits + selection of a prompt portion
    python bench_kernels.py experts      --tokens 8         # routed experts of one layer: plan, gather, two products

Shapes default to the M2-family attention (48 q heads, 8 kv heads of 128, pages of 16 tokens).  Caches
are random, pages are dealt in a random order, every request of a decode case has the same context.
Times are medians of CUDA-event intervals around one call, after warm-up; inputs are larger than L2
except in the smallest cases, which say so by their size.  ``GB/s`` counts the keys and values read
once; ``TFLOP/s`` counts 4 * head_dim flops per (query head, visible key).
"""

from __future__ import annotations

import argparse
import json

import torch

from quanta_b200 import kernels as k

DEV = "cuda:0"


def timed(fn, n: int = 10, warm: int = 3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def timed_graph(fn, reps: int = 20) -> float:
    """Median time of one call, ``reps`` calls captured back to back in a CUDA graph: the kernel's own
    time for kernels that are shorter than the host's launch path."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    return timed(g.replay) / reps


def attn_decode(batch: int, context: int, nq: int, nkv: int, hd: int, page: int) -> dict:
    """One new token of ``batch`` requests against ``context`` cached keys each.  As in a decode step, every
    call reads another layer's cache (as many layers as fit 6 GB, at most 16), and the calls are captured back
    to back in a CUDA graph: the time is the kernel's own, cold in L2, without the host's launch path."""
    max_pages = -(-context // page)
    num_pages = batch * max_pages
    per_layer = 2 * num_pages * nkv * page * hd * 2
    layers = max(1, min(16, int(6e9 // per_layer)))
    table = torch.randperm(num_pages, dtype=torch.int32).view(batch, max_pages).to(DEV)
    caches = [(torch.randn(num_pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16),
               torch.randn(num_pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)) for _ in range(layers)]
    q = torch.randn(batch, nq, hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    tok_pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    tok_req = torch.arange(batch, dtype=torch.int32, device=DEV)
    dec = torch.arange(batch, dtype=torch.int32, device=DEV)
    st = k.new_status(DEV)
    n_parts = k.attn_decode_parts(nkv, context)
    po = torch.empty(batch * nq * n_parts * hd, device=DEV)
    pml = torch.empty(batch * nq * n_parts * 2, device=DEV)

    def step():
        for kc, vc in caches:
            k.attn_decode(q, kc, vc, out, po, pml, dec, batch, tok_pos, tok_req, table, hd ** -0.5, 0, n_parts, st)

    ms = timed_graph(step, reps=2) / layers
    k.raise_on_status(st.cpu())
    gb = batch * context * nkv * hd * 2 * 2 / 1e9
    return {"kernel": "attn_decode", "batch": batch, "context": context, "q_heads": nq, "kv_heads": nkv,
            "head_dim": hd, "page": page, "layers": layers, "us": round(ms * 1e3, 1), "kv_gb": round(gb, 3),
            "GB/s": round(gb / ms * 1e3, 1)}


def attn_span(tokens: int, start: int, nq: int, nkv: int, hd: int, page: int) -> dict:
    """A portion of ``tokens`` prompt tokens of one request whose cache already holds ``start`` keys."""
    max_pages = -(-(start + tokens) // page)
    table = torch.randperm(max_pages, dtype=torch.int32).view(1, -1).to(DEV)
    kc = torch.randn(max_pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn(max_pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    q = torch.randn(tokens, nq, hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    tok_pos = torch.arange(start, start + tokens, dtype=torch.int32, device=DEV)
    group = nq // nkv
    rows = k.attn_span_rows(hd, nq, nkv, page)
    tiles = [[0, 0, tokens, r0] for r0 in range(0, tokens * group, rows)]
    tiles.reverse()                       # the tiles that read the most keys first, as the engine orders them
    tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    st = k.new_status(DEV)
    ms = timed(lambda: k.attn_span(q, kc, vc, out, tok_pos, table, tiles, hd ** -0.5, 0, st))
    k.raise_on_status(st.cpu())
    keys = sum(range(start + 1, start + tokens + 1))
    flops = 4.0 * hd * nq * keys
    return {"kernel": "attn_span", "tcgen05": bool(k.attn_span_tc_supported(nq, nkv, hd, page)), "tokens": tokens,
            "start": start, "q_heads": nq, "kv_heads": nkv, "head_dim": hd, "page": page, "ms": round(ms, 4),
            "TFLOP/s": round(flops / ms / 1e9, 1)}


def router(tokens: int, hidden: int, experts: int, top_k: int) -> dict:
    """The router of a step of ``tokens`` tokens, timed as twenty launches in a CUDA graph: below 256 tokens
    one kernel (float32 logits on the CUDA cores, selection, expert plan); from 256 on the logits on the tensor
    cores (float32 gate in three bfloat16 pieces) and the selection."""
    x = torch.randn(tokens, hidden, device=DEV).bfloat16()
    gate = torch.randn(experts, hidden, device=DEV) / hidden ** 0.5
    if tokens < 256 and k.router_small_selects(tokens, experts, top_k):
        # what a small step runs: float32 logits on the CUDA cores, selection and the expert plan, one launch
        logits = torch.empty(tokens, experts, device=DEV)
        bias = torch.zeros(experts, device=DEV)
        idx = torch.empty(tokens, top_k, dtype=torch.int32, device=DEV)
        w = torch.empty(tokens, top_k, device=DEV)
        bm = k.expert_tile_rows(tokens, tokens * top_k / experts)
        words, max_tiles = k.moe_plan_sizes(tokens * top_k, experts, bm)
        plan = torch.empty(words, dtype=torch.int32, device=DEV)
        sp = torch.empty(tokens * top_k, dtype=torch.int32, device=DEV)
        te, tr = (torch.empty(max_tiles, dtype=torch.int32, device=DEV) for _ in range(2))
        counters, st = torch.zeros(1 + -(-tokens // 8), dtype=torch.int32, device=DEV), k.new_status(DEV)
        t_logits = timed_graph(lambda: k.router_small(x, gate, bias, logits))
        t_all = timed_graph(lambda: k.router_small(x, gate, bias, logits, idx, w, True, 1.0, counters=counters, bm=bm,
                                                   plan=plan, sorted_pair=sp, tile_expert=te, tile_row0=tr, status=st))
        return {"kernel": "router_small", "tokens": tokens, "hidden": hidden, "experts": experts, "top_k": top_k,
                "logits_only_us": round(t_logits * 1e3, 1), "logits_selection_plan_us": round(t_all * 1e3, 1)}
    pieces = k.split3_bf16(gate)
    logits = torch.empty(k.router_gemm_mma_parts(hidden), tokens, experts, device=DEV)
    bias = torch.zeros(experts, device=DEV)
    idx = torch.empty(tokens, top_k, dtype=torch.int32, device=DEV)
    w = torch.empty(tokens, top_k, device=DEV)
    t_gemm = timed_graph(lambda: k.router_gemm_mma(x, pieces, logits))
    t_sel = timed_graph(lambda: k.router_topk(logits, bias, idx, w, True, 1.0))
    flops = 2.0 * 3 * tokens * experts * hidden
    return {"kernel": "router_gemm_mma + router_topk", "tokens": tokens, "hidden": hidden, "experts": experts,
            "top_k": top_k, "gemm_us": round(t_gemm * 1e3, 1), "gemm_TFLOP/s": round(flops / t_gemm / 1e9, 1),
            "topk_us": round(t_sel * 1e3, 1)}


def experts(tokens: int, hidden: int, width: int, n_experts: int, top_k: int, even: bool = False) -> dict:
    """The routed experts of one layer for a step of ``tokens`` tokens (random routing, a fresh one each
    call so that no call finds its experts in L2): expert plan, row gather and the two tcgen05 products, each
    timed as launches in a CUDA graph.  ``GB/s`` counts the weights of the distinct experts once, ``TFLOP/s``
    the multiply-adds of the rows.  ``even``: every expert gets the same number of rows (no ragged last tiles)."""
    w13 = torch.empty(n_experts, 2 * width, hidden, device=DEV, dtype=torch.bfloat16).normal_(0, 0.02)
    w2 = torch.empty(n_experts, hidden, width, device=DEV, dtype=torch.bfloat16).normal_(0, 0.02)
    n_pairs, st = tokens * top_k, k.new_status(DEV)
    bm = k.expert_tile_rows(tokens, n_pairs / n_experts)
    plan_words, max_tiles = k.moe_plan_sizes(n_pairs, n_experts, bm)
    sets, distinct = [], []
    for i in range(4):
        x = torch.randn(tokens, hidden, device=DEV).bfloat16()
        if even:
            idx = ((torch.arange(tokens, device=DEV)[:, None] * top_k + torch.arange(top_k, device=DEV)[None, :] + i)
                   % n_experts).int()
        else:
            idx = torch.stack([torch.randperm(n_experts, device=DEV)[:top_k] for _ in range(tokens)]).int()
        w = torch.rand(tokens, top_k, device=DEV)
        plan = torch.empty(plan_words, dtype=torch.int32, device=DEV)
        sp = torch.empty(n_pairs, dtype=torch.int32, device=DEV)
        te, tr = (torch.empty(max_tiles, dtype=torch.int32, device=DEV) for _ in range(2))
        xg = torch.empty(n_pairs, hidden, device=DEV, dtype=torch.bfloat16)
        act = torch.empty(n_pairs, width, device=DEV, dtype=torch.bfloat16)
        y = torch.empty(n_pairs, hidden, device=DEV)
        k.moe_plan(idx, n_experts, bm, plan, sp, te, tr, st)
        k.gather_rows(x, xg, sp, top_k)
        sets.append((x, idx, w, plan, sp, te, tr, xg, act, y))
        distinct.append(int(idx.unique().numel()))
    calls = {
        "plan": lambda s: k.moe_plan(s[1], n_experts, bm, s[3], s[4], s[5], s[6], st),
        "gather": lambda s: k.gather_rows(s[0], s[7], s[4], top_k),
        "up": lambda s: k.expert_gemm_tc(1, s[7], w13, s[8], s[4], s[2].view(-1), s[3], s[5], s[6], n_experts, bm, st),
        "down": lambda s: k.expert_gemm_tc(2, s[8], w2, s[9], s[4], s[2].view(-1), s[3], s[5], s[6], n_experts, bm, st),
    }
    if tokens <= 1024:    # what steps of few rows an expert run: no gathered copy, the kernel fetches each pair's token row
        calls["up_fetching_rows"] = lambda s: k.expert_gemm_tc(1, s[0], w13, s[8], s[4], s[2].view(-1), s[3], s[5], s[6],
                                                               n_experts, bm, st, gather_top_k=top_k)
    out = {"kernel": "moe_plan + gather_rows + expert_gemm_tc", "tokens": tokens, "hidden": hidden, "width": width,
           "experts": n_experts, "top_k": top_k, "tile_rows": bm, "distinct_experts": round(sum(distinct) / 4, 1)}
    for name, fn in calls.items():
        def four(fn=fn):
            for s in sets:
                fn(s)
        out[f"{name}_us"] = round(timed_graph(four, reps=5) / 4 * 1e3, 1)
    gb = sum(distinct) / 4 * hidden * width * 2 / 1e9
    out["up_GB/s"] = round(2 * gb / (out["up_us"] * 1e-6), 0)
    out["down_GB/s"] = round(gb / (out["down_us"] * 1e-6), 0)
    tf = 2.0 * n_pairs * hidden * width / 1e12
    out["up_TFLOP/s"] = round(2 * tf / (out["up_us"] * 1e-6), 0)
    out["down_TFLOP/s"] = round(tf / (out["down_us"] * 1e-6), 0)
    assert int(st[0]) == 0
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["attn_decode", "attn_span", "attn_sweep", "router", "experts"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--start", type=int, default=0)
    ap.add_argument("--q-heads", type=int, default=48)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=3072)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--width", type=int, default=1536, help="inner size of an expert")
    ap.add_argument("--even-routing", action="store_true", help="experts: the same number of rows for every expert")
    a = ap.parse_args()
    shape = (a.q_heads, a.kv_heads, a.head_dim, a.page)
    if a.what == "attn_decode":
        print(json.dumps(attn_decode(a.batch, a.context, *shape)), flush=True)
    elif a.what == "attn_span":
        print(json.dumps(attn_span(a.tokens, a.start, *shape)), flush=True)
    elif a.what == "experts":
        print(json.dumps(experts(a.tokens, a.hidden, a.width, a.experts, a.top_k, a.even_routing)), flush=True)
    elif a.what == "router":
        print(json.dumps(router(a.tokens, a.hidden, a.experts, a.top_k)), flush=True)
    else:
        for batch, context in [(1, 4096), (8, 4096), (64, 4096), (32, 16384), (8, 32768), (1, 131072), (4, 131072)]:
            print(json.dumps(attn_decode(batch, context, *shape)), flush=True)
            torch.cuda.empty_cache()
        for tokens, start in [(2048, 0), (8192, 0), (8192, 122880)]:
            print(json.dumps(attn_span(tokens, start, *shape)), flush=True)
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
