"""The decode attention entry point that allocates nothing (``qb_attn_decode_noalloc``).

Some users of the library's C ABI cannot hand the split-key decode attention the scratch memory it
wants: their host program gave the whole device to its own pool and treats a later ``cudaMalloc`` as
a failure, or they are a plug-in without a handle on that pool, or they sit in a loop where an
allocation may stall or fail.  For them the partial results live in a static device array inside the
library.  This test calls that entry point through its exported C symbol, twice in a row with
different inputs (the array keeps the first call's contents), and checks each output against the
existing entry point, which takes its scratch from the caller, and against plain float32 attention
computed here (two entry points that were wrong in the same way would else agree).  Two more cases
take paths of the static array's own: more single tokens than one launch of the kernel holds (the
second launch starts further into the array, and the merge step spans both), and a window.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process and after the other tests.
"""

import ctypes
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE = -3


def _plain(c, window=0):
    """float32 attention of each token over its request's keys, straight from the pages."""
    out = torch.empty(c["n"], c["nq"], c["hd"], device=DEV)
    G = c["nq"] // c["nkv"]
    for r in range(c["n"]):
        p = int(c["pos"][r])
        lo = max(0, p - window + 1) if window else 0
        pages = c["table"][r, : p // c["page"] + 1].long()
        ks = c["kc"][pages].permute(1, 0, 2, 3).reshape(c["nkv"], -1, c["hd"])[:, lo:p + 1].float()
        vs = c["vc"][pages].permute(1, 0, 2, 3).reshape(c["nkv"], -1, c["hd"])[:, lo:p + 1].float()
        qr = c["q"][r].float().view(c["nkv"], G, c["hd"])
        s = torch.einsum("gjd,gld->gjl", qr, ks) * c["hd"] ** -0.5
        out[r] = torch.einsum("gjl,gld->gjd", torch.softmax(s, -1), vs).reshape(c["nq"], c["hd"])
    return out


def _case(seed, contexts, nq=12, nkv=2, hd=128, page=16):
    """Single new tokens of len(contexts) requests whose caches hold ``contexts[i]`` keys."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = len(contexts)
    max_pages = max(-(-c // page) for c in contexts)
    num_pages = n * max_pages + 2
    ids = list(range(num_pages))
    random.Random(seed).shuffle(ids)
    table = torch.tensor([ids[r * max_pages:(r + 1) * max_pages] for r in range(n)], dtype=torch.int32)
    kc = torch.randn(num_pages, nkv, page, hd, generator=g).bfloat16()
    vc = torch.randn(num_pages, nkv, page, hd, generator=g).bfloat16()
    q = torch.randn(n, nq, hd, generator=g).bfloat16()
    pos = torch.tensor([c - 1 for c in contexts], dtype=torch.int32)
    req = torch.arange(n, dtype=torch.int32)
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV), pos=pos.to(DEV), req=req.to(DEV),
                dec=torch.arange(n, dtype=torch.int32, device=DEV), n=n, nq=nq, nkv=nkv, hd=hd, page=page,
                num_pages=num_pages, longest=max(contexts))


def _existing(k, c, window=0):
    """The entry point that takes its scratch from the caller."""
    n_splits = k.attn_decode_parts(c["nkv"], c["longest"])
    out = torch.full_like(c["q"], float("nan"))
    po = torch.empty(c["n"] * c["nq"] * n_splits * c["hd"], device=DEV)
    pml = torch.empty(c["n"] * c["nq"] * n_splits * 2, device=DEV)
    st = k.new_status(DEV)
    k.attn_decode(c["q"], c["kc"], c["vc"], out, po, pml, c["dec"], c["n"], c["pos"], c["req"], c["table"],
                  c["hd"] ** -0.5, window, n_splits, st)
    assert int(st[0]) == 0
    return out, n_splits


def _no_alloc(lib, c, n_splits, status, out, window=0):
    p = lambda t: ctypes.c_void_p(t.data_ptr())      # noqa: E731
    rc = lib.qb_attn_decode_noalloc(
        p(c["q"]), p(c["kc"]), p(c["vc"]), p(out), p(c["dec"]), c["n"], p(c["pos"]), p(c["req"]), p(c["table"]),
        c["table"].shape[1], c["nq"], c["nkv"], c["hd"], c["page"], c["num_pages"], ctypes.c_float(c["hd"] ** -0.5),
        int(window), n_splits, p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_no_alloc_entry_point_matches_the_existing_one_twice_in_a_row():
    from quanta_b200 import kernels as k
    lib = k.lib()
    lib.qb_attn_decode_noalloc_floats.restype = ctypes.c_longlong
    lib.qb_attn_decode_noalloc_capacity.restype = ctypes.c_longlong
    assert lib.qb_attn_decode_noalloc_capacity() == 2 * 1024 * 1024
    status = k.new_status(DEV)
    first = _case(1, [300, 70, 513])
    second = _case(2, [1025, 17, 256, 640])          # other sizes: the array still holds the first call's partials
    # 300 single tokens (one launch holds 256: the second starts further into the array) of short contexts
    many = _case(3, [1 + (37 * i) % 200 for i in range(300)], nq=4, nkv=2, hd=64)
    windowed = _case(4, [700, 90, 333])
    for case, window in ((first, 0), (second, 0), (many, 0), (windowed, 100)):
        want, n_splits = _existing(k, case, window)
        need = lib.qb_attn_decode_noalloc_floats(case["n"], case["nq"], case["hd"], n_splits)
        assert 0 < need <= lib.qb_attn_decode_noalloc_capacity()
        got = torch.full_like(case["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        rc, got = _no_alloc(lib, case, n_splits, status, got, window)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before        # nothing was taken from torch's allocator either
        assert int(status[0]) == 0
        assert not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)        # the same kernels in the same order: bit for bit
        assert torch.allclose(got.float(), _plain(case, window), atol=2e-2, rtol=2e-2)
    # a problem beyond the array is refused, and nothing is launched
    big = dict(first)
    too_many_splits = lib.qb_attn_decode_noalloc_capacity() // (first["n"] * first["nq"] * (first["hd"] + 2)) + 1
    rc, got = _no_alloc(lib, big, int(too_many_splits), status, torch.full_like(big["q"], float("nan")))
    torch.cuda.synchronize()
    assert rc == TOO_LARGE
    assert torch.isnan(got.float()).all()
