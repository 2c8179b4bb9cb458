"""Python face of the CUDA kernels: argument checks, pointers, launch on torch's current stream.

Every function here launches hand-written sm_100a code from ``csrc``; there is no CPU or library
fallback, and a missing or unbuildable extension raises at the first call.  Tensors must be CUDA,
contiguous and of the stated dtype; a violated precondition is a ``ValueError`` before anything is
launched.
"""

from __future__ import annotations

import ctypes
import os

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
NORM_NONE, NORM_PER_LAYER, NORM_PER_HEAD = 0, 1, 2

_STATUS_TEXT = {1: "token id outside the vocabulary", 2: "page id outside the pool (block table)",
                3: "expert id outside the expert table", 4: "a bounded device wait ran out",
                5: "the decode attention scratch has too few entries per row",
                6: "a request's state slot on the device is free or at another position than the host's record"}
_KERNEL_TEXT = {1: "embedding", 2: "rope/cache write", 3: "paged attention", 4: "expert plan",
                5: "expert product", 6: "decode attention", 7: "prefill attention", 8: "state slots"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    return _build.load()


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"dtype {t.dtype} is not float32 or bfloat16") from None


def _p(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ValueError("kernel arguments must be CUDA tensors")
    if not t.is_contiguous():
        raise ValueError("kernel arguments must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """torch's current stream of the current device, as a cudaStream_t."""
    if _raw_stream is not None:       # the same answer as below, without building a Stream object each launch
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0        # kernels of this library launched so far (a plain counter; reset it to count a region)


def _check(rc: int, what: str, n_kernels: int = 1) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += n_kernels
        return
    if rc == -1:
        raise ValueError(f"{what}: bad argument")
    if rc == -2:
        raise ValueError(f"{what}: a size outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {rc}")


def _want(t: torch.Tensor, dtype, name: str) -> None:
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def new_status(device) -> torch.Tensor:
    """Status words the kernels write when they meet an index they cannot honour."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def raise_on_status(status_host) -> None:
    code = int(status_host[0])
    if code:
        raise KernelError(f"device reported: {_STATUS_TEXT.get(code, code)} (value {int(status_host[1])}) in "
                          f"{_KERNEL_TEXT.get(int(status_host[2]), 'kernel ' + str(int(status_host[2])))}")


# ------------------------------------------------------------------------------------------------
def embedding(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor) -> None:
    _want(h, torch.float32, "h"); _want(ids, torch.int32, "ids")
    T, H = h.shape
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() != T:
        raise ValueError("embedding: shape mismatch")
    _check(lib().qb_embedding(_p(h), _p(table), _code(table), _p(ids), T, H, V, _p(status), _stream()),
           "embedding")


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor | None, rows: torch.Tensor | None = None, store_h: bool = True) -> None:
    """``h += sum_s delta[:, s]`` (float32) and ``out = weight * h * rsqrt(mean(h^2) + eps)``.

    ``delta`` is ``[T, H]`` or ``[T, S, H]`` or None; ``rows`` (int32) selects token rows, in which case
    ``out`` has one row per entry.  ``out`` None only folds the delta into ``h``."""
    _want(h, torch.float32, "h"); _want(weight, torch.float32, "weight")
    T, H = h.shape
    S = 1
    if delta is not None:
        if delta.dim() == 3:
            S = delta.shape[1]
        if delta.shape[0] != T or delta.shape[-1] != H:
            raise ValueError("add_rmsnorm: delta shape mismatch")
    n = T if rows is None else rows.numel()
    if rows is not None:
        _want(rows, torch.int32, "rows")
    if out is not None and (out.shape[0] != n or out.shape[1] != H):
        raise ValueError("add_rmsnorm: out shape mismatch")
    if weight.numel() != H:
        raise ValueError("add_rmsnorm: weight shape mismatch")
    _check(lib().qb_add_rmsnorm(_p(h), _p(delta), _code(delta) if delta is not None else F32, S, _p(weight),
                                _p(out), _code(out) if out is not None else F32, _p(rows), n, H,
                                ctypes.c_float(eps), int(store_h), _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    n, two_i = gate_up.shape
    if out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise ValueError("silu_mul: shape/dtype mismatch")
    _check(lib().qb_silu_mul(_p(gate_up), _p(out), _code(out), n, two_i // 2, _stream()), "silu_mul")


def qknorm_rope_write(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, norm_kind: int, eps: float,
                      inv_freq, pair_axis, positions, tok_pos, tok_req, block_table, nq: int, nkv: int,
                      hd: int, rd: int, page_size: int, status) -> None:
    T = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * hd:
        raise ValueError("qknorm_rope_write: qkv width mismatch")
    if q_out.dtype != qkv.dtype or q_out.numel() != T * nq * hd:
        raise ValueError("qknorm_rope_write: q_out mismatch")
    num_pages = 0
    if k_cache is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise ValueError("qknorm_rope_write: cache dtype differs from activations")
        if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape:
            raise ValueError("qknorm_rope_write: cache shape mismatch")
        num_pages = k_cache.shape[0]
    _want(inv_freq, torch.float32, "inv_freq")
    if inv_freq.numel() != rd // 2:
        raise ValueError("qknorm_rope_write: inv_freq length")
    n_axes = 1 if positions.dim() == 1 else positions.shape[1]
    for t, n in ((positions, "positions"), (tok_pos, "tok_pos"), (tok_req, "tok_req"), (block_table, "block_table")):
        _want(t, torch.int32, n)
    if pair_axis is not None:
        _want(pair_axis, torch.int32, "pair_axis")
    if norm_kind != NORM_NONE:
        want = (nq * hd, nkv * hd) if norm_kind == NORM_PER_LAYER else (hd, hd)
        if q_norm_w.numel() != want[0] or k_norm_w.numel() != want[1]:
            raise ValueError("qknorm_rope_write: norm weight length does not fit the norm kind")
    _check(lib().qb_qknorm_rope_write(
        _p(qkv), _code(qkv), _p(q_out), _p(k_cache), _p(v_cache), _p(q_norm_w), _p(k_norm_w), norm_kind,
        ctypes.c_float(eps), _p(inv_freq), _p(pair_axis), _p(positions), n_axes, _p(tok_pos), _p(tok_req),
        _p(block_table), block_table.shape[1], T, nq, nkv, hd, rd, page_size, num_pages, _p(status),
        _stream()), "qknorm_rope_write")


def paged_attention_simt(q, k_cache, v_cache, out, tok_pos, tok_req, block_table, scale: float,
                         window: int, status) -> None:
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    if hd2 != hd or out.shape != q.shape or out.dtype != q.dtype or k_cache.dtype != q.dtype:
        raise ValueError("paged_attention: shape/dtype mismatch")
    _check(lib().qb_paged_attention_simt(
        _p(q), _code(q), _p(k_cache), _p(v_cache), _p(out), _p(tok_pos), _p(tok_req), _p(block_table),
        block_table.shape[1], T, nq, nkv, hd, page_size, num_pages, ctypes.c_float(scale), int(window),
        _p(status), _stream()), "paged_attention_simt")


def attn_span_rows(hd: int, nq: int, nkv: int, page_size: int) -> int:
    """Query rows (token x head-of-group) per tile of the kernel that runs portions of these shapes."""
    return int(lib().qb_attn_span_rows(int(hd), int(nq), int(nkv), int(page_size)))


def attn_decode_parts(nkv: int, max_len: int) -> int:
    """Entries per (token, q head) row of the decode attention scratch for contexts of up to ``max_len`` keys."""
    n = int(lib().qb_attn_decode_parts(int(nkv), int(max_len)))
    if n < 2:
        raise KernelError(f"attn_decode_parts({nkv}, {max_len}) failed with code {n}")
    return n


ATTN_DECODE_MAX_GROUP = 64      # q heads per kv head that the decode kernel takes


def attn_span_tc_supported(nq: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether portions of these shapes run on the tcgen05 kernel (else on the mma.sync kernel)."""
    return bool(lib().qb_attn_span_tc_supported(int(nq), int(nkv), int(hd), int(page_size)))


def attn_span(q, k_cache, v_cache, out, tok_pos, block_table, tiles, scale: float, window: int, status) -> None:
    """bfloat16 tensor-core attention for prompt portions.  ``tiles`` int32 [n, 4]: request row, first
    token row of the portion, tokens in the portion, first flattened (token*G + head) row of the tile."""
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    _want(q, torch.bfloat16, "q"); _want(k_cache, torch.bfloat16, "k_cache"); _want(tiles, torch.int32, "tiles")
    if hd2 != hd or out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("attn_span: shape/dtype mismatch")
    _check(lib().qb_attn_span(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(tok_pos), _p(block_table),
                              block_table.shape[1], _p(tiles), tiles.shape[0], nq, nkv, hd, page_size, num_pages,
                              ctypes.c_float(scale), int(window), _p(status), _stream()), "attn_span")


def attn_decode(q, k_cache, v_cache, out, part_o, part_ml, dec_tok, n_dec: int, tok_pos, tok_req, block_table,
                scale: float, window: int, n_parts: int, status) -> None:
    """bfloat16 tensor-core attention for single tokens; ``part_o`` / ``part_ml`` are float32 scratch of
    at least n_dec*nq*n_parts*hd and n_dec*nq*n_parts*2 elements, ``n_parts`` from ``attn_decode_parts``."""
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    _want(q, torch.bfloat16, "q"); _want(k_cache, torch.bfloat16, "k_cache")
    _want(part_o, torch.float32, "part_o"); _want(part_ml, torch.float32, "part_ml"); _want(dec_tok, torch.int32, "dec_tok")
    if hd2 != hd or out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("attn_decode: shape/dtype mismatch")
    if part_o.numel() < n_dec * nq * n_parts * hd or part_ml.numel() < n_dec * nq * n_parts * 2:
        raise ValueError("attn_decode: scratch too small")
    _check(lib().qb_attn_decode(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_o), _p(part_ml), _p(dec_tok),
                                int(n_dec), _p(tok_pos), _p(tok_req), _p(block_table), block_table.shape[1], nq, nkv,
                                hd, page_size, num_pages, ctypes.c_float(scale), int(window), int(n_parts),
                                _p(status), _stream()), "attn_decode", 2)


def split3_bf16(w: torch.Tensor) -> torch.Tensor:
    """A float32 tensor as three bfloat16 tensors ``[3, *w.shape]`` whose sum is ``w`` to float32 accuracy
    (each is the bfloat16 rounding of what the ones before leave over)."""
    _want(w, torch.float32, "w")
    w = w.contiguous()
    out = torch.empty((3, *w.shape), dtype=torch.bfloat16, device=w.device)
    _check(lib().qb_split3_bf16(_p(w), _p(out), ctypes.c_longlong(w.numel()), _stream()), "split3_bf16")
    return out


def router_gemm_mma_parts(K: int) -> int:
    """Ranges the inner dimension of ``router_gemm_mma`` is cut into (a function of K alone)."""
    return int(lib().qb_router_gemm_mma_parts(int(K)))


def router_gemm_mma(x: torch.Tensor, pieces: torch.Tensor, logits: torch.Tensor) -> None:
    """``sum_p logits[p, T, E] = x[T, K] @ (pieces[0] + pieces[1] + pieces[2]).T`` in float32 on the tensor
    cores, ``pieces`` from ``split3_bf16`` of the float32 gate; the inner dimension in fixed chunks of 64,
    and in ``router_gemm_mma_parts(K)`` fixed ranges whose sums ``router_topk`` adds in order."""
    T, K = x.shape
    _want(x, torch.bfloat16, "x"); _want(pieces, torch.bfloat16, "pieces"); _want(logits, torch.float32, "logits")
    E = pieces.shape[1]
    parts = router_gemm_mma_parts(K)
    if (pieces.shape[0] != 3 or pieces.shape[2] != K or logits.numel() != parts * T * E
            or not logits.is_contiguous()):
        raise ValueError(f"router_gemm_mma: shape mismatch (logits must be [{parts}, {T}, {E}])")
    _check(lib().qb_router_gemm_mma(_p(x), _p(pieces), _p(logits), T, E, K, _stream()), "router_gemm_mma")


def router_topk(logits, bias, idx_out, w_out, renorm: bool, scale: float) -> None:
    """``logits`` [T, E], or [P, T, E] partial sums that are added in index order first."""
    _want(logits, torch.float32, "logits"); _want(idx_out, torch.int32, "idx_out"); _want(w_out, torch.float32, "w_out")
    n_partials = 1 if logits.dim() == 2 else logits.shape[0]
    T, E = logits.shape[-2:]
    k = idx_out.shape[1]
    if bias is not None:
        _want(bias, torch.float32, "bias")
    _check(lib().qb_router_topk(_p(logits), n_partials, _p(bias), _p(idx_out), _p(w_out), T, E, k, int(renorm),
                                ctypes.c_float(scale), _stream()), "router_topk")


ROUTER_SMALL_MAX_TILE_BYTES = 200 * 1024          # eight token rows must fit the router's shared-memory tile


def router_small_selects(n_tokens: int, n_experts: int, top_k: int) -> bool:
    """Whether ``router_small`` can select and lay the expert plan down in the same launch."""
    return bool(lib().qb_router_small_selects(int(n_tokens), int(n_experts), int(top_k)))


def router_small(x, gate, bias, logits, idx_out=None, w_out=None, renorm: bool = True, scale: float = 1.0, *,
                 counters=None, bm: int = 0, plan=None, sorted_pair=None, tile_expert=None, tile_row0=None,
                 status=None) -> None:
    """Float32 router logits ``logits[T, E] = x[T, K] @ gate[E, K].T`` on the CUDA cores, every logit one sum in
    an order that depends on K alone.  With ``idx_out`` / ``w_out`` / the plan tensors (and
    ``router_small_selects``): the selection (``router_topk``) and the expert plan (``moe_plan``) in the same
    launch; ``counters``: ``1 + ceil(T / 8)`` int32 that are zero before the call and are left zero."""
    _want(gate, torch.float32, "gate"); _want(logits, torch.float32, "logits")
    T, K = x.shape
    E = gate.shape[0]
    if gate.shape[1] != K or tuple(logits.shape) != (T, E):
        raise ValueError("router_small: shape mismatch")
    if 8 * K * x.element_size() > ROUTER_SMALL_MAX_TILE_BYTES:
        raise ValueError(f"router_small: rows of {K} elements do not fit the kernel's shared-memory tile "
                         f"(at most {ROUTER_SMALL_MAX_TILE_BYTES // (8 * x.element_size())})")
    if bias is not None:
        _want(bias, torch.float32, "bias")
    select = idx_out is not None
    k = 0
    if select:
        _want(idx_out, torch.int32, "idx_out"); _want(w_out, torch.float32, "w_out"); _want(counters, torch.int32, "counters")
        k = idx_out.shape[1]
        if not router_small_selects(T, E, k) or counters.numel() < 1 + -(-T // 8):
            raise ValueError("router_small: sizes outside what the selecting form takes, or too few counters")
    _check(lib().qb_router_small(_p(x), _code(x), _p(gate), _p(bias), _p(logits), _p(idx_out), _p(w_out), T, E, K, k,
                                 int(renorm), ctypes.c_float(scale), int(select), _p(counters), int(bm), _p(plan),
                                 _p(sorted_pair), _p(tile_expert), _p(tile_row0),
                                 tile_expert.numel() if tile_expert is not None else 0, _p(status), _stream()),
           "router_small")


MOE_SIMT_BM = 32


def moe_plan_sizes(n_pairs: int, n_experts: int, bm: int) -> tuple[int, int]:
    """(plan words, max tiles) for ``n_pairs`` (token, slot) pairs."""
    return 4 * n_experts + 4, (n_pairs + bm - 1) // bm + min(n_experts, n_pairs)


def moe_plan(idx, n_experts: int, bm: int, plan, sorted_pair, tile_expert, tile_row0, status) -> None:
    n_pairs = idx.numel()
    max_tiles = tile_expert.numel()
    _check(lib().qb_moe_plan(_p(idx), n_pairs, n_experts, bm, _p(plan), _p(sorted_pair), _p(tile_expert),
                             _p(tile_row0), max_tiles, _p(status), _stream()), "moe_plan", 3)


def moe_grouped_simt(mode: int, x, weights, out, sorted_pair, pair_w, plan, tile_expert, tile_row0,
                     n_experts: int, top_k: int) -> None:
    """mode 1: ``out[p, :I] = silu(x[tok] W13_e[:I]^T) * (x[tok] W13_e[I:]^T)``; mode 2:
    ``out[pair] = w[pair] * (x[p] W2_e^T)``; rows p sorted by expert (see ``moe_plan``)."""
    K = x.shape[1]
    N = out.shape[1]
    want = (n_experts, 2 * N, K) if mode == 1 else (n_experts, N, K)
    if tuple(weights.shape) != want:
        raise ValueError(f"moe_grouped: weights {tuple(weights.shape)} != {want}")
    _check(lib().qb_moe_grouped_simt(mode, _p(x), _code(x), _p(weights), _code(weights), _p(out), _code(out),
                                     _p(sorted_pair), _p(pair_w), _p(plan), _p(tile_expert), _p(tile_row0),
                                     tile_expert.numel(), n_experts, top_k, K, N, _stream()), "moe_grouped_simt")


def expert_gemm_tc_supported(x: torch.Tensor, hidden: int, inner: int) -> bool:
    """The tcgen05 expert kernel takes bfloat16 and inner dimensions that are multiples of 8 (16-byte rows
    for TMA)."""
    return x.dtype == torch.bfloat16 and hidden % 8 == 0 and inner % 8 == 0


def expert_tile_rows(n_tokens: int, rows_per_expert: float = 0.0) -> int:
    """Token tile (the MMA's N) of the tcgen05 expert kernel for a step of ``n_tokens`` tokens: an expert
    never receives more rows than there are tokens; from about a hundred rows an expert on average
    (``rows_per_expert``) the products are no longer bound by memory alone, and tiles of 256 rows, which pairs
    of blocks take, read the operands least often (measured on a B200, both products of a layer: 96 rows an
    expert 1,464 against 1,399 us with tiles of 128; 128 rows 1,559 against 1,755 us; 256 rows 2,372 against
    2,889 us; an expert's last tile of a few rows costs the tensor cores only those rows)."""
    for nt in (16, 32, 64):
        if n_tokens <= nt:
            return nt
    big = int(os.environ.get("QUANTA_B200_EXPERT_TILE", "0"))
    if big:
        return big
    return 256 if rows_per_expert >= 112 else 128


def gather_rows(x, out, sorted_pair, top_k: int) -> None:
    """``out[p] = x[sorted_pair[p] // top_k]``: the token rows in expert order, contiguous for TMA."""
    n_pairs, K = out.shape
    _want(x, torch.bfloat16, "x"); _want(out, torch.bfloat16, "out")
    if x.shape[1] != K or sorted_pair.numel() != n_pairs:
        raise ValueError("gather_rows: shape mismatch")
    _check(lib().qb_gather_rows(_p(x), _p(out), _p(sorted_pair), n_pairs, top_k, K, _stream()), "gather_rows")


def expert_gemm_tc(mode: int, x_rows, weights, out, sorted_pair, pair_w, plan, tile_expert, tile_row0,
                   n_experts: int, tile_rows: int, status, gather_top_k: int = 0) -> None:
    """Expert products on tcgen05/TMEM fed by TMA.  ``x_rows`` bf16 [pairs, K] in expert order; mode 1:
    ``out[p, :I] = silu(gate) * up`` (bf16), mode 2: ``out[pair(p)] = w[pair(p)] * down`` (float32).  The plan's
    tile list must have been made with ``bm = tile_rows``.  Mode 1 with ``gather_top_k`` > 0: ``x_rows`` is the
    step's activations [T, K] and the kernel fetches the row of token ``pair // gather_top_k`` itself, one
    TMA box a row (for steps of few tokens: it saves the gathered copy and its launch)."""
    n_x, K = x_rows.shape
    n_pairs = sorted_pair.numel()
    N = out.shape[1]
    want = (n_experts, 2 * N, K) if mode == 1 else (n_experts, N, K)
    if tuple(weights.shape) != want:
        raise ValueError(f"expert_gemm_tc: weights {tuple(weights.shape)} != {want}")
    if gather_top_k == 0 and n_x != n_pairs:
        raise ValueError(f"expert_gemm_tc: {n_x} rows for {n_pairs} pairs")
    _want(x_rows, torch.bfloat16, "x_rows"); _want(weights, torch.bfloat16, "weights")
    _want(out, torch.bfloat16 if mode == 1 else torch.float32, "out")
    _check(lib().qb_expert_gemm_tc(mode, _p(x_rows), _p(weights), _p(out), _p(sorted_pair), _p(pair_w), _p(plan),
                                   _p(tile_expert), _p(tile_row0), tile_expert.numel(), n_pairs, n_experts, K, N,
                                   int(tile_rows), int(gather_top_k), n_x, _p(status), _stream()), "expert_gemm_tc")


# ---- state slots (csrc/request_state.h) ------------------------------------------------------------------
SLOT_WORDS = 16
SLOT_LIVE, SLOT_POSITION, SLOT_PROMPT, SLOT_DRAWN, SLOT_LAST, SLOT_SEED_LO, SLOT_SEED_HI, SLOT_TOP_K = range(8)
SLOT_TEMPERATURE, SLOT_TOP_P, SLOT_MIN_P = 8, 9, 10


def slot_record(*, position: int = 0, prompt_len: int = 0, drawn: int = 0, last: int = 0, seed: int = 0,
                temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0) -> torch.Tensor:
    """A live request's record as int32 ``[SLOT_WORDS]`` on the host (floats as their bit patterns)."""
    import struct

    def bits(x: float) -> int:
        return struct.unpack("<i", struct.pack("<f", float(x)))[0]

    def word(x: int) -> int:
        x &= 0xFFFFFFFF
        return x - (1 << 32) if x >= (1 << 31) else x

    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    rec = [0] * SLOT_WORDS
    rec[SLOT_LIVE], rec[SLOT_POSITION], rec[SLOT_PROMPT], rec[SLOT_DRAWN], rec[SLOT_LAST] = 1, position, prompt_len, drawn, last
    rec[SLOT_SEED_LO], rec[SLOT_SEED_HI], rec[SLOT_TOP_K] = word(seed), word(seed >> 32), int(top_k)
    rec[SLOT_TEMPERATURE], rec[SLOT_TOP_P], rec[SLOT_MIN_P] = bits(temperature), bits(top_p), bits(min_p)
    return torch.tensor(rec, dtype=torch.int32)


def slots_advance(slots, req_slot, req_start, req_len_after, n_requests: int, status) -> None:
    """Move each request's position in its state slot to what it holds after the step; a slot that is free
    or at another position than the step assumes is recorded in ``status``."""
    _want(slots, torch.int32, "slots")
    if slots.dim() != 2 or slots.shape[1] != SLOT_WORDS:
        raise ValueError(f"slots must be [n, {SLOT_WORDS}]")
    _check(lib().qb_slots_advance(_p(slots), slots.shape[0], _p(req_slot), _p(req_start), _p(req_len_after),
                                  int(n_requests), _p(status), _stream()), "slots_advance")


def sample_rows(logits, slots, row_slot, out, all_greedy: bool = False) -> None:
    """One token a row of float32 logits.  ``slots`` int32 ``[n_slots, SLOT_WORDS]`` and ``row_slot`` int32
    ``[n]``: each row's options and draw number come from its slot's record, which then counts the draw and
    holds the token.  ``slots`` None: every row is greedy (first maximum) and nothing is recorded.
    ``all_greedy``: the caller knows every row's temperature is <= 0 (a large vocabulary is then cut over
    many blocks)."""
    _want(logits, torch.float32, "logits"); _want(out, torch.int32, "out")
    n, V = logits.shape
    n_slots = 0
    if slots is not None:
        _want(slots, torch.int32, "slots"); _want(row_slot, torch.int32, "row_slot")
        if slots.dim() != 2 or slots.shape[1] != SLOT_WORDS or row_slot.numel() != n:
            raise ValueError("sample_rows: slots must be [n_slots, SLOT_WORDS] and row_slot [n]")
        n_slots = slots.shape[0]
    if (slots is None or all_greedy) and V >= 4096:
        # all greedy: a row is cut over many blocks, then the first maximum of the chunks is taken
        parts = 32
        sv = torch.empty(n * parts, dtype=torch.float32, device=logits.device)
        si = torch.empty(n * parts, dtype=torch.int32, device=logits.device)
        _check(lib().qb_argmax_rows(_p(logits), n, V, parts, _p(sv), _p(si), _p(slots), _p(row_slot), n_slots, _p(out),
                                    _stream()), "argmax_rows", 2)
        return
    _check(lib().qb_sample_rows(_p(logits), n, V, _p(slots), _p(row_slot), n_slots, _p(out), _stream()), "sample_rows")


def apply_penalties(logits, prev, prev_off, pparams) -> None:
    _want(logits, torch.float32, "logits")
    n, V = logits.shape
    _check(lib().qb_apply_penalties(_p(logits), n, V, _p(prev), _p(prev_off), _p(pparams), _stream()),
           "apply_penalties")
