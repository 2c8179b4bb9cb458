"""Grouped-query softmax attention over the paged cache.

Formula, in order (src/quanta/minimax/attention.py:166-204): q/k/v projections without bias; q/k
RMSNorm before the rotation, either over the concatenated heads (``"per_layer"``, weight
``[heads*head_dim]``) or per head (``"per_head"``, weight ``[head_dim]``); rotation of the first
``rotary_dim`` dims by the position encoding part; K (rotated) and V appended to the cache; scores
``q.k * scale`` over the keys at positions <= the query's (and inside the window, if any), softmax in
float32, ``P V``; output projection.  q head ``h`` reads kv head ``h // (n_q / n_kv)``.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import KVCacheSpec, Mixer, TensorSpec, make, register

_NORM_KIND = {None: kernels.NORM_NONE, "per_layer": kernels.NORM_PER_LAYER, "per_head": kernels.NORM_PER_HEAD}


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 position, qk_norm: str | None, qk_norm_eps: float, names: dict, window: int | None = None):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} q heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
        if qk_norm not in _NORM_KIND:
            raise ValueError(f"qk_norm {qk_norm!r} is not None, 'per_layer' or 'per_head'")
        self.hidden, self.nq, self.nkv, self.hd = int(hidden_size), int(n_q_heads), int(n_kv_heads), int(head_dim)
        self.scale, self.qk_norm, self.eps = float(scale), qk_norm, float(qk_norm_eps)
        self.window = window
        self.position = make("position", position) if isinstance(position, tuple) else position
        self.names = dict(names)      # q, k, v, o, and q_norm, k_norm when normed
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        # more q heads per kv head than the single-token kernel takes: single tokens run as portions of one,
        # whose tile list comes from the host each step, so such a model's decode steps are not captured
        self.graph_safe = self.nq // self.nkv <= kernels.ATTN_DECODE_MAX_GROUP

    def children(self):
        return [self.position]

    def tensor_specs(self):
        n, H, hd = self.names, self.hidden, self.hd
        specs = [TensorSpec(n["q"], (self.nq * hd, H)), TensorSpec(n["k"], (self.nkv * hd, H)),
                 TensorSpec(n["v"], (self.nkv * hd, H)), TensorSpec(n["o"], (H, self.nq * hd))]
        if self.qk_norm == "per_layer":
            specs += [TensorSpec(n["q_norm"], (self.nq * hd,), "f32", "gain"),
                      TensorSpec(n["k_norm"], (self.nkv * hd,), "f32", "gain")]
        elif self.qk_norm == "per_head":
            specs += [TensorSpec(n["q_norm"], (hd,), "f32", "gain"), TensorSpec(n["k_norm"], (hd,), "f32", "gain")]
        return specs

    def load(self, fetch):
        n = self.names
        q = fetch(n["q"])
        self.w_qkv = torch.empty(((self.nq + 2 * self.nkv) * self.hd, self.hidden), dtype=q.dtype, device=q.device)
        a, b = self.nq * self.hd, (self.nq + self.nkv) * self.hd
        self.w_qkv[:a].copy_(q)
        del q
        self.w_qkv[a:b].copy_(fetch(n["k"]))
        self.w_qkv[b:].copy_(fetch(n["v"]))
        self.w_o = fetch(n["o"])
        if self.qk_norm is not None:
            self.q_norm_w, self.k_norm_w = fetch(n["q_norm"]), fetch(n["k_norm"])

    def cache_spec(self):
        return KVCacheSpec(self.nkv, self.hd, self.window)

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        qkv = linear(x, self.w_qkv)
        q = torch.empty((T, self.nq, self.hd), dtype=x.dtype, device=x.device)
        tables = self.position.rotary_tables(x.device)
        if tables is None:
            inv_freq = torch.empty(0, dtype=torch.float32, device=x.device)
            pair_axis, rd = None, 0
        else:
            inv_freq, pair_axis, rd, n_axes = tables
            if ctx.positions.dim() != 2 or ctx.positions.shape[1] < n_axes:
                raise ValueError(f"the position encoding reads {n_axes} position axes; the step gives "
                                 f"{tuple(ctx.positions.shape)}")
        kernels.qknorm_rope_write(
            qkv, q, cache.k if cache.write else None, cache.v if cache.write else None, self.q_norm_w,
            self.k_norm_w, _NORM_KIND[self.qk_norm], self.eps, inv_freq, pair_axis, ctx.positions, ctx.tok_pos,
            ctx.tok_req, cache.block_table, self.nq, self.nkv, self.hd, rd, cache.page_size, ctx.status)
        out = empty_rows(T, self.nq, self.hd, dtype=x.dtype, device=x.device)
        self.attend(q, cache, out, ctx)
        return linear(out.view(T, self.nq * self.hd), self.w_o)

    def attend(self, q, cache, out, ctx):
        """float32: the SIMT kernel, every token alike.  bfloat16: tensor-core kernels, one for single
        tokens (the keys of all of them dealt evenly over the SMs) and one for portions (tiles of
        token-by-head rows)."""
        window = self.window or 0
        if q.dtype != torch.bfloat16:
            kernels.paged_attention_simt(q, cache.k, cache.v, out, ctx.tok_pos, ctx.tok_req, cache.block_table,
                                         self.scale, window, ctx.status)
            return
        dec_tok, n_dec, spans = step_work(ctx, q.device)
        G = self.nq // self.nkv
        if n_dec and G > kernels.ATTN_DECODE_MAX_GROUP:
            # more q heads per kv head than the single-token kernel takes: such a token is a portion of one
            starts = ctx.host.get("req_start") or [0, ctx.n_tokens]
            spans = [(r, starts[r], starts[r + 1] - starts[r]) for r in range(len(starts) - 1)]
            n_dec = 0
        if n_dec:
            n_parts = kernels.attn_decode_parts(self.nkv, max(1, ctx.max_len_after))
            part_o = torch.empty(n_dec * self.nq * n_parts * self.hd, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(n_dec * self.nq * n_parts * 2, dtype=torch.float32, device=q.device)
            kernels.attn_decode(q, cache.k, cache.v, out, part_o, part_ml, dec_tok, n_dec, ctx.tok_pos, ctx.tok_req,
                                cache.block_table, self.scale, window, n_parts, ctx.status)
        if spans:
            key = ("span_tiles", G, self.hd, kernels.attn_span_rows(self.hd, self.nq, self.nkv, cache.page_size))
            if key not in ctx.work:
                rows = kernels.attn_span_rows(self.hd, self.nq, self.nkv, cache.page_size)
                tiles = [[r, t0, n, r0] for (r, t0, n) in spans for r0 in range(0, n * G, rows)]
                # tiles that read the most keys first: the short ones fill the SMs at the end
                after = ctx.host.get("req_len_after")
                if after is not None:
                    tiles.sort(key=lambda t: -(after[t[0]] - t[2] + min(t[2], (t[3] + rows) // G)))
                ctx.work[key] = torch.tensor(tiles, dtype=torch.int32).to(q.device, non_blocking=True)
            kernels.attn_span(q, cache.k, cache.v, out, ctx.tok_pos, cache.block_table, ctx.work[key], self.scale,
                              window, ctx.status)


def step_work(ctx, device):
    """(token rows of single-token requests, their number, portions of the other requests)."""
    if ctx.spans is None and ctx.dec_tok is None:
        starts = ctx.host.get("req_start") or [0, ctx.n_tokens]
        dec, spans = [], []
        for r in range(len(starts) - 1):
            n = starts[r + 1] - starts[r]
            (dec.append(starts[r]) if n == 1 else spans.append((r, starts[r], n)))
        ctx.spans, ctx.n_dec = spans, len(dec)
        ctx.dec_tok = torch.tensor(dec, dtype=torch.int32).to(device, non_blocking=True) if dec else None
    return ctx.dec_tok, ctx.n_dec, ctx.spans or []
