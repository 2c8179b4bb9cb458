"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step holds, for each scheduled request, a contiguous run of its next tokens: a portion of a prompt
of any size, or one decoded token; all of them are one flat batch.  (The reference never mixes the
two: it prefills one request alone, src/quanta/minimax/batched_runtime_m3.py:409-420, or decodes one
token for each of B requests, :172-187.)  The step reserves pages, packs the small integer arrays
into one pinned buffer, copies it once, runs the model on exactly these tokens, and returns float32
logits at the wanted places.  Nothing inside synchronises with the host.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels
from ..cache.manager import CacheManager
from ..parts.base import LayerCache, PositionEncoding, StepContext


@dataclass
class StepEntry:
    rid: object
    tokens: list
    want: tuple = ()          # indices into ``tokens`` whose logits are returned


class Engine:
    def __init__(self, model, *, num_pages: int, page_size: int = 16, max_requests: int = 64):
        if not model.loaded:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.device = model.device
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        kernels.lib()                       # build/load the kernels now; fails loudly if that is impossible
        self.page_size = int(page_size)
        needs = model.cache_needs()
        self.manager = CacheManager(needs, page_size, num_pages, max_requests)
        self.kv: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        for pos, spec in enumerate(needs):
            if spec is not None:
                shape = (num_pages, spec.n_kv_heads, page_size, spec.head_dim)
                self.kv[pos] = (torch.zeros(shape, dtype=model.dtype, device=self.device),
                                torch.zeros(shape, dtype=model.dtype, device=self.device))
        self.state: list[dict[str, torch.Tensor]] = []
        for need in model.state_needs():
            self.state.append({name: torch.zeros((max_requests, *shape), dtype=dt, device=self.device)
                               for name, (shape, dt) in need.items()})
        self.status = kernels.new_status(self.device)
        self.n_axes = max([p.n_axes for p in model.parts() if isinstance(p, PositionEncoding)] or [1])
        self.vocab_size = model.spec.vocab_size
        self.steps = 0
        self.tokens_run = 0
        self.last_h2d_bytes = 0

    # ---- requests -----------------------------------------------------------------------------------
    def _admit(self, rid) -> None:
        slot = self.manager.add_request(rid)
        for per_pos in self.state:
            for t in per_pos.values():
                t[slot].zero_()

    def release(self, rid) -> None:
        if self.manager.has(rid):
            self.manager.free(rid)

    def check(self) -> None:
        """Read the device status words (synchronises) and raise if a kernel refused an index."""
        st = self.status.cpu()
        if int(st[0]):
            self.status.zero_()
            kernels.raise_on_status(st)

    # ---- the step -------------------------------------------------------------------------------------
    def step(self, entries: list[StepEntry], end=()) -> torch.Tensor | None:
        """Run one batch.  Returns logits ``[wanted, vocab]`` float32 on the device, in the order of the
        entries and of each entry's ``want``; None if nothing is wanted.  ``end`` lists requests that
        are finished after this step: their pages and slot are given back."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        mgr = self.manager
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r}: an entry must bring at least one token")
            bad = [t for t in e.tokens if not 0 <= int(t) < self.vocab_size]
            if bad:
                raise ValueError(f"request {e.rid!r}: token id {bad[0]} outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.rid!r}: wanted place {w} outside its {len(e.tokens)} tokens")
        new = [e.rid for e in entries if not mgr.has(e.rid)]
        if len(new) > mgr.slots.free_count:
            from ..cache.manager import OutOfSlots
            raise OutOfSlots(f"{len(new)} new request(s), {mgr.slots.free_count} free state slots")
        for rid in new:
            self._admit(rid)
        wants = {e.rid: mgr.length(e.rid) + len(e.tokens) for e in entries}
        if not mgr.can_reserve(wants):
            for rid in new:
                mgr.free(rid)
            from ..cache.manager import OutOfPages
            raise OutOfPages(f"the step needs more pages than are free: {mgr.stats()['groups']}")
        for rid, n in wants.items():
            mgr.reserve(rid, n)

        logits = None
        if entries:
            logits = self._run(entries)
            for e in entries:
                mgr.advance(e.rid, len(e.tokens))
            self.steps += 1
            self.tokens_run += sum(len(e.tokens) for e in entries)
        for rid in end:
            self.release(rid)
        return logits

    def _run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        mgr, ps = self.manager, self.page_size
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        rids = [e.rid for e in entries]
        token_ids, tok_pos, tok_req, want_rows = [], [], [], []
        req_start, req_len_after, req_slot = [0], [], []
        for r, e in enumerate(entries):
            base = mgr.length(e.rid)
            row0 = len(token_ids)
            n = len(e.tokens)
            token_ids.extend(int(t) for t in e.tokens)
            tok_pos.extend(range(base, base + n))
            tok_req.extend([r] * n)
            want_rows.extend(row0 + int(w) for w in e.want)
            req_start.append(row0 + n)
            req_len_after.append(base + n)
            req_slot.append(mgr.slot(e.rid))
        max_len_after = max(req_len_after)
        max_pages = -(-max_len_after // ps)
        tables = []
        for g in range(len(mgr.groups)):
            flat = []
            for row in mgr.block_table_rows(g, rids):
                flat.extend(row[:max_pages])
                flat.extend([-1] * (max_pages - len(row[:max_pages])))
            tables.append(flat)
        positions = tok_pos if self.n_axes == 1 else [p for p in tok_pos for _ in range(self.n_axes)]
        dec_rows = [req_start[r] for r in range(R) if req_start[r + 1] - req_start[r] == 1]
        spans = [(r, req_start[r], req_start[r + 1] - req_start[r]) for r in range(R)
                 if req_start[r + 1] - req_start[r] > 1]
        pieces = [token_ids, tok_pos, tok_req, positions, req_start, req_len_after, req_slot, want_rows, dec_rows,
                  *tables]
        total = sum(len(p) for p in pieces)
        host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=True)
        flat_all = [x for p in pieces for x in p]
        host[:total] = torch.tensor(flat_all, dtype=torch.int32)
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = total * 4
        out, off = [], 0
        for p in pieces:
            out.append(dev[off: off + len(p)])
            off += len(p)
        d_ids, d_pos, d_req, d_positions, d_start, d_len, d_slot, d_want, d_dec = out[:9]
        d_tables = [t.view(R, max_pages) for t in out[9:]]
        ctx = StepContext(
            n_tokens=T, positions=d_positions.view(T, self.n_axes), tok_pos=d_pos, tok_req=d_req, req_slot=d_slot,
            req_start=d_start, req_len_after=d_len, status=self.status, dtype=self.model.dtype,
            max_new_tokens_per_req=max(len(e.tokens) for e in entries), max_len_after=max_len_after,
            host={"req_start": req_start, "req_len_after": req_len_after, "req_slot": req_slot},
            dec_tok=d_dec if dec_rows else None, n_dec=len(dec_rows), spans=spans)
        caches = []
        for pos, entry in enumerate(self.model.schedule):
            src = pos if entry.read_cache_of is None else entry.read_cache_of
            if src in self.kv:
                k, v = self.kv[src]
                caches.append(LayerCache(k, v, ps, d_tables[mgr.group_of[src]], write=entry.read_cache_of is None))
            else:
                caches.append(None)
        return self.model.forward(d_ids, ctx, caches, self.state, d_want if want_rows else None)
