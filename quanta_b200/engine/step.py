"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step holds, for each scheduled request, a contiguous run of its next tokens: a portion of a prompt
of any size, or one decoded token; all of them are one flat batch.  (The reference never mixes the
two: it prefills one request alone, src/quanta/minimax/batched_runtime_m3.py:409-420, or decodes one
token for each of B requests, :172-187.)  The step reserves pages, packs the small integer arrays
into one pinned buffer, copies it once, runs the model on exactly these tokens, and returns float32
logits at the wanted places.  Nothing inside synchronises with the host.

Steps in which every request brings exactly one token (decoding) are launch-bound when run kernel
by kernel, so they are captured once per (batch size, context bucket) in a CUDA graph and replayed:
the graph reads its integers from a fixed device buffer that each step overwrites.  At most
``max_graphs`` captured steps are kept; the one used longest ago goes when another is captured.

Every live request has a state slot: a row of each mixer's fixed-size state and one record of the
``slots`` array on the device (csrc/request_state.h: live flag, position, prompt length, draws so far,
last sampled token, seed and sampling options).  The record is written when the request is admitted,
every step moves its position (and checks it against the host's), the sampler reads and updates it,
and it is zeroed when the request is freed.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheManager, OutOfPages, OutOfSlots
from ..parts.base import LayerCache, PositionEncoding, StepContext


@dataclass
class StepEntry:
    rid: object
    tokens: list
    want: tuple = ()          # indices into ``tokens`` whose logits are returned
    from_device: bool = False  # a single decode token whose id is the one last sampled into the request's slot


class _DecodeGraph:
    """A captured decode step for one (batch size, context bucket)."""

    def __init__(self):
        self.graph = None
        self.seen = 0             # eager runs at this shape before the capture
        self.dev = None           # the fixed device buffer of the step's integers
        self.logits = None
        self.launches = 0
        self.used_at = 0          # the engine's step count when it last ran


def _fill(host: torch.Tensor, pieces: list) -> None:
    """Lay the step's arrays down one after the other in the pinned buffer."""
    view, off = host.numpy(), 0
    for p in pieces:
        view[off: off + p.size] = p
        off += p.size


class Engine:
    def __init__(self, model, *, num_pages: int, page_size: int = 16, max_requests: int = 64,
                 use_graphs: bool = True, max_graphs: int = 16):
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
        # per cache-writing schedule position: the pages of every stream its mixer declared
        self.kv: dict[int, dict[str, torch.Tensor]] = {}
        for pos, spec in enumerate(needs):
            if spec is not None:
                self.kv[pos] = {st.name: torch.zeros((num_pages, st.heads, page_size, st.width), dtype=model.dtype,
                                                     device=self.device) for st in spec.streams}
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
        # graphs only when every part says its step reads nothing from the host
        self.use_graphs = bool(use_graphs) and all(getattr(p, "graph_safe", False) for p in model.parts())
        self._graphs: dict[tuple[int, int], _DecodeGraph] = {}
        self.max_graphs = max(1, int(max_graphs))
        self._graph_pool = None        # one memory pool for all captured steps: only one of them runs at a time
        self.graph_replays = 0
        # one record per state slot (csrc/request_state.h).  Among other things it holds the token last
        # sampled for the request: a decode step can take its ids from there, so that it can be launched
        # before the host has read them
        self.slots = torch.zeros((max_requests, kernels.SLOT_WORDS), dtype=torch.int32, device=self.device)
        self.manager.on_free = self._slot_freed
        self.last_want_slots = None         # device: the state slot of each row of the logits the last step returned

    # ---- requests -----------------------------------------------------------------------------------
    def admit(self, rid, *, prompt_len: int = 0, params=None, drawn: int = 0) -> int:
        """Give ``rid`` a state slot: its mixer state rows are zeroed and its record is written (one small
        copy).  ``params``: the request's sampling options (an object with temperature, top_k, top_p, min_p,
        seed; None: greedy); ``drawn``: tokens it has sampled before (a request that comes back after it
        was preempted goes on with the next draw number).  ``step`` admits requests it does not know with a
        default record; call this first when the sampler is to read the request's options."""
        slot = self.manager.add_request(rid)
        for per_pos in self.state:
            for t in per_pos.values():
                t[slot].zero_()
        opts = {} if params is None else dict(seed=params.seed, temperature=params.temperature, top_k=params.top_k,
                                                top_p=params.top_p, min_p=params.min_p)
        rec = kernels.slot_record(prompt_len=prompt_len, drawn=drawn, **opts).pin_memory()
        self.slots[slot].copy_(rec, non_blocking=True)
        return slot

    def _slot_freed(self, slot: int) -> None:
        self.slots[slot].zero_()

    def release(self, rid) -> None:
        if self.manager.has(rid):
            self.manager.free(rid)

    def stats(self) -> dict:
        """The cache manager's figures and what the captured decode steps hold."""
        graphs = [g for g in self._graphs.values() if g.graph is not None]
        held = sum(g.logits.numel() * g.logits.element_size() + g.dev.numel() * 4 for g in graphs)
        return {**self.manager.stats(), "graphs": len(graphs), "graph_output_bytes": held,
                "graph_replays": self.graph_replays}

    def check(self) -> None:
        """Read the device status words (synchronises) and raise if a kernel refused an index."""
        st = self.status.cpu()
        if int(st[0]):
            self.status.zero_()
            kernels.raise_on_status(st)

    # ---- the step -------------------------------------------------------------------------------------
    def step(self, entries: list[StepEntry], end=()) -> torch.Tensor | None:
        """Run one batch.  Returns logits ``[wanted, vocab]`` float32 on the device, in the order of the
        entries and of each entry's ``want``; None if nothing is wanted.  The tensor may be overwritten
        by the next step.  ``end`` lists requests that are finished after this step: their pages and
        slot are given back."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        mgr = self.manager
        self.last_want_slots = None
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r}: an entry must bring at least one token")
            if e.from_device and (len(e.tokens) != 1 or not self.decode_graph_ready(len(entries), 0, entries)
                                  or not all(x.from_device for x in entries)):
                raise ValueError(f"request {e.rid!r}: ids come from the device for every request of a captured "
                                 f"decode step, or for none")
            if not e.from_device:
                ids = np.asarray(e.tokens, dtype=np.int64)
                bad = ids[(ids < 0) | (ids >= self.vocab_size)]
                if bad.size:
                    raise ValueError(f"request {e.rid!r}: token id {int(bad[0])} outside the vocabulary of "
                                     f"{self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.rid!r}: wanted place {w} outside its {len(e.tokens)} tokens")
        new = [e.rid for e in entries if not mgr.has(e.rid)]
        if len(new) > mgr.slots.free_count:
            raise OutOfSlots(f"{len(new)} new request(s), {mgr.slots.free_count} free state slots")
        wants = {e.rid: (mgr.length(e.rid) if mgr.has(e.rid) else 0) + len(e.tokens) for e in entries}
        if not mgr.can_reserve(wants):
            raise OutOfPages(f"the step needs more pages than are free: {mgr.stats()['groups']}")
        for rid in new:
            self.admit(rid)
        for rid, n in wants.items():
            mgr.reserve(rid, n)

        logits = None
        if entries:
            if self.use_graphs and all(len(e.tokens) == 1 for e in entries):
                logits = self._run_decode(entries)
            else:
                logits = self._run(entries)
            for e in entries:
                mgr.advance(e.rid, len(e.tokens))
            self.steps += 1
            self.tokens_run += sum(len(e.tokens) for e in entries)
        for rid in end:
            self.release(rid)
        return logits

    # ---- packing the step's integers ---------------------------------------------------------------------
    def _pack(self, entries: list[StepEntry], max_pages: int) -> tuple[list, dict]:
        """The step's integer arrays (int32 numpy), in the fixed order of the device buffer."""
        mgr = self.manager
        rids = [e.rid for e in entries]
        R = len(entries)
        token_ids, tok_pos, tok_req, want_rows, want_slot = [], [], [], [], []
        req_start, req_len_after, req_slot = [0], [], []
        row0 = 0
        for r, e in enumerate(entries):
            base = mgr.length(e.rid)
            n = len(e.tokens)
            token_ids.append(np.asarray(e.tokens, dtype=np.int32))
            tok_pos.append(np.arange(base, base + n, dtype=np.int32))
            tok_req.append(np.full(n, r, dtype=np.int32))
            want_rows.extend(row0 + int(w) for w in e.want)
            want_slot.extend([mgr.slot(e.rid)] * len(e.want))
            row0 += n
            req_start.append(row0)
            req_len_after.append(base + n)
            req_slot.append(mgr.slot(e.rid))
        token_ids, tok_pos, tok_req = np.concatenate(token_ids), np.concatenate(tok_pos), np.concatenate(tok_req)
        tables = [mgr.block_table_matrix(g, rids, max_pages).reshape(-1) for g in range(len(mgr.groups))]
        positions = tok_pos if self.n_axes == 1 else np.repeat(tok_pos, self.n_axes)
        dec_rows = [req_start[r] for r in range(R) if req_start[r + 1] - req_start[r] == 1]
        spans = [(r, req_start[r], req_start[r + 1] - req_start[r]) for r in range(R)
                 if req_start[r + 1] - req_start[r] > 1]
        pieces = [np.asarray(p, dtype=np.int32) for p in (token_ids, tok_pos, tok_req, positions, req_start,
                                                          req_len_after, req_slot, want_rows, want_slot, dec_rows)] + tables
        info = {"req_start": req_start, "req_len_after": req_len_after, "req_slot": req_slot, "spans": spans,
                "n_dec": len(dec_rows), "n_want": len(want_rows)}
        return pieces, info

    def _context(self, dev: torch.Tensor, sizes: list[int], R: int, T: int, max_pages: int, info: dict,
                 max_len_after: int, max_new: int, with_host: bool):
        out, off = [], 0
        for n in sizes:
            out.append(dev[off: off + n])
            off += n
        d_ids, d_pos, d_req, d_positions, d_start, d_len, d_slot, d_want, d_want_slot, d_dec = out[:10]
        d_tables = [t.view(R, max_pages) for t in out[10:]]
        self.last_want_slots = d_want_slot
        ctx = StepContext(
            n_tokens=T, positions=d_positions.view(T, self.n_axes), tok_pos=d_pos, tok_req=d_req, req_slot=d_slot,
            req_start=d_start, req_len_after=d_len, status=self.status, dtype=self.model.dtype,
            max_new_tokens_per_req=max_new, max_len_after=max_len_after,
            host={k: info[k] for k in ("req_start", "req_len_after", "req_slot")} if with_host else {},
            dec_tok=d_dec if info["n_dec"] else None, n_dec=info["n_dec"], spans=info["spans"])
        caches = []
        for pos, entry in enumerate(self.model.schedule):
            src = pos if entry.read_cache_of is None else entry.read_cache_of
            if src in self.kv:
                caches.append(LayerCache(streams=self.kv[src], page_size=self.page_size,
                                         block_table=d_tables[self.manager.group_of[src]],
                                         write=entry.read_cache_of is None))
            else:
                caches.append(None)
        return d_ids, d_want, ctx, caches

    # ---- eager ---------------------------------------------------------------------------------------------
    def _run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        mgr, ps = self.manager, self.page_size
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        max_len_after = max(mgr.length(e.rid) + len(e.tokens) for e in entries)
        max_pages = -(-max_len_after // ps)
        pieces, info = self._pack(entries, max_pages)
        sizes = [int(p.size) for p in pieces]
        total = sum(sizes)
        host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=True)
        _fill(host, pieces)
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = total * 4
        d_ids, d_want, ctx, caches = self._context(dev, sizes, R, T, max_pages, info, max_len_after,
                                                   max(len(e.tokens) for e in entries), with_host=True)
        kernels.slots_advance(self.slots, ctx.req_slot, ctx.req_start, ctx.req_len_after, R, self.status)
        return self.model.forward(d_ids, ctx, caches, self.state, d_want if info["n_want"] else None)

    # ---- decoding through a captured graph ----------------------------------------------------------------------
    @staticmethod
    def _bucket(max_len_after: int) -> int:
        bucket = 512
        while bucket < max_len_after:
            bucket *= 2
        return bucket

    def decode_graph_ready(self, batch: int, max_len_after: int, entries=None) -> bool:
        """Whether a decode step of ``batch`` requests, the longest ``max_len_after`` tokens afterwards,
        replays a captured graph (else it runs eagerly and is captured at its second use)."""
        if not self.use_graphs:
            return False
        if entries is not None:
            max_len_after = max(self.manager.length(e.rid) + 1 for e in entries if self.manager.has(e.rid))
        g = self._graphs.get((batch, self._bucket(max_len_after)))
        return g is not None and g.graph is not None

    def _run_decode(self, entries: list[StepEntry]) -> torch.Tensor | None:
        mgr, ps = self.manager, self.page_size
        B = len(entries)
        max_len_after = max(mgr.length(e.rid) + 1 for e in entries)
        bucket = self._bucket(max_len_after)
        key = (B, bucket)
        g = self._graphs.setdefault(key, _DecodeGraph())
        if g.graph is None and g.seen < 1:
            g.seen += 1
            return self._run(entries)            # first time at this shape: eager (also warms the libraries up)
        max_pages = -(-bucket // ps)
        # every row's logits are computed inside the graph; the wanted ones are picked afterwards
        full = [StepEntry(e.rid, e.tokens, (0,)) for e in entries]
        pieces, info = self._pack(full, max_pages)
        sizes = [int(p.size) for p in pieces]
        total = sum(sizes)
        if g.graph is None:
            g.dev = torch.empty(total, dtype=torch.int32, device=self.device)
        # a fresh pinned buffer every step: the host may run ahead of the device, and the pinned
        # allocator does not hand a block out again before the copy that reads it is done
        host = torch.empty(total, dtype=torch.int32, pin_memory=True)
        _fill(host, pieces)
        g.dev.copy_(host, non_blocking=True)
        self.last_h2d_bytes = total * 4
        slots_at = sum(sizes[:6])            # the req_slot piece
        row_slots = g.dev[slots_at: slots_at + B]
        if entries[0].from_device:
            # ids sampled by the step before, still on the device, in the requests' records
            g.dev[:B].copy_(torch.index_select(self.slots[:, kernels.SLOT_LAST], 0, row_slots))
        if g.graph is None:
            d_ids, d_want, ctx, caches = self._context(g.dev, sizes, B, B, max_pages, info, bucket, 1, with_host=False)
            torch.cuda.synchronize()
            before = kernels.LAUNCHES
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                kernels.slots_advance(self.slots, ctx.req_slot, ctx.req_start, ctx.req_len_after, B, self.status)
                g.logits = self.model.forward(d_ids, ctx, caches, self.state, d_want)
            g.launches = kernels.LAUNCHES - before
            g.graph = graph
            self._drop_old_graphs(keep=key)
        else:
            kernels.LAUNCHES += g.launches
        g.used_at = self.steps
        g.graph.replay()
        self.graph_replays += 1
        want = [r for r, e in enumerate(entries) for _ in e.want]
        if not want:
            self.last_want_slots = None
            return None
        if want == list(range(B)):
            self.last_want_slots = row_slots
            return g.logits
        picked = torch.tensor(want, device=self.device)
        self.last_want_slots = row_slots[picked]
        return g.logits[picked]

    def _drop_old_graphs(self, keep) -> None:
        """Every captured step keeps its logits ([batch, vocab] float32) and its nodes alive; beyond
        ``max_graphs`` the one that ran longest ago is given up (its shape is captured again if it returns)."""
        captured = [k for k, g in self._graphs.items() if g.graph is not None]
        while len(captured) > self.max_graphs:
            oldest = min((k for k in captured if k != keep), key=lambda k: self._graphs[k].used_at)
            del self._graphs[oldest]
            captured.remove(oldest)
