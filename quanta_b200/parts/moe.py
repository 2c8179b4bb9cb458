"""Feed-forward part: sigmoid-routed SwiGLU experts.

Routed experts (src/quanta/minimax/moe.py:36-88): router logits in float32 from a float32 gate;
``sigmoid`` scores; a correction bias added for the choice only; top-k (ties to the lower expert
index); weights are the bias-free scores, renormalised (``+ 1e-20``) and scaled; each chosen expert is
``down(silu(gate x) * up x)`` (``w1`` gate, ``w3`` up, ``w2`` down); the weight is applied after
``down``; the k results are summed in float32 in slot order.  No shared expert.
"""

from __future__ import annotations

import os

import torch

from .. import kernels
from .base import FeedForward, TensorSpec, register


@register("feed_forward", "sigmoid_topk_experts")
class SigmoidTopKExperts(FeedForward):
    """``trace``: a list assigned here receives, for every step, the experts each token chose (int32
    ``[T, k]`` on the device, in choice order), for tools that follow the routing; while it is set the
    part is not graph-safe, so an engine built then runs its decode steps kernel by kernel."""

    @property
    def graph_safe(self):
        return self.trace is None

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top_k: int, use_bias: bool,
                 renormalize: bool, scaling: float, names: dict):
        if top_k > n_experts:
            raise ValueError(f"top_k {top_k} > {n_experts} experts")
        if n_experts > 1024:
            raise ValueError(f"{n_experts} experts: the routing kernels take at most 1024")
        if 8 * 4 * hidden_size > kernels.ROUTER_SMALL_MAX_TILE_BYTES:
            raise ValueError(f"hidden size {hidden_size}: the router kernel stages eight float32 token rows in shared "
                             f"memory and takes at most {kernels.ROUTER_SMALL_MAX_TILE_BYTES // 32} features")
        self.H, self.I, self.E, self.k = int(hidden_size), int(expert_size), int(n_experts), int(top_k)
        self.use_bias, self.renorm, self.scaling = bool(use_bias), bool(renormalize), float(scaling)
        self.names = dict(names)   # gate, bias, and templates w1/w2/w3 with "{e}"
        self.gate_w = self.bias = self.w13 = self.w2 = self.gate_pieces = None
        self.last_counts = None      # rows per expert in the last step (device tensor; for measurements)
        self._plan_counter = None    # the router kernel's counters of finished blocks (zero at rest)
        self.trace = None

    def tensor_specs(self):
        n = self.names
        specs = [TensorSpec(n["gate"], (self.E, self.H), "f32", "normal")]
        if self.use_bias:
            specs.append(TensorSpec(n["bias"], (self.E,), "f32", "bias"))
        for e in range(self.E):
            specs += [TensorSpec(n["w1"].format(e=e), (self.I, self.H)),
                      TensorSpec(n["w3"].format(e=e), (self.I, self.H)),
                      TensorSpec(n["w2"].format(e=e), (self.H, self.I))]
        return specs

    def load(self, fetch):
        n = self.names
        self.gate_w = fetch(n["gate"])
        self.bias = fetch(n["bias"]) if self.use_bias else None
        first = fetch(n["w1"].format(e=0))
        dt, dev = first.dtype, first.device
        # gate rows then up rows of each expert, so one tile of the first product holds both
        self.w13 = torch.empty((self.E, 2 * self.I, self.H), dtype=dt, device=dev)
        self.w2 = torch.empty((self.E, self.H, self.I), dtype=dt, device=dev)
        for e in range(self.E):
            self.w13[e, : self.I].copy_(first if e == 0 else fetch(n["w1"].format(e=e)))
            self.w13[e, self.I:].copy_(fetch(n["w3"].format(e=e)))
            self.w2[e].copy_(fetch(n["w2"].format(e=e)))
        del first
        # prompt portions take their router logits on the tensor cores, from the gate as three bfloat16 pieces
        if dt == torch.bfloat16 and self.H % 8 == 0 and self.gate_w.is_cuda:
            self.gate_pieces = kernels.split3_bf16(self.gate_w)

    # Which kernels run the expert products: "tc" (tcgen05 + TMA) for bfloat16, "simt" (float32 CUDA
    # cores) for float32 and for widths that are no multiple of 8.  QUANTA_B200_EXPERT_KERNELS=simt forces
    # the latter for the whole process (a knob for measurements).
    expert_kernels = os.environ.get("QUANTA_B200_EXPERT_KERNELS", "auto")
    # steps of fewer tokens take their logits on the CUDA cores, in one launch with selection and plan (and the
    # float32 path always); measured on a B200 the two ways cost the same at about a hundred tokens
    router_mma_min_tokens = 96
    # steps with at most this many rows an expert on average fetch the token rows inside the product (one TMA box a
    # row, the producer warp's lanes sharing them) instead of from a gathered copy; measured on a B200 the box a
    # row costs more than the copy from some 12 rows an expert on (300 tokens: 701 against 717 us a layer, 512
    # tokens: 746 against 732 us, 2,048 tokens: 1,358 against 815 us)
    gather_in_kernel_max_rows = 10

    def path_for(self, x) -> str:
        ok16 = kernels.expert_gemm_tc_supported(x, self.H, self.I) and self.w13.dtype == torch.bfloat16
        return "tc" if ok16 and self.expert_kernels != "simt" else "simt"

    def _on_tensor_cores(self, x) -> bool:
        return self.gate_pieces is not None and x.dtype == torch.bfloat16 and x.shape[0] >= self.router_mma_min_tokens

    def router_logits(self, x):
        """float32 ``[T, E]``, or ``[chunks, T, E]`` partial sums that the selection adds in index order."""
        T = x.shape[0]
        if self._on_tensor_cores(x):
            # many tokens: float32-accurate logits on the tensor cores (fixed chunks of the inner dimension)
            logits = torch.empty((kernels.router_gemm_mma_parts(self.H), T, self.E), dtype=torch.float32,
                                 device=x.device)
            kernels.router_gemm_mma(x, self.gate_pieces, logits)
        else:
            # a warp a (token, expert) pair: the order of a logit's additions depends on the width alone
            logits = torch.empty((T, self.E), dtype=torch.float32, device=x.device)
            kernels.router_small(x, self.gate_w, self.bias, logits)
        return logits

    def route(self, x):
        """Router of this part alone: ``(idx int32 [T,k], weights float32 [T,k])``."""
        T = x.shape[0]
        logits = self.router_logits(x)
        idx = torch.empty((T, self.k), dtype=torch.int32, device=x.device)
        w = torch.empty((T, self.k), dtype=torch.float32, device=x.device)
        kernels.router_topk(logits, self.bias, idx, w, self.renorm, self.scaling)
        return idx, w

    def forward(self, x, ctx):
        T = x.shape[0]
        if x.is_cuda and not self._on_tensor_cores(x) and kernels.router_small_selects(T, self.E, self.k):
            # logits, selection and the expert plan in one launch
            return self.experts(x, None, None, ctx)
        idx, w = self.route(x)
        return self.experts(x, idx, w, ctx)

    def experts(self, x, idx, w, ctx):
        """The chosen experts' SwiGLU of every token, weighted: float32 ``[T, k, hidden]``, one slot a choice.
        ``idx`` None: route here, in one launch with the plan."""
        T, dev = x.shape[0], x.device
        n_pairs = T * self.k
        path = self.path_for(x)
        bm = kernels.expert_tile_rows(T, n_pairs / self.E) if path == "tc" else kernels.MOE_SIMT_BM
        plan_words, max_tiles = kernels.moe_plan_sizes(n_pairs, self.E, bm)
        ints = torch.empty(plan_words + n_pairs + 2 * max_tiles, dtype=torch.int32, device=dev)
        plan = ints[:plan_words]
        sorted_pair = ints[plan_words: plan_words + n_pairs]
        tile_expert = ints[plan_words + n_pairs: plan_words + n_pairs + max_tiles]
        tile_row0 = ints[plan_words + n_pairs + max_tiles:]
        if idx is None:
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev)
            idx = torch.empty((T, self.k), dtype=torch.int32, device=dev)
            w = torch.empty((T, self.k), dtype=torch.float32, device=dev)
            if self._plan_counter is None or self._plan_counter.numel() < 1 + -(-T // 8):
                self._plan_counter = torch.zeros(max(64, 1 + -(-T // 8)), dtype=torch.int32, device=dev)
            kernels.router_small(x, self.gate_w, self.bias, logits, idx, w, self.renorm, self.scaling,
                                 counters=self._plan_counter, bm=bm, plan=plan, sorted_pair=sorted_pair,
                                 tile_expert=tile_expert, tile_row0=tile_row0, status=ctx.status)
        else:
            kernels.moe_plan(idx, self.E, bm, plan, sorted_pair, tile_expert, tile_row0, ctx.status)
        self.last_counts = plan[: self.E]
        if self.trace is not None:
            self.trace.append(idx)
        act = torch.empty((n_pairs, self.I), dtype=x.dtype, device=dev)
        y = torch.empty((T, self.k, self.H), dtype=torch.float32, device=dev)
        if path == "tc":
            # bfloat16: TMA-fed tcgen05 products, weights as the 128-row operand, accumulators in TMEM
            if n_pairs <= self.gather_in_kernel_max_rows * self.E:
                # few tokens: the kernel fetches each pair's token row itself
                kernels.expert_gemm_tc(1, x, self.w13, act, sorted_pair, w.view(-1), plan, tile_expert,
                                       tile_row0, self.E, bm, ctx.status, gather_top_k=self.k)
            else:
                xg = torch.empty((n_pairs, self.H), dtype=x.dtype, device=dev)
                kernels.gather_rows(x, xg, sorted_pair, self.k)
                kernels.expert_gemm_tc(1, xg, self.w13, act, sorted_pair, w.view(-1), plan, tile_expert, tile_row0,
                                       self.E, bm, ctx.status)
            kernels.expert_gemm_tc(2, act, self.w2, y.view(n_pairs, self.H), sorted_pair, w.view(-1), plan,
                                   tile_expert, tile_row0, self.E, bm, ctx.status)
        else:
            kernels.moe_grouped_simt(1, x, self.w13, act, sorted_pair, w, plan, tile_expert, tile_row0, self.E, self.k)
            kernels.moe_grouped_simt(2, act, self.w2, y.view(n_pairs, self.H), sorted_pair, w.view(-1), plan,
                                     tile_expert, tile_row0, self.E, self.k)
        return y
